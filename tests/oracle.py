"""ctypes access to the CPU oracle (oracle/qlinear_ref.c) for the tests, the smoke check and the
benchmark's CPU-baseline leg.  Test infrastructure only: the product never imports this."""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")
LIB_PATH = os.path.join(ORACLE_DIR, "_build", "libqlinear_ref.so")

_lib = None


def build(force: bool = False) -> str:
    src = os.path.join(ORACLE_DIR, "qlinear_ref.c")
    stale = (not os.path.exists(LIB_PATH)) or os.path.getmtime(LIB_PATH) < os.path.getmtime(src)
    if force or stale:
        subprocess.run(["make", "-C", ORACLE_DIR], check=True, capture_output=True)
    return LIB_PATH


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        l = C.CDLL(LIB_PATH)
        vp, sz = C.c_void_p, C.c_size_t
        l.nne_ref_fill_normal.argtypes = [C.c_uint64, C.c_uint64, C.c_double, C.c_double, sz, vp]
        l.nne_ref_fill_normal.restype = None
        l.nne_ref_int8tensor_from_raw.argtypes = [vp, sz, vp, vp]
        l.nne_ref_int8tensor_from_raw.restype = None
        l.nne_ref_dequantize.argtypes = [vp, sz, C.c_float, vp]
        l.nne_ref_dequantize.restype = None
        l.nne_ref_quantize_rows.argtypes = [vp, sz, sz, vp, vp]
        l.nne_ref_quantize_rows.restype = None
        l.nne_ref_to_linear.argtypes = [vp, vp, sz, sz, vp]
        l.nne_ref_to_linear.restype = None
        l.nne_ref_qlinear_memory_bytes.argtypes = [sz, sz, C.c_int]
        l.nne_ref_qlinear_memory_bytes.restype = sz
        l.nne_ref_dot_f32_i8_scalar.argtypes = [vp, vp, sz]
        l.nne_ref_dot_f32_i8_scalar.restype = C.c_float
        l.nne_ref_dot_f32_i8_avx2.argtypes = [vp, vp, sz]
        l.nne_ref_dot_f32_i8_avx2.restype = C.c_float
        l.nne_ref_has_avx2_fma.argtypes = []
        l.nne_ref_has_avx2_fma.restype = C.c_int
        l.nne_ref_forward.argtypes = [vp, vp, vp, sz, sz, vp, sz, vp, C.c_int, C.c_int]
        l.nne_ref_forward.restype = C.c_int
        l.nne_ref_forward_f64.argtypes = [vp, vp, vp, sz, sz, vp, sz, vp]
        l.nne_ref_forward_f64.restype = None
        l.nne_ref_tolerance.argtypes = [vp, vp, sz, sz, vp, sz, vp]
        l.nne_ref_tolerance.restype = C.c_float
        l.nne_ref_rms_norm.argtypes = [vp, vp, C.c_float, sz, sz, vp, C.c_int]
        l.nne_ref_rms_norm.restype = None
        l.nne_ref_silu_mul.argtypes = [vp, vp, sz, vp]
        l.nne_ref_silu_mul.restype = None
        _lib = l
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def normal(seed: int, stream: int, shape, mean: float = 0.0, std: float = 1.0) -> np.ndarray:
    """Seeded N(mean, std) f32 array from the oracle's counter-based generator."""
    out = np.empty(shape, dtype=np.float32)
    lib().nne_ref_fill_normal(seed, stream, mean, std, out.size, _p(out))
    return out


def quantize_rows(w: np.ndarray):
    w = np.ascontiguousarray(w, dtype=np.float32)
    rows, cols = w.shape
    q = np.empty((rows, cols), dtype=np.int8)
    s = np.empty(rows, dtype=np.float32)
    lib().nne_ref_quantize_rows(_p(w), rows, cols, _p(q), _p(s))
    return q, s


def int8tensor_from_raw(v: np.ndarray):
    v = np.ascontiguousarray(v, dtype=np.float32)
    q = np.empty(v.size, dtype=np.int8)
    s = np.empty(1, dtype=np.float32)
    lib().nne_ref_int8tensor_from_raw(_p(v), v.size, _p(q), _p(s))
    return q.reshape(v.shape), np.float32(s[0])


def dequantize(q: np.ndarray, scale) -> np.ndarray:
    q = np.ascontiguousarray(q, dtype=np.int8)
    out = np.empty(q.shape, dtype=np.float32)
    lib().nne_ref_dequantize(_p(q), q.size, float(scale), _p(out))
    return out


def to_linear(q: np.ndarray, scales: np.ndarray) -> np.ndarray:
    q = np.ascontiguousarray(q, dtype=np.int8)
    rows, cols = q.shape
    out = np.empty((rows, cols), dtype=np.float32)
    lib().nne_ref_to_linear(_p(q), _p(np.ascontiguousarray(scales, dtype=np.float32)), rows, cols,
                            _p(out))
    return out


def forward(q, scales, bias, x, threads: int = 0, use_avx2: int = -1) -> np.ndarray:
    """Reference-order f32 forward.  threads=0 -> one thread per input row up to the core count,
    which is all the parallelism the reference's row split offers."""
    q = np.ascontiguousarray(q, dtype=np.int8)
    n, k = q.shape
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, k)
    m = x.shape[0]
    y = np.empty((m, n), dtype=np.float32)
    if threads <= 0:
        threads = max(1, min(m, os.cpu_count() or 1))
    s = np.ascontiguousarray(scales, dtype=np.float32)
    b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
    lib().nne_ref_forward(_p(q), _p(s), _p(b), n, k, _p(x), m, _p(y), threads, use_avx2)
    return y


def forward_f64(q, scales, bias, x) -> np.ndarray:
    q = np.ascontiguousarray(q, dtype=np.int8)
    n, k = q.shape
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, k)
    y = np.empty((x.shape[0], n), dtype=np.float64)
    s = np.ascontiguousarray(scales, dtype=np.float32)
    b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
    lib().nne_ref_forward_f64(_p(q), _p(s), _p(b), n, k, _p(x), x.shape[0], _p(y))
    return y


def tolerance(q, scales, x):
    """tol_j = 1e-3 * ||x||_inf * scale_j * sum_k |q_jk|; returns (tol[n], ||x||_inf)."""
    q = np.ascontiguousarray(q, dtype=np.int8)
    n, k = q.shape
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, k)
    tol = np.empty(n, dtype=np.float32)
    s = np.ascontiguousarray(scales, dtype=np.float32)
    xinf = lib().nne_ref_tolerance(_p(q), _p(s), n, k, _p(x), x.shape[0], _p(tol))
    return tol, float(xinf)


def rms_norm(x, gamma, eps: float = 1e-6, use_avx2: int = -1) -> np.ndarray:
    """RMSNorm::forward (src/nn/norm.rs:141-165) over the last dimension."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    d = x.shape[-1]
    out = np.empty_like(x)
    g = np.ascontiguousarray(gamma, dtype=np.float32)
    lib().nne_ref_rms_norm(_p(x), _p(g), eps, x.size // d if d else 0, d, _p(out), use_avx2)
    return out


def silu_mul(gate, up) -> np.ndarray:
    """silu(gate) * up, the element-wise step of SwiGLU (src/models/llama.rs:343-346)."""
    g = np.ascontiguousarray(gate, dtype=np.float32)
    u = np.ascontiguousarray(up, dtype=np.float32)
    out = np.empty_like(g)
    lib().nne_ref_silu_mul(_p(g), _p(u), g.size, _p(out))
    return out


# ---- independent numpy restatement of the quantize step (src/nn/quantized.rs:107-127) ---------
def numpy_quantize_rows(w: np.ndarray):
    """Written separately from the C oracle: f32 ops in numpy, the half-away rounding done in
    float64 where t + 0.5 is exact.  Used to cross-check the C oracle byte for byte."""
    w = np.asarray(w, dtype=np.float32)
    a = np.abs(w)
    a = np.where(np.isnan(a), np.float32(0), a)
    max_abs = a.max(axis=1) if w.shape[1] else np.zeros(w.shape[0], np.float32)
    with np.errstate(divide="ignore", invalid="ignore", over="ignore"):
        scale = np.where(max_abs > 0, max_abs / np.float32(127.0), np.float32(1.0)).astype(np.float32)
        inv = (np.float32(1.0) / scale).astype(np.float32)
        t = (w * inv[:, None]).astype(np.float32)
        t64 = t.astype(np.float64)
        r = np.sign(t64) * np.floor(np.abs(t64) + 0.5)
        r = np.where(np.isnan(r), 0.0, np.clip(r, -128.0, 127.0))
    return r.astype(np.int8), scale


# ---- independent numpy restatement of the forward's AVX2 dot product ---------------------------
def _fma_f32(a: np.ndarray, b: np.ndarray, c: np.ndarray) -> np.ndarray:
    """Correctly rounded f32 fused multiply-add, element-wise, without an FMA instruction: the
    product of two f32 is exact in f64; the f64 sum with c is taken with its rounding error
    (TwoSum) and, when inexact, moved to the neighbour with an odd last bit ("round to odd"), after
    which the rounding to f32 is the rounding of the exact value (f64 has more than two spare bits)."""
    p = a.astype(np.float64) * b.astype(np.float64)
    c64 = c.astype(np.float64)
    with np.errstate(over="ignore", invalid="ignore"):
        s = p + c64
        bb = s - p
        err = (p - (s - bb)) + (c64 - bb)
        inexact = np.isfinite(s) & (err != 0)
        even = (s.view(np.int64) & 1) == 0
        toward = np.where(err > 0, np.inf, -np.inf)
        s = np.where(inexact & even, np.nextafter(s, toward), s)
        return s.astype(np.float32)


def numpy_dot_f32_i8_avx2(x: np.ndarray, w: np.ndarray) -> np.float32:
    """dot_f32_i8_avx2 (src/nn/quantized.rs:276-324), written from the Rust source and not from the
    C oracle: element i of a 16-block goes to lane i % 16 of two 8-lane accumulators updated by
    fmadd (:299-300); then acc0 + acc1 (:305), low half + high half (:308-310), the pairwise
    movehdup / movehl sums (:311-314) and the scalar tail with a separate multiply and add (:318-321)."""
    x = np.asarray(x, dtype=np.float32)
    wf = np.asarray(w, dtype=np.int8).astype(np.float32)          # cvtepi8_epi32 + cvtepi32_ps: exact
    n = x.size
    blocks = n // 16
    acc = np.zeros(16, dtype=np.float32)                          # lanes 0-7: acc0, lanes 8-15: acc1
    xb = x[:blocks * 16].reshape(blocks, 16)
    wb = wf[:blocks * 16].reshape(blocks, 16)
    for b in range(blocks):
        acc = _fma_f32(xb[b], wb[b], acc)
    a8 = acc[:8] + acc[8:]                                         # _mm256_add_ps(acc0, acc1)
    s4 = a8[:4] + a8[4:]                                           # lo128 + hi128
    sums0 = s4[0] + s4[1]                                          # sum128 + movehdup: lanes 0 and 2
    sums2 = s4[2] + s4[3]
    total = np.float32(sums0 + sums2)                              # add_ss(sums, movehl(sums, sums))
    for i in range(blocks * 16, n):
        total = np.float32(total + np.float32(x[i] * wf[i]))
    return total


def numpy_forward_avx2(q, scales, bias, x) -> np.ndarray:
    """QLinear::forward_quantized (src/nn/quantized.rs:176-193) over numpy_dot_f32_i8_avx2: dot, then
    val = dot * scale, then val += bias as separate f32 operations.  Small cases only (Python loops)."""
    q = np.asarray(q, dtype=np.int8)
    x = np.asarray(x, dtype=np.float32).reshape(-1, q.shape[1])
    s = np.asarray(scales, dtype=np.float32)
    y = np.empty((x.shape[0], q.shape[0]), dtype=np.float32)
    for r in range(x.shape[0]):
        for j in range(q.shape[0]):
            val = np.float32(numpy_dot_f32_i8_avx2(x[r], q[j]) * s[j])
            if bias is not None:
                val = np.float32(val + np.float32(bias[j]))
            y[r, j] = val
    return y
