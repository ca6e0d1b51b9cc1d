"""GPU parity of the quantize / dequantize kernels against the CPU oracle, through the C ABI.
Codes and scales must be bit-exact (reference src/nn/quantized.rs:32-57, :107-127)."""
import os

import numpy as np
import pytest

import oracle

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "qlinear_golden.npz")


def bits(a):
    return np.asarray(a, dtype=np.float32).view(np.uint32)


def gpu_quantize_rows(nne, ctx, w):
    import ctypes as C
    w = np.ascontiguousarray(w, dtype=np.float32)
    rows, cols = w.shape
    q = np.empty((rows, cols), np.int8)
    s = np.empty(rows, np.float32)
    vp = lambda a: a.ctypes.data_as(C.c_void_p)
    st = nne.load().nne_quantize_rows(ctx.handle, vp(w), rows, cols, vp(q), vp(s))
    assert st == 0
    return q, s


def test_golden_rows_bit_exact(nne, ctx):
    g = np.load(GOLDEN)
    q, s = gpu_quantize_rows(nne, ctx, g["w"])
    assert np.array_equal(q, g["q"])
    assert np.array_equal(bits(s), bits(g["scales"]))


def test_rounding_known_answers_on_gpu(nne, ctx):
    row = np.array([[127.0, 0.5, -0.5, 1.5, -1.5, 2.5, -2.5, 126.5, -126.5, 0.49999997, -0.49999997,
                     1.0, -0.0, 63.5]], dtype=np.float32)
    q, s = gpu_quantize_rows(nne, ctx, row)
    assert s[0] == np.float32(1.0)
    assert q[0].tolist() == [127, 1, -1, 2, -2, 3, -3, 127, -127, 0, 0, 1, 0, 64]


@pytest.mark.parametrize("rows,cols", [(1, 1), (3, 7), (5, 15), (2, 17), (7, 31), (128, 64),
                                       (64, 1024), (33, 1028), (9, 1030), (16, 4096),
                                       (3, 11008), (2, 28672), (2, 70001), (1, 131072)])
def test_rows_match_oracle(nne, ctx, rows, cols):
    w = oracle.normal(40, rows * 100003 + cols, (rows, cols), 0.0, 0.02)
    q, s = gpu_quantize_rows(nne, ctx, w)
    qo, so = oracle.quantize_rows(w)
    assert np.array_equal(q, qo)
    assert np.array_equal(bits(s), bits(so))


def test_edge_rows_on_gpu(nne, ctx):
    cols = 2048  # long enough for the one-CTA-per-row kernel
    with np.errstate(all="ignore"):
        w = oracle.normal(41, 0, (8, cols), 0.0, 0.02)
        w[0] = 0.0
        w[1, 100] = np.nan
        w[2, 7] = np.inf
        w[2, 9] = -np.inf
        w[3] = (oracle.normal(41, 1, (cols,)) * np.float32(1e-42)).astype(np.float32)
        w[4] = 0.0
        w[4, 0] = 1e-44
        w[4, 1] = -1e-45
        w[5] = oracle.normal(41, 2, (cols,), 0.0, 3e38)
        qo, so = oracle.quantize_rows(w)
    q, s = gpu_quantize_rows(nne, ctx, w)
    assert np.array_equal(q, qo)
    assert np.array_equal(bits(s), bits(so))
    assert s[0] == 1.0 and q[1, 100] == 0 and np.isinf(s[2]) and not q[2].any()
    assert s[4] == 0.0 and q[4, 0] == 127 and q[4, 1] == -128


def test_config1_codes_bit_exact(nne, ctx):
    """Config 1: 4096x4096 weights ~ N(0, 0.02), seed 0."""
    w = oracle.normal(0, 0, (4096, 4096), 0.0, 0.02)
    q, s = gpu_quantize_rows(nne, ctx, w)
    qo, so = oracle.quantize_rows(w)
    assert np.array_equal(q, qo)
    assert np.array_equal(bits(s), bits(so))
    # how many codes the wrong rounding modes would have flipped on this very matrix
    inv = (np.float32(1.0) / so).astype(np.float32)
    t = (w * inv[:, None]).astype(np.float32)
    ties = int((np.abs(t - np.trunc(t)) == 0.5).sum())
    print(f"config 1: exact .5 ties = {ties}")


def test_empty_shapes(nne, ctx):
    q, s = gpu_quantize_rows(nne, ctx, np.zeros((0, 16), np.float32))
    assert q.size == 0 and s.size == 0
    q, s = gpu_quantize_rows(nne, ctx, np.zeros((3, 0), np.float32))
    assert q.size == 0 and s.tolist() == [1.0, 1.0, 1.0]


@pytest.mark.parametrize("shape", [(32, 64), (1,), (5,), (3, 5, 7), (1000003,), (4096, 1024)])
def test_int8tensor_from_raw_and_dequantize(nne, ctx, shape):
    raw = oracle.normal(42, int(np.prod(shape)), shape)
    t = nne.Int8Tensor.from_raw(raw, ctx)
    qo, so = oracle.int8tensor_from_raw(raw)
    assert t.shape == list(shape) and t.data.size == raw.size
    assert np.array_equal(t.data.reshape(shape), qo)
    assert bits(t.scale) == bits(so)
    deq = t.dequantize(ctx)
    assert deq.shape == raw.shape
    assert np.array_equal(bits(deq), bits(oracle.dequantize(qo, so)))
    assert t.memory_bytes() == raw.size + 56


def test_int8tensor_edge_values(nne, ctx):
    with np.errstate(all="ignore"):
        for vals in ([0.0, 0.0, 0.0], [np.nan, 1.0, -3.0], [np.inf, 1.0], [1e-44, -1e-45, 0.0]):
            raw = np.array(vals, np.float32)
            t = nne.Int8Tensor.from_raw(raw, ctx)
            qo, so = oracle.int8tensor_from_raw(raw)
            assert np.array_equal(t.data, qo) and bits(t.scale) == bits(so)


def test_quantize_linearity_property_full_size(nne, ctx):
    """Size-independent property at a 70B-shaped row count: scaling a row by a power of two
    scales its scale by the same factor and leaves every code unchanged."""
    w = oracle.normal(43, 0, (64, 28672), 0.0, 0.015)
    q1, s1 = gpu_quantize_rows(nne, ctx, w)
    q2, s2 = gpu_quantize_rows(nne, ctx, w * np.float32(4.0))
    assert np.array_equal(q1, q2)
    assert np.array_equal(bits(s1 * np.float32(4.0)), bits(s2))
    assert np.abs(q1).max(axis=1).min() == 127  # every row reaches full scale
