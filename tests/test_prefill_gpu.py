"""GPU parity of the tensor-core (tcgen05/TMEM) forward used for m > 16, against the CPU oracle.

Two kinds of check:
  * integer-valued activations: every product and partial sum is an integer below 2^24, so the
    fp32 result does not depend on summation order or on the bf16 rounding of x, and the kernel
    must match the oracle BIT FOR BIT.  Any error in the swizzled shared-memory layout, the
    descriptors or the digit split shows up here as a mismatch.
  * N(0,1) activations: rounding x to a per-row fixed-point grid (2^-15 of the row's largest
    magnitude, rounded up to a power of two) is the one approximation; results must stay within
    tol_j = 1e-3 * ||x||_inf * scale_j * sum_k |q_jk| (printed per case).
The default kernel is the integer one (tcgen05.mma.kind::i8 on two int8 digit planes of x); the
bf16 kernel (int8 dequantized to bf16 in shared memory) is covered by tests/test_zz_no_alloc.py."""
import os

import numpy as np
import pytest

import oracle

pytestmark = pytest.mark.gpu
BF16 = os.environ.get("NNE_PREFILL", "").startswith("b")  # the bf16 kernel stands in (NNE_PREFILL=bf16)


def layer(nne, ctx, seed, n, k, bias):
    w = oracle.normal(seed, 0, (n, k), 0.0, 0.02)
    b = oracle.normal(seed, 1, (n,), 0.0, 0.1) if bias else None
    ql = nne.QLinear.from_linear(nne.Linear(w, b), ctx)
    qo, so = oracle.quantize_rows(w)
    assert np.array_equal(ql.qweight.reshape(n, k), qo)
    return ql, qo, so, b


def int_activations(seed, m, k, lim=8):
    rng = np.random.default_rng(seed)
    return rng.integers(-lim, lim + 1, size=(m, k)).astype(np.float32)


@pytest.mark.parametrize("n,k,m", [
    (256, 64, 128),      # one tile, one k-block
    (256, 256, 128),     # one tile, four k-blocks (wraps the 3-stage ring)
    (256, 1024, 128),    # many k-blocks
    (512, 512, 256),     # 2 x 2 tiles
    (256, 64, 17),       # smallest m on this path, heavy row padding
    (100, 128, 50),      # n and m tails
    (300, 80, 130),      # k tail (80 = 64 + 16), n tail, m tail
    (1000, 1008, 200),
    (4096, 4096, 384),   # more tiles than SMs: persistent loop + both accumulator buffers
])
def test_integer_activations_bit_exact(nne, ctx, n, k, m):
    ql, qo, so, b = layer(nne, ctx, 300 + n + k, n, k, bias=(n % 3 == 0))
    assert ql.kernel_for(m) == 2
    x = int_activations(n + k + m, m, k)
    y = ql.forward(x)
    ctx.check()
    y_ref = oracle.forward(qo, so, b, x)
    assert np.array_equal(y.view(np.uint32), y_ref.view(np.uint32)), \
        f"mismatch at {np.argwhere(y != y_ref)[:5].tolist()}"


@pytest.mark.parametrize("n,k,m,bias", [(256, 512, 128, True), (768, 2048, 300, False),
                                        (11008, 4096, 128, False), (4096, 11008, 128, True)])
def test_normal_activations_within_tolerance(nne, ctx, n, k, m, bias):
    ql, qo, so, b = layer(nne, ctx, 3, n, k, bias)
    x = oracle.normal(3, 100 + m, (m, k))
    y = ql.forward(x)
    ctx.check()
    y_ref = oracle.forward(qo, so, b, x)
    tol, xinf = oracle.tolerance(qo, so, x)
    err = np.abs(y - y_ref)
    ratio = float((err / tol).max())
    # the same contraction with x put on the kernel's fixed-point grid on the host (per row:
    # rint(x * 2^e) * 2^-e, max|x| * 2^e in [2^14, 2^15), one binade lower where that product
    # would exceed 32639: the top digit has to fit int8) must agree to fp32 accuracy
    mx = np.abs(x).max(axis=1, keepdims=True)
    e = 14 - np.floor(np.log2(mx)).astype(np.int32)
    e = np.where(np.ldexp(mx.astype(np.float64), e) > 32639.0, e - 1, e).astype(np.int32)
    xg = (np.rint(np.ldexp(x.astype(np.float64), e)) * np.ldexp(1.0, -e)).astype(np.float32)
    y_g = oracle.forward(qo, so, b, xg)
    print(f"prefill {k}->{n} M={m}: max|err| {err.max():.3e}, max err/tol {ratio:.3e}, "
          f"rms(y) {np.sqrt((y_ref ** 2).mean()):.3f}, ||x||inf {xinf:.2f}, "
          f"vs grid-rounded-x oracle {np.abs(y - y_g).max():.3e}")
    assert ratio <= 1.0
    if not BF16:  # the bf16 kernel rounds x to bf16, not to this grid
        assert float((np.abs(y - y_g) / tol).max()) <= 2e-3


def test_config3_m2048_sampled_rows(nne, ctx):
    """Config 3 at full size (4096 -> 11008, M = 2048): every row is an independent contraction,
    so 48 sampled rows are checked against the oracle, plus a checksum property over all rows:
    forward(x)[r] must equal the M=1 streaming kernel's result for row r within tolerance."""
    n, k, m = 11008, 4096, 2048
    ql, qo, so, b = layer(nne, ctx, 3, n, k, False)
    x = oracle.normal(3, 2048, (m, k))
    y = ql.forward(x)
    ctx.check()
    rows = np.random.default_rng(0).choice(m, 48, replace=False)
    y_ref = oracle.forward(qo, so, None, x[rows])
    tol, _ = oracle.tolerance(qo, so, x)
    ratio = float((np.abs(y[rows] - y_ref) / tol).max())
    print(f"config3 M=2048 sampled rows: max err/tol {ratio:.3e}")
    assert ratio <= 1.0
    y4 = ql.forward(x[:4])          # streaming fp32 kernel on the first rows
    assert float((np.abs(y[:4] - y4) / tol).max()) <= 1.0
    assert np.isfinite(y).all()


@pytest.mark.parametrize("n,k,m", [(11008, 4096, 512), (4096, 11008, 512), (4096, 11008, 2048),
                                   (11008, 4096, 8192), (4096, 11008, 8192)])
def test_config3_remaining_sizes_sampled_rows(nne, ctx, n, k, m):
    """The other sizes of config 3 (M = 512 and 8192 on both FFN shapes, 11008 -> 4096 at M = 2048):
    activations drawn on the device, the forward through the device entry point, 48 sampled rows
    (first and last included) against the oracle; every row is an independent contraction."""
    import torch
    ql, qo, so, b = layer(nne, ctx, 3, n, k, False)
    assert ql.kernel_for(m) == 2
    gen = torch.Generator(device="cuda")
    gen.manual_seed(3000 + m + n)
    xd = torch.randn(m, k, generator=gen, device="cuda")
    yd = torch.full((m, n), float("nan"), device="cuda")
    ql.forward_device(xd.data_ptr(), m, yd.data_ptr(), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    ctx.check()
    rows = np.unique(np.concatenate([[0, m - 1], np.random.default_rng(m).choice(m, 46, replace=False)]))
    idx = torch.from_numpy(rows).cuda()
    x = xd[idx].cpu().numpy()
    y = yd[idx].cpu().numpy()
    y_ref = oracle.forward(qo, so, None, x)
    xinf_all = float(xd.abs().max())
    tol, _ = oracle.tolerance(qo, so, x)
    err = np.abs(y - y_ref)
    ratio = float((err / tol).max())
    rms = float(np.sqrt((y_ref.astype(np.float64) ** 2).mean()))
    print(f"config3 {k}->{n} M={m}: 48 sampled rows, max|err| {err.max():.3e}, max err/tol {ratio:.3e}, "
          f"max|err|/rms(y) {err.max() / rms:.3e}, ||x||inf {xinf_all:.2f}")
    assert ratio <= 1.0
    assert bool(torch.isfinite(yd).all())


def test_dominant_activation_on_the_prefill_grid(nne, ctx):
    """One element of a row 500 times larger than the rest (LLM activations have such outliers): the
    prefill kernel's fixed-point grid is per ROW, 2^-15 of the row's power-of-two ceiling, so the
    small elements of that row lose most of their bits.  The result stays inside the tolerance by
    construction (it scales with ||x||inf); the tight number, max|err| / rms(y), is printed."""
    n, k, m = 1024, 4096, 64
    ql, qo, so, b = layer(nne, ctx, 8, n, k, False)
    x = oracle.normal(8, 1, (m, k))
    x[5, 100] = 500.0
    x[40, 7] = -3000.0
    y = ql.forward(x)
    ctx.check()
    y_ref = oracle.forward(qo, so, None, x)
    y64 = oracle.forward_f64(qo, so, None, x)
    for r in (5, 40, 0):
        tol_r, _ = oracle.tolerance(qo, so, x[r:r + 1])
        err = np.abs(y[r] - y_ref[r])
        rms = float(np.sqrt((y64[r] ** 2).mean()))
        print(f"prefill row {r} (max|x| {np.abs(x[r]).max():.0f}): max|err| {err.max():.3e}, "
              f"max err/tol {float((err / tol_r).max()):.3e}, max|err|/rms(y) {err.max() / rms:.3e}")
        assert float((err / tol_r).max()) <= 1.0


def test_strided_output_and_device_entry(nne, ctx):
    import torch
    n, k, m = 512, 256, 160
    ql, qo, so, b = layer(nne, ctx, 5, n, k, True)
    x = int_activations(9, m, k)
    xd = torch.from_numpy(x).cuda()
    wide = torch.full((m, 1536), -3.0, device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    ql.forward_device(xd.data_ptr(), m, wide.data_ptr() + 4 * 512, s, ldy=1536)
    torch.cuda.synchronize()
    ctx.check()
    y_ref = oracle.forward(qo, so, b, x)
    assert np.array_equal(wide[:, 512:1024].cpu().numpy(), y_ref)
    assert bool((wide[:, :512] == -3.0).all()) and bool((wide[:, 1024:] == -3.0).all())


def test_m_between_gemv_and_tile(nne, ctx):
    ql, qo, so, b = layer(nne, ctx, 6, 384, 192, True)
    for m in (17, 31, 64, 127, 129):
        x = int_activations(m, m, 192)
        y = ql.forward(x)
        assert np.array_equal(y, oracle.forward(qo, so, b, x))
    ctx.check()


def test_rows_with_nonfinite_activations_yield_nan(nne, ctx):
    ql, qo, so, b = layer(nne, ctx, 7, 256, 256, True)
    x = oracle.normal(7, 9, (40, 256))
    x[3, 17] = np.inf
    x[9, 0] = np.nan
    y = ql.forward(x)
    if BF16:  # the bf16 kernel propagates Inf through the MMA: +-Inf or NaN, never a finite value
        assert not np.isfinite(y[3]).any() and np.isnan(y[9]).all()
    else:
        assert np.isnan(y[3]).all() and np.isnan(y[9]).all()
    ok = np.ones(40, bool); ok[[3, 9]] = False
    y_ref = oracle.forward(qo, so, b, x[ok])
    tol, _ = oracle.tolerance(qo, so, x[ok])
    assert float((np.abs(y[ok] - y_ref) / tol).max()) <= 1.0
