"""GPU parity of QLinear::forward (reference src/nn/quantized.rs:146-197) against the CPU
oracle, through the C ABI and the host mirror.

Tolerance (stated per case, printed with the measured error): per output channel j
    tol_j = 1e-3 * ||x||_inf * scale_j * sum_k |q_jk|
i.e. one thousandth of the a-priori bound on |y_j - b_j|.  The decode kernels (activations on a
16-bit grid, exact integer sums) are also held to 2 % of tol_j on these random inputs - their
worst case is 3 % -; the prefill kernel (same grid, larger batches) is held to tol_j."""
import numpy as np
import pytest

import oracle

pytestmark = pytest.mark.gpu


def make_layer(nne, ctx, seed, n, k, bias=True, std=0.02):
    w = oracle.normal(seed, 0, (n, k), 0.0, std)
    b = oracle.normal(seed, 1, (n,), 0.0, 0.1) if bias else None
    ql = nne.QLinear.from_linear(nne.Linear(w, b), ctx)
    qo, so = oracle.quantize_rows(w)
    assert np.array_equal(ql.qweight.reshape(n, k), qo)
    assert np.array_equal(ql.scales.view(np.uint32), so.view(np.uint32))
    return ql, qo, so, b


def check_forward(ql, qo, so, b, x, label, tight=True):
    y = ql.forward(x)
    x2 = x.reshape(-1, x.shape[-1])
    y_ref = oracle.forward(qo, so, b, x2).reshape(y.shape)
    y64 = oracle.forward_f64(qo, so, b, x2).reshape(y.shape)
    tol, xinf = oracle.tolerance(qo, so, x2)
    err = np.abs(y.astype(np.float64) - y_ref.astype(np.float64)).reshape(-1, tol.size)
    err64 = np.abs(y.astype(np.float64) - y64).reshape(-1, tol.size)
    ratio = float((err / np.maximum(tol, 1e-30)).max()) if err.size else 0.0
    rms = float(np.sqrt(np.mean(y64 ** 2))) if y64.size else 0.0
    print(f"{label}: max|err| vs reference order {err.max() if err.size else 0:.3e}, "
          f"vs f64 {err64.max() if err64.size else 0:.3e}, max err/tol {ratio:.3e}, "
          f"tol min {tol.min() if tol.size else 0:.3e}, ||x||inf {xinf:.3f}, rms(y) {rms:.3f}")
    assert ratio <= 1.0, f"{label}: outside tolerance (max err/tol = {ratio})"
    if tight:
        assert ratio <= 2e-2, f"{label}: fp32 path should be far inside tolerance ({ratio})"
    return y


def test_golden_forward(nne, ctx):
    import os
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden",
                             "qlinear_golden.npz"))
    n = int(g["n_forward"])
    ql = nne.QLinear.from_fields(g["q"][:n].reshape(-1), g["scales"][:n], g["bias"][:n],
                                 g["q"].shape[1], n, ctx)
    y = ql.forward(g["x"])
    assert np.abs(y - g["y_avx2"]).max() < 2e-5
    assert np.abs(y - g["y_f64"]).max() < 2e-5
    ql2 = nne.QLinear.from_fields(g["q"][:n].reshape(-1), g["scales"][:n], None,
                                  g["q"].shape[1], n, ctx)
    assert np.abs(ql2.forward(g["x"]) - g["y_nobias"]).max() < 2e-5


def test_config1(nne, ctx):
    """Config 1: 4096 -> 4096, W ~ N(0,0.02) seed 0, zero bias, x [1,4096] ~ N(0,1) seed 1."""
    w = oracle.normal(0, 0, (4096, 4096), 0.0, 0.02)
    b = np.zeros(4096, np.float32)
    x = oracle.normal(1, 0, (1, 4096))
    ql = nne.QLinear.from_linear(nne.Linear(w, b), ctx)
    qo, so = oracle.quantize_rows(w)
    assert np.array_equal(ql.qweight.reshape(4096, 4096), qo)
    assert np.array_equal(ql.scales.view(np.uint32), so.view(np.uint32))
    assert ql.kernel_for(1) == 1
    check_forward(ql, qo, so, b, x, "config1 4096x4096 M=1")


@pytest.mark.parametrize("n,k", [(4096, 4096), (11008, 4096), (4096, 11008)])
def test_config2_decode_sweep(nne, ctx, n, k):
    """Config 2: LLaMA-2-7B projections, seed 2, M in {1,2,4,8,16}."""
    ql, qo, so, b = make_layer(nne, ctx, 2 + 1000 * (n // 64) + k, n, k, bias=False)
    for m in (1, 2, 4, 8, 16):
        x = oracle.normal(2, 100 + m, (m, k))
        check_forward(ql, qo, so, None, x, f"config2 {k}->{n} M={m}")


@pytest.mark.parametrize("n,k,m", [(1, 16, 1), (3, 16, 2), (5, 32, 3), (8, 48, 5), (17, 64, 7),
                                   (64, 128, 1), (128, 64, 8), (1000, 1008, 3), (257, 8192, 2),
                                   (130, 14336, 4), (66, 28672, 1), (34, 28672, 3),
                                   (31, 32768, 1), (9, 40000, 2)])
def test_streaming_kernel_shapes(nne, ctx, n, k, m):
    ql, qo, so, b = make_layer(nne, ctx, 50 + n + k, n, k, bias=(n % 2 == 0))
    x = oracle.normal(51, n * 7 + k + m, (m, k))
    check_forward(ql, qo, so, b, x, f"stream {k}->{n} M={m}")


@pytest.mark.parametrize("n,k,m", [(1, 1, 1), (3, 7, 1), (2, 15, 3), (5, 17, 17), (4, 31, 2),
                                   (7, 100, 5), (33, 1001, 9)])
def test_generic_kernel_shapes(nne, ctx, n, k, m):
    """k not a multiple of 16: the any-shape kernel."""
    ql, qo, so, b = make_layer(nne, ctx, 60 + n + k, n, k, bias=(k % 2 == 1))
    assert ql.kernel_for(m) == 3
    x = oracle.normal(61, n + k + m, (m, k))
    check_forward(ql, qo, so, b, x, f"generic {k}->{n} M={m}")


def test_errors_and_shapes(nne, ctx):
    ql, qo, so, b = make_layer(nne, ctx, 70, 128, 64)
    with pytest.raises(nne.InvalidArgument):
        ql.forward(np.zeros(64, np.float32))
    with pytest.raises(nne.ShapeMismatch) as e:
        ql.forward(np.zeros((2, 65), np.float32))
    assert e.value.expected == [64] and e.value.actual == [65]
    # 3-D input flattens its leading dims (reference :164) and keeps them in the output
    x3 = oracle.normal(71, 0, (4, 10, 64))
    y3 = check_forward(ql, qo, so, b, x3, "3-D [4,10,64]", tight=False)
    assert y3.shape == (4, 10, 128)
    # m = 0: empty output of the right shape
    y0 = ql.forward(np.zeros((0, 64), np.float32))
    assert y0.shape == (0, 128)
    # non-contiguous input is gathered first (reference :165)
    xt = oracle.normal(71, 1, (64, 6)).T
    assert not xt.flags["C_CONTIGUOUS"]
    check_forward(ql, qo, so, b, np.ascontiguousarray(xt), "contig copy of transposed")
    assert np.array_equal(ql.forward(xt), ql.forward(np.ascontiguousarray(xt)))
    # the C ABI reports the mismatch itself when called directly
    import ctypes as C
    st = nne.load().nne_qlinear_forward_host(ql._handle, None, 1, 63, None)
    assert st == 2


def test_clone_and_from_fields_match(nne, ctx):
    ql, qo, so, b = make_layer(nne, ctx, 72, 96, 256)
    x = oracle.normal(73, 0, (5, 256))
    y = ql.forward(x)
    c = ql.clone()
    assert np.array_equal(c.forward(x), y)
    assert c.memory_bytes() == 96 * 256 + 96 * 4 + 96 * 4


def test_device_forward_and_strided_output(nne, ctx):
    """The device-pointer entry points, on torch-owned memory and torch's current stream."""
    import torch
    ql, qo, so, b = make_layer(nne, ctx, 74, 256, 512)
    x = oracle.normal(75, 0, (4, 512))
    xd = torch.from_numpy(x).cuda()
    yd = torch.full((4, 256), float("nan"), device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    ql.forward_device(xd.data_ptr(), 4, yd.data_ptr(), s)
    wide = torch.full((4, 1000), -7.0, device="cuda")
    ql.forward_device(xd.data_ptr(), 4, wide.data_ptr() + 4 * 100, s, ldy=1000)
    torch.cuda.synchronize()
    y_host = ql.forward(x)
    assert np.array_equal(yd.cpu().numpy(), y_host)
    assert np.array_equal(wide[:, 100:356].cpu().numpy(), y_host)
    assert bool((wide[:, :100] == -7.0).all()) and bool((wide[:, 356:] == -7.0).all())


def test_forward_linearity_property_70b_shape(nne, ctx):
    """Config-5-shaped layer slice (K = 8192 and K = 28672): f(a*x) = a*f(x) exactly for a power
    of two, and f(x1) + f(x2) ~= f(x1 + x2) within the three forwards' rounding of their activations
    to the 16-bit grid (5 % of the summed tolerances; the measured ratio is printed)."""
    for n, k in ((512, 8192), (256, 28672)):
        ql, qo, so, b = make_layer(nne, ctx, 76 + k, n, k, bias=False, std=0.015)
        x1 = oracle.normal(77, k, (1, k))
        x2 = oracle.normal(77, k + 1, (1, k))
        y1, y2 = ql.forward(x1), ql.forward(x2)
        assert np.array_equal(ql.forward(x1 * np.float32(8.0)), y1 * np.float32(8.0))
        y12 = ql.forward(x1 + x2)
        tsum = sum(oracle.tolerance(qo, so, v)[0] for v in (x1, x2, x1 + x2))
        lin = float((np.abs(y12 - (y1 + y2)) / tsum).max())
        print(f"70B-shape {k}->{n}: |f(x1+x2) - f(x1) - f(x2)| / summed tolerances = {lin:.3e}")
        assert lin <= 5e-2
        check_forward(ql, qo, so, None, x1, f"70B-shape {k}->{n} M=1")


def test_nonfinite_and_extreme_activations(nne, ctx):
    """Inf/NaN in x must propagate as IEEE arithmetic does (the streaming kernel switches to its
    fp32 loop for such rows); huge, tiny and all-zero activations must stay within tolerance."""
    n, k = 96, 4096
    ql, qo, so, b = make_layer(nne, ctx, 80, n, k, bias=True)
    x = oracle.normal(81, 0, (1, k))
    xn = x.copy(); xn[0, 1234] = np.nan
    assert np.isnan(ql.forward(xn)).all()
    xi = x.copy(); xi[0, 77] = np.inf
    with np.errstate(all="ignore"):
        y, y_ref = ql.forward(xi), oracle.forward(qo, so, b, xi)
    assert np.array_equal(np.isnan(y), np.isnan(y_ref))
    assert np.array_equal(y[~np.isnan(y)], y_ref[~np.isnan(y_ref)])   # +/-inf by the sign of q[:,77]
    for scale in (1e30, 1e-30, 1e-41):
        check_forward(ql, qo, so, b * np.float32(0), (x * np.float32(scale)).astype(np.float32),
                      f"x scaled by {scale:g}") if False else None
    ql0, qo0, so0, _ = make_layer(nne, ctx, 80, n, k, bias=False)
    for scale in (1e30, 1e-30, 1e-41):
        xs = (x * np.float32(scale)).astype(np.float32)
        check_forward(ql0, qo0, so0, None, xs, f"x scaled by {scale:g}")
    y0 = ql.forward(np.zeros((1, k), np.float32))
    assert np.array_equal(y0[0], b)
    # one dominant element: the small ones fall below the fixed-point grid, still within tolerance
    xd = x.copy(); xd[0, 5] = 1.0e6
    check_forward(ql0, qo0, so0, None, xd, "one dominant activation", tight=False)


def test_two_row_blocks_match_single_rows(nne, ctx):
    """m = 2..4 go through the kernel in blocks of two rows; every row must equal its m = 1 result
    exactly (per-row fixed-point grids are independent)."""
    ql, qo, so, b = make_layer(nne, ctx, 82, 200, 4096, bias=False)
    x = oracle.normal(83, 0, (4, 4096))
    x[2] *= 100.0
    y = ql.forward(x)
    for r in range(4):
        assert np.array_equal(y[r], ql.forward(x[r:r + 1])[0])
