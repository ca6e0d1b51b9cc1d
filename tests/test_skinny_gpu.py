"""GPU parity of the small-batch tensor-core forward (3 <= m <= 16) against the CPU oracle.

The kernel puts each activation row on the same fixed-point grid as the streaming GEMV
(rint(x * 2^e), max|x| * 2^e in [2^14, 2^15)) and keeps exact integer sums, so besides the
tolerance check against the oracle there are two bit-for-bit checks: integer-valued activations
against the oracle, and every row of a batch against the single-row forward of that row (which
runs the streaming GEMV, a different kernel)."""
import os

import numpy as np
import pytest

import oracle

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(os.environ.get("NNE_SKINNY", "").startswith("0"),
                                 reason="the small-batch kernel is switched off (NNE_SKINNY=0)")]


def layer(nne, ctx, seed, n, k, bias):
    w = oracle.normal(seed, 0, (n, k), 0.0, 0.02)
    b = oracle.normal(seed, 1, (n,), 0.0, 0.1) if bias else None
    ql = nne.QLinear.from_linear(nne.Linear(w, b), ctx)
    qo, so = oracle.quantize_rows(w)
    assert np.array_equal(ql.qweight.reshape(n, k), qo)
    return ql, qo, so, b


SHAPES = [
    (128, 128),     # one tile, one k-block: a single CTA owns the tile (no atomics)
    (128, 4096),    # one tile split over many CTAs (partial sums + last-arriver finish)
    (4096, 4096),   # 32 tiles x 32 k-blocks over 148 CTAs: ranges straddle tile boundaries
    (11008, 4096),
    (4096, 11008),
    (1000, 272),    # channel tail (1000 = 7*128 + 104) and k tail (272 = 2*128 + 16)
    (130, 4112),    # 2 tiles, second almost empty
    (40000, 256),   # more tiles than CTAs: several whole tiles per CTA, both TMEM buffers
]


@pytest.mark.parametrize("n,k", SHAPES)
@pytest.mark.parametrize("m", [3, 8, 16])
def test_integer_activations_bit_exact(nne, ctx, n, k, m):
    ql, qo, so, b = layer(nne, ctx, 500 + n + k, n, k, bias=(n % 3 == 1))
    assert ql.kernel_for(m) == 4
    rng = np.random.default_rng(n + k + m)
    x = rng.integers(-8, 9, size=(m, k)).astype(np.float32)
    y = ql.forward(x)
    ctx.check()
    y_ref = oracle.forward(qo, so, b, x)
    assert np.array_equal(y.view(np.uint32), y_ref.view(np.uint32)), \
        f"mismatch at {np.argwhere(y != y_ref)[:5].tolist()}"


@pytest.mark.parametrize("n,k", SHAPES)
@pytest.mark.parametrize("m", [4, 5, 16])
def test_normal_activations(nne, ctx, n, k, m):
    ql, qo, so, b = layer(nne, ctx, 7, n, k, bias=(k % 3 == 1))
    x = oracle.normal(7, 100 + m, (m, k)) * np.float32(1.0 + m)  # rows of different magnitude
    x *= np.linspace(0.01, 30.0, m, dtype=np.float32)[:, None]
    y = ql.forward(x)
    ctx.check()
    y_ref = oracle.forward(qo, so, b, x)
    tol, _ = oracle.tolerance(qo, so, x)
    ratio = float((np.abs(y - y_ref) / tol).max())
    print(f"skinny {k}->{n} M={m}: max err/tol {ratio:.3e}")
    assert ratio <= 1.0
    # row by row through the streaming GEMV (m = 1): same grid, same exact sums, same rounding
    if ql.kernel_for(1) == 1 and 256 <= k <= 32768:   # shorter rows take the fp32 GEMV
        for r in range(m):
            y1 = ql.forward(x[r:r + 1])
            assert np.array_equal(y1.view(np.uint32)[0], y.view(np.uint32)[r]), f"row {r} differs"
    ctx.check()


def test_two_calls_and_other_m_between(nne, ctx):
    """The stream-ordered workspace is zeroed by each call's own pre-pass."""
    ql, qo, so, b = layer(nne, ctx, 11, 4096, 4096, True)
    x = oracle.normal(11, 5, (16, 4096))
    y1 = ql.forward(x)
    ql.forward(x[:2])
    ql.forward(oracle.normal(11, 6, (64, 4096)))
    y2 = ql.forward(x)
    y3 = ql.forward(x[:7])
    ctx.check()
    assert np.array_equal(y1.view(np.uint32), y2.view(np.uint32))
    assert np.array_equal(y1.view(np.uint32)[:7], y3.view(np.uint32))


def test_non_finite_row_is_nan_others_untouched(nne, ctx):
    ql, qo, so, b = layer(nne, ctx, 13, 512, 1024, False)
    x = oracle.normal(13, 1, (6, 1024))
    y_clean = ql.forward(x)
    x2 = x.copy()
    x2[2, 17] = np.inf
    x2[4, 900] = np.nan
    y = ql.forward(x2)
    ctx.check()
    assert np.isnan(y[2]).all() and np.isnan(y[4]).all()
    for r in (0, 1, 3, 5):
        assert np.array_equal(y[r].view(np.uint32), y_clean[r].view(np.uint32))


def test_zero_rows_and_tiny_values(nne, ctx):
    ql, qo, so, b = layer(nne, ctx, 17, 384, 512, True)
    x = oracle.normal(17, 1, (5, 512))
    x[1] = 0.0
    x[3] *= np.float32(1e-30)
    y = ql.forward(x)
    ctx.check()
    y_ref = oracle.forward(qo, so, b, x)
    tol, _ = oracle.tolerance(qo, so, x)
    assert np.array_equal(y[1], b.astype(np.float32))
    assert float((np.abs(y - y_ref) / np.maximum(tol, 1e-37)).max()) <= 1.0


def test_strided_output(nne, ctx):
    import torch
    ql, qo, so, b = layer(nne, ctx, 19, 640, 768, True)
    m, ld = 9, 1000
    x = oracle.normal(19, 1, (m, 768))
    xd = torch.from_numpy(x).cuda()
    wide = torch.full((m, ld), -7.0, device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    ql.forward_device(xd.data_ptr(), m, wide.data_ptr() + 4 * 100, s, ldy=ld)
    torch.cuda.synchronize()
    ctx.check()
    y = wide.cpu().numpy()
    assert np.array_equal(y[:, 100:740], ql.forward(x))
    assert (y[:, :100] == -7.0).all() and (y[:, 740:] == -7.0).all()
