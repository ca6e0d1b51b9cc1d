"""The steps either side of a QLinear in a LLaMA decoder block on the device: RMSNorm
(reference src/nn/norm.rs:141-165), silu(gate) * up (src/models/llama.rs:343-346) and the residual
add, as standalone kernels and fused into the forwards of a plan, against the CPU oracle's
restatement of those lines.  Tolerance for the element-wise kernels: 1e-5 relative to the row's
largest magnitude (the sum of squares is taken in another order than the reference's AVX2 lanes);
for forwards: the path's tolerance 1e-3 * ||x'||inf * scale_j * sum|q_jk| with x' the transformed
input, and a tight check at 2e-5 of that bound for the fp-exact decode kernels."""
import numpy as np
import pytest

import oracle

pytestmark = pytest.mark.gpu


def dev(t):
    import torch
    return torch.from_numpy(np.ascontiguousarray(t)).cuda()


@pytest.mark.parametrize("rows,cols", [(1, 4096), (8, 11008), (3, 77), (300, 1024), (2, 1)])
def test_rmsnorm_kernel(nne, ctx, rows, cols):
    import torch
    x = oracle.normal(500, rows + cols, (rows, cols), 0.0, 2.0)
    g = oracle.normal(501, cols, (cols,), 1.0, 0.2)
    xd, gd = dev(x), dev(g)
    yd = torch.empty_like(xd)
    for eps in (1e-6, 1e-5):
        nne.rmsnorm_device(ctx, xd.data_ptr(), gd.data_ptr(), eps, rows, cols, yd.data_ptr(),
                           torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        y = yd.cpu().numpy()
        for avx in (1, 0):
            ref = oracle.rms_norm(x, g, eps, avx)
            rel = np.abs(y - ref).max() / max(np.abs(ref).max(), 1e-30)
            assert rel <= 1e-5, f"rows={rows} cols={cols} eps={eps}: rel err {rel}"
    ctx.check()


def test_silu_mul_and_add_kernels(nne, ctx):
    import torch
    n = 3 * 11008 + 5
    g = oracle.normal(502, 0, (n,), 0.0, 3.0)
    u = oracle.normal(502, 1, (n,), 0.0, 1.0)
    g[:6] = [0.0, -0.0, 80.0, -80.0, -100.0, 20.0]       # saturating ends of the sigmoid
    gd, ud = dev(g), dev(u)
    od = torch.empty_like(gd)
    s = torch.cuda.current_stream().cuda_stream
    nne.silu_mul_device(ctx, gd.data_ptr(), ud.data_ptr(), n, od.data_ptr(), s)
    torch.cuda.synchronize()
    ref = oracle.silu_mul(g, u)
    out = od.cpu().numpy()
    assert np.abs(out - ref).max() <= 1e-5 * max(np.abs(ref).max(), 1.0)
    assert np.all(np.abs(out - ref) <= 4e-6 * np.abs(ref) + 1e-30)      # element-wise: a few ulp of exp
    nne.add_device(ctx, gd.data_ptr(), ud.data_ptr(), n, od.data_ptr(), s)
    torch.cuda.synchronize()
    assert np.array_equal(od.cpu().numpy().view(np.uint32), (g + u).view(np.uint32))
    ctx.check()


def make(nne, ctx, seed, n, k):
    w = oracle.normal(seed, 0, (n, k), 0.0, 0.02)
    ql = nne.QLinear.from_linear(nne.Linear(w), ctx)
    return ql, ql.qweight.reshape(n, k), ql.scales


@pytest.mark.parametrize("m", [1, 2, 8, 40])
def test_fused_plan_matches_the_oracle_chain(nne, ctx, m):
    """q/k/v-style: three layers reading RMSNorm(h); down-style: one layer reading silu(g) * u and
    adding a residual.  m = 1: the decode kernel does it all itself; m = 2, 8: small-batch kernel and
    m = 40: prefill kernel, with the standalone kernels run by the plan."""
    import torch
    d, f = 1024, 2816
    s = torch.cuda.current_stream().cuda_stream
    h = oracle.normal(510, m, (m, d), 0.0, 1.5)
    gamma = oracle.normal(511, 0, (d,), 1.0, 0.1)
    eps = 1e-6
    qs = [make(nne, ctx, 520 + i, n, d) for i, n in enumerate((d, 512, 512))]
    hd, gd = dev(h), dev(gamma)
    outs = [torch.full((m, n), float("nan"), device="cuda") for n in (d, 512, 512)]
    plan = nne.FusedPlan([{"layer": q[0], "x": hd.data_ptr(), "y": o.data_ptr(),
                           "rmsnorm": (gd.data_ptr(), eps)} for q, o in zip(qs, outs)], m, ctx)
    plan.run(s)
    torch.cuda.synchronize()
    ctx.check()
    # m = 1: one launch; m = 2, 8: RMSNorm once for the three + pre-pass + kernel; m = 40: RMSNorm + a forward per layer
    assert plan.launches == {1: 1, 2: 3, 8: 3, 40: 4}[m]
    xn = oracle.rms_norm(h, gamma, eps)
    for (ql, q, sc), o in zip(qs, outs):
        ref = oracle.forward(q, sc, None, xn)
        tol, _ = oracle.tolerance(q, sc, xn)
        ratio = float((np.abs(o.cpu().numpy() - ref) / tol).max())
        assert ratio <= (2e-2 if m <= 16 else 1.0), f"m={m}: err/tol {ratio}"
    # down-style
    down, qd, sd = make(nne, ctx, 530, d, f)
    g = oracle.normal(512, m, (m, f), 0.0, 2.0)
    u = oracle.normal(513, m, (m, f), 0.0, 1.0)
    res = oracle.normal(514, m, (m, d), 0.0, 1.0)
    gdv, udv, rdv = dev(g), dev(u), dev(res)
    y = torch.full((m, d), float("nan"), device="cuda")
    plan2 = nne.FusedPlan([{"layer": down, "x": gdv.data_ptr(), "y": y.data_ptr(),
                            "silu_mul": udv.data_ptr(), "residual": rdv.data_ptr()}], m, ctx)
    plan2.run(s)
    torch.cuda.synchronize()
    ctx.check()
    hh = oracle.silu_mul(g, u)
    ref = oracle.forward(qd, sd, None, hh) + res
    tol, _ = oracle.tolerance(qd, sd, hh)
    ratio = float((np.abs(y.cpu().numpy() - ref) / tol).max())
    print(f"fused m={m}: down-style err/tol {ratio:.3e}, launches {plan.launches} / {plan2.launches}")
    assert ratio <= (2e-2 if m <= 16 else 1.0)
    if m > 1:
        # not the decode kernel: the plan ran the standalone kernels, so it equals them bit for bit
        tmp = torch.empty_like(gdv)
        nne.silu_mul_device(ctx, gdv.data_ptr(), udv.data_ptr(), m * f, tmp.data_ptr(), s)
        y2 = torch.empty_like(y)
        down.forward_device(tmp.data_ptr(), m, y2.data_ptr(), s)
        nne.add_device(ctx, y2.data_ptr(), rdv.data_ptr(), m * d, y2.data_ptr(), s)
        torch.cuda.synchronize()
        assert torch.equal(y2.view(torch.int32), y.view(torch.int32))
    plan.close()
    plan2.close()


def test_nonfinite_input_through_a_fused_decode_plan(nne, ctx):
    """An Inf in h makes rrms 0 and Inf * 0 = NaN (as the reference's row function gives): every
    channel of that forward is NaN; a second, finite layer of the same plan is untouched."""
    import torch
    d = 512
    ql, q, sc = make(nne, ctx, 540, 256, d)
    h = oracle.normal(541, 0, (1, d))
    h[0, 7] = np.inf
    h2 = oracle.normal(541, 1, (1, d))
    gamma = np.ones(d, np.float32)
    hd, h2d, gd = dev(h), dev(h2), dev(gamma)
    y = torch.zeros(2, 256, device="cuda")
    plan = nne.FusedPlan([{"layer": ql, "x": hd.data_ptr(), "y": y[0].data_ptr(), "rmsnorm": (gd.data_ptr(), 1e-6)},
                          {"layer": ql, "x": h2d.data_ptr(), "y": y[1].data_ptr(), "rmsnorm": (gd.data_ptr(), 1e-6)}],
                         1, ctx)
    plan.run(torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    ctx.check()
    out = y.cpu().numpy()
    assert np.isnan(out[0]).all()
    xn = oracle.rms_norm(h2, gamma, 1e-6)
    tol, _ = oracle.tolerance(q, sc, xn)
    assert float((np.abs(out[1] - oracle.forward(q, sc, None, xn)[0]) / tol).max()) <= 2e-2
    plan.close()
