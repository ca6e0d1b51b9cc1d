"""The steps either side of a QLinear in a LLaMA decoder block on the device: RMSNorm
(reference src/nn/norm.rs:141-165), silu(gate) * up (src/models/llama.rs:343-346) and the residual
add, as standalone kernels and fused into the forwards of a plan, against the CPU oracle's
restatement of those lines.  Tolerance for the element-wise kernels: 1e-5 relative to the row's
largest magnitude (the sum of squares is taken in another order than the reference's AVX2 lanes);
for forwards: the path's tolerance 1e-3 * ||x'||inf * scale_j * sum|q_jk| with x' the transformed
input, and a tight check at 2 % of that tolerance for the decode kernels (16-bit activation grid)."""
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


@pytest.mark.parametrize("m", [1, 2, 8])
def test_chained_items_in_one_plan(nne, ctx, m):
    """A whole decoder block's linear layers as ONE plan whose items consume one another's outputs:
    [q, k, v] <- RMSNorm(h); o <- v, + h -> h2; [gate, up] <- RMSNorm(h2); down <- silu(gate) * up,
    + h2 -> out.  The library finds the dependencies itself.  m = 1: one launch of the decode kernel
    whose grid meets between the groups; other m: the groups run one after another.  Must equal, bit
    for bit, the same groups run as four separate plans, and agree with the oracle's chain."""
    import torch
    d, f = 1024, 2816
    s = torch.cuda.current_stream().cuda_stream
    eps = 1e-6
    shapes = {"q": (d, d), "k": (512, d), "v": (d, d), "o": (d, d), "gate": (f, d), "up": (f, d), "down": (d, f)}
    L = {nm: make(nne, ctx, 600 + i, n, k) for i, (nm, (n, k)) in enumerate(shapes.items())}
    h = oracle.normal(610, m, (m, d), 0.0, 1.5)
    g1 = oracle.normal(611, 0, (d,), 1.0, 0.1)
    g2 = oracle.normal(611, 1, (d,), 1.0, 0.1)
    hd, g1d, g2d = dev(h), dev(g1), dev(g2)

    def buffers():
        b = {nm: torch.full((m, n), float("nan"), device="cuda") for nm, (n, _) in shapes.items()}
        b["h2"] = torch.full((m, d), float("nan"), device="cuda")
        return b

    def groups(b):
        return [
            [{"layer": L[nm][0], "x": hd.data_ptr(), "y": b[nm].data_ptr(), "rmsnorm": (g1d.data_ptr(), eps)}
             for nm in ("q", "k", "v")],
            [{"layer": L["o"][0], "x": b["v"].data_ptr(), "y": b["h2"].data_ptr(), "residual": hd.data_ptr()}],
            [{"layer": L[nm][0], "x": b["h2"].data_ptr(), "y": b[nm].data_ptr(), "rmsnorm": (g2d.data_ptr(), eps)}
             for nm in ("gate", "up")],
            [{"layer": L["down"][0], "x": b["gate"].data_ptr(), "y": b["down"].data_ptr(),
              "silu_mul": b["up"].data_ptr(), "residual": b["h2"].data_ptr()}],
        ]

    b_sep, b_one = buffers(), buffers()
    separate = [nne.FusedPlan(g, m, ctx) for g in groups(b_sep)]
    one = nne.FusedPlan([it for g in groups(b_one) for it in g], m, ctx)
    for p in separate:
        p.run(s)
    for _ in range(3):          # run it again and again: the rendezvous counter carries over
        one.run(s)
    torch.cuda.synchronize()
    ctx.check()
    if m == 1:
        assert one.launches == 1
    else:
        assert one.launches == sum(p.launches for p in separate)
    for nm in list(shapes) + ["h2"]:
        assert torch.equal(b_one[nm].view(torch.int32), b_sep[nm].view(torch.int32)), nm
    # the oracle's chain on the same codes
    xn = oracle.rms_norm(h, g1, eps)
    v = oracle.forward(L["v"][1], L["v"][2], None, xn)
    h2 = oracle.forward(L["o"][1], L["o"][2], None, v) + h
    xn2 = oracle.rms_norm(h2, g2, eps)
    gate = oracle.forward(L["gate"][1], L["gate"][2], None, xn2)
    up = oracle.forward(L["up"][1], L["up"][2], None, xn2)
    act = oracle.silu_mul(gate, up)
    out = oracle.forward(L["down"][1], L["down"][2], None, act) + h2
    got = b_one["down"].cpu().numpy()
    rel = float(np.abs(got - out).max() / np.abs(out).max())
    print(f"chained plan m={m}: launches {one.launches}, max |diff| / max |out| vs the oracle chain {rel:.2e}")
    assert rel <= 1e-4
    one.close()
    for p in separate:
        p.close()


def test_chained_plan_hazards_and_refusals(nne, ctx):
    """Write-after-write and write-after-read inside one plan are ordered too; an item that would
    overwrite its own input is refused."""
    import torch
    d = 512
    s = torch.cuda.current_stream().cuda_stream
    a, qa, sa = make(nne, ctx, 620, d, d)
    b, qb, sb = make(nne, ctx, 621, d, d)
    x = oracle.normal(622, 0, (1, d))
    xd = dev(x)
    y = torch.zeros(1, d, device="cuda")
    z = torch.zeros(1, d, device="cuda")
    # item 0: y = a(x); item 1: z = b(y); item 2: y = b(x)  (overwrites what item 1 reads)
    plan = nne.FusedPlan([{"layer": a, "x": xd.data_ptr(), "y": y.data_ptr()},
                          {"layer": b, "x": y.data_ptr(), "y": z.data_ptr()},
                          {"layer": b, "x": xd.data_ptr(), "y": y.data_ptr()}], 1, ctx)
    assert plan.launches == 1
    for _ in range(2):
        plan.run(s)
    torch.cuda.synchronize()
    ctx.check()
    ya = oracle.forward(qa, sa, None, x)
    tol, _ = oracle.tolerance(qb, sb, ya)
    assert float((np.abs(z.cpu().numpy() - oracle.forward(qb, sb, None, ya)) / tol).max()) <= 2e-2
    tol, _ = oracle.tolerance(qb, sb, x)
    assert float((np.abs(y.cpu().numpy() - oracle.forward(qb, sb, None, x)) / tol).max()) <= 2e-2
    plan.close()
    with pytest.raises(nne.InvalidArgument):
        nne.FusedPlan([{"layer": a, "x": y.data_ptr(), "y": y.data_ptr()}], 1, ctx)
    # a residual that IS the output is fine (read and written by the same thread)
    y.copy_(dev(x))
    p2 = nne.FusedPlan([{"layer": a, "x": xd.data_ptr(), "y": y.data_ptr(), "residual": y.data_ptr()}], 1, ctx)
    p2.run(s)
    torch.cuda.synchronize()
    ctx.check()
    tol, _ = oracle.tolerance(qa, sa, x)
    assert float((np.abs(y.cpu().numpy() - (ya + x)) / tol).max()) <= 2e-2
    p2.close()
