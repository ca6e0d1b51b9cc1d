"""A plan runs several independent forwards as one launch; its results must be bit-identical to
the same forwards issued one by one (and therefore inherit their parity with the oracle)."""
import os

import numpy as np
import pytest

import oracle

pytestmark = pytest.mark.gpu
SKINNY_OFF = os.environ.get("NNE_SKINNY", "").startswith("0")  # small-batch kernel switched off


def build(nne, ctx, shapes, m, seed):
    import torch
    layers, xs, ys, refs = [], [], [], []
    for i, (n, k, bias) in enumerate(shapes):
        w = oracle.normal(seed, 10 * i, (n, k), 0.0, 0.02)
        b = oracle.normal(seed, 10 * i + 1, (n,), 0.0, 0.1) if bias else None
        ql = nne.QLinear.from_linear(nne.Linear(w, b), ctx)
        x = oracle.normal(seed, 10 * i + 2, (m, k)) * np.float32(1.0 + i)
        layers.append(ql)
        xs.append(torch.from_numpy(x).cuda())
        ys.append(torch.full((m, n), float("nan"), device="cuda"))
        refs.append((ql, x, b))
    return layers, xs, ys, refs


@pytest.mark.parametrize("m", [1, 2])
@pytest.mark.parametrize("shapes", [
    [(300, 512, True), (129, 4096, False), (64, 11008, True)],
    [(256, 1024, False)] * 3 + [(100, 2048, True)] * 4 + [(40, 4096, False)] * 5,  # > inline descriptors
])
def test_plan_equals_single_forwards(nne, ctx, shapes, m):
    import torch
    layers, xs, ys, refs = build(nne, ctx, shapes, m, 90 + m)
    plan = nne.QLinearPlan(layers, [t.data_ptr() for t in xs], [t.data_ptr() for t in ys], m, ctx)
    # m = 1: one streaming-GEMV launch; m = 2: pre-pass + one small-batch tensor-core launch
    assert plan.launches == (1 if SKINNY_OFF else m)
    s = torch.cuda.current_stream().cuda_stream
    plan.run(s)
    plan.run(s)  # twice: the second run must not depend on state left by the first
    torch.cuda.synchronize()
    ctx.check()
    for (ql, x, b), y in zip(refs, ys):
        single = ql.forward(x)
        got = y.cpu().numpy()
        assert np.array_equal(got.view(np.uint32), single.view(np.uint32))
        qo, so = oracle.quantize_rows(ql.to_linear().weight / 1.0)  # codes round-trip exactly
        tol, _ = oracle.tolerance(ql.qweight.reshape(ql.out_features, ql.in_features), ql.scales, x)
        y_ref = oracle.forward(ql.qweight.reshape(ql.out_features, ql.in_features), ql.scales, b, x)
        assert float((np.abs(got - y_ref) / tol).max()) <= 2e-2


def test_plan_falls_back_for_other_shapes(nne, ctx):
    import torch
    # m = 3 and a k that is no multiple of 16: the plan runs its layers one after the other
    shapes = [(64, 512, True), (33, 1001, False)]
    layers, xs, ys, refs = build(nne, ctx, shapes, 3, 95)
    plan = nne.QLinearPlan(layers, [t.data_ptr() for t in xs], [t.data_ptr() for t in ys], 3, ctx)
    assert plan.launches == 2
    plan.run(torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    for (ql, x, b), y in zip(refs, ys):
        assert np.array_equal(y.cpu().numpy(), ql.forward(x))


def test_plan_argument_errors(nne, ctx):
    import torch
    layers, xs, ys, _ = build(nne, ctx, [(64, 512, False)], 1, 96)
    with pytest.raises(nne.InvalidArgument):
        nne.QLinearPlan(layers, [0], [ys[0].data_ptr()], 1, ctx)
    empty = nne.QLinearPlan(layers, [xs[0].data_ptr()], [ys[0].data_ptr()], 0, ctx)
    empty.run(0)  # m = 0: nothing to do


@pytest.mark.parametrize("m,slabs", [(1, True), (2, False), (5, True)])
def test_plan_run_host_equals_single_forwards(nne, ctx, m, slabs):
    """Host round trip of a plan: one slab each way (buffers continue one another) or one copy
    per layer (scattered buffers); m = 5 takes the layer-by-layer path."""
    import torch
    shapes = [(300, 512, True), (129, 4096, False), (64, 1024, True), (256, 256, False)]
    layers, xs, ys, refs = build(nne, ctx, shapes, m, 97 + m)
    if slabs:
        xslab = torch.empty(sum(m * k for _, k, _ in shapes), device="cuda")
        yslab = torch.full((sum(m * n for n, _, _ in shapes),), float("nan"), device="cuda")
        xp, yp, xo, yo = [], [], 0, 0
        for n, k, _ in shapes:
            xp.append(xslab.data_ptr() + 4 * xo)
            yp.append(yslab.data_ptr() + 4 * yo)
            xo += m * k
            yo += m * n
    else:
        xp, yp = [t.data_ptr() for t in xs], [t.data_ptr() for t in ys]
    plan = nne.QLinearPlan(layers, xp, yp, m, ctx)
    x_all = np.concatenate([x.reshape(-1) for (_, x, _) in refs])
    y_all = plan.run_host(x_all)
    y_again = plan.run_host(x_all)
    ctx.check()
    assert np.array_equal(y_all.view(np.uint32), y_again.view(np.uint32))
    off = 0
    for (ql, x, b) in refs:
        single = ql.forward(x).reshape(-1)
        got = y_all[off:off + single.size]
        assert np.array_equal(got.view(np.uint32), single.view(np.uint32))
        off += single.size
    with pytest.raises(nne.ShapeMismatch):
        plan.run_host(x_all[:-1])


@pytest.mark.parametrize("m", [1, 4, 40])
def test_plan_run_host_from_pinned_memory(nne, ctx, m):
    """With PINNED host slabs (and 16-byte aligned runs) the host round trip moves x and y with
    copy kernels chained to the forwards instead of copy-engine transfers: same bits as from
    pageable memory, run after run, also when the slabs change."""
    import torch
    shapes = [(512, 1024, True), (256, 4096, False), (128, 1024, True)]
    layers, xs, ys, refs = build(nne, ctx, shapes, m, 197 + m)
    xslab = torch.empty(sum(m * k for _, k, _ in shapes), device="cuda")
    yslab = torch.full((sum(m * n for n, _, _ in shapes),), float("nan"), device="cuda")
    xp, yp, xo, yo = [], [], 0, 0
    for n, k, _ in shapes:
        xp.append(xslab.data_ptr() + 4 * xo)
        yp.append(yslab.data_ptr() + 4 * yo)
        xo += m * k
        yo += m * n
    plan = nne.QLinearPlan(layers, xp, yp, m, ctx)
    x_all = np.concatenate([x.reshape(-1) for (_, x, _) in refs])
    want = plan.run_host(x_all)                      # pageable memory: copy engines
    launches0 = nne.load().nne_launch_count()
    plan.run_host(x_all)
    per_run = nne.load().nne_launch_count() - launches0
    xpin = torch.from_numpy(x_all).pin_memory()
    for trial in range(3):
        ypin = torch.full((want.size,), float("nan")).pin_memory()
        launches0 = nne.load().nne_launch_count()
        got = plan.run_host(xpin.numpy(), ypin.numpy())
        small = 4 * (x_all.size + want.size) <= (1 << 20)   # larger transfers stay with the copy engines
        assert nne.load().nne_launch_count() - launches0 == per_run + (2 if small else 0)   # the two copy kernels
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), f"trial {trial}"
    ctx.check()
    # other activations through the same pinned slab
    x2 = (x_all * np.float32(0.5)).astype(np.float32)
    xpin.copy_(torch.from_numpy(x2))
    got2 = plan.run_host(xpin.numpy(), ypin.numpy())
    assert np.array_equal(got2.view(np.uint32), plan.run_host(x2).view(np.uint32))
    ctx.check()


@pytest.mark.parametrize("m", [3, 8, 16])
@pytest.mark.parametrize("shared", [False, True])
def test_small_batch_plan_equals_single_forwards(nne, ctx, m, shared):
    """3 <= m <= 16: the list runs as one pre-pass + one small-batch tensor-core launch.  With
    `shared`, the first three layers read the same x (q/k/v) and the last two another (gate/up)."""
    import torch
    shapes = [(512, 1024, True), (300, 1024, False), (1024, 1024, True), (2048, 512, False),
              (130, 512, True)]
    layers, xs, ys, refs = build(nne, ctx, shapes, m, 120 + m)
    if shared:
        xs = [xs[0], xs[0], xs[0], xs[3], xs[3]]
        refs = [(refs[i][0], refs[0][1] if i < 3 else refs[3][1], refs[i][2]) for i in range(5)]
    plan = nne.QLinearPlan(layers, [t.data_ptr() for t in xs], [t.data_ptr() for t in ys], m, ctx)
    assert plan.launches == (len(layers) if SKINNY_OFF else 2)
    s = torch.cuda.current_stream().cuda_stream
    plan.run(s)
    plan.run(s)
    torch.cuda.synchronize()
    ctx.check()
    for (ql, x, b), y in zip(refs, ys):
        single = ql.forward(x)
        got = y.cpu().numpy()
        assert np.array_equal(got.view(np.uint32), single.view(np.uint32))
        qw = ql.qweight.reshape(ql.out_features, ql.in_features)
        tol, _ = oracle.tolerance(qw, ql.scales, x)
        y_ref = oracle.forward(qw, ql.scales, b, x)
        assert float((np.abs(got - y_ref) / tol).max()) <= 1e-2


def test_small_batch_plan_many_layers_big_shapes(nne, ctx):
    """More units than one CTA range per layer and more layers than SMs' worth of tiles: 7B-shaped
    q/k/v/o + gate/up + down as one list at m = 8."""
    import torch
    shapes = [(4096, 4096, False)] * 4 + [(11008, 4096, False)] * 2 + [(4096, 11008, True)]
    layers, xs, ys, refs = build(nne, ctx, shapes, 8, 131)
    plan = nne.QLinearPlan(layers, [t.data_ptr() for t in xs], [t.data_ptr() for t in ys], 8, ctx)
    assert plan.launches == (len(layers) if SKINNY_OFF else 2)
    plan.run(torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    ctx.check()
    for (ql, x, b), y in zip(refs, ys):
        assert np.array_equal(y.cpu().numpy().view(np.uint32), ql.forward(x).view(np.uint32))


def test_reserved_sms_leave_results_unchanged(nne, ctx):
    """nne_cuda_ctx_reserve_sms shrinks the streaming kernel's grid; row ranges per CTA change,
    results must not (each output channel is one exact integer sum)."""
    import torch
    lib = nne.load()
    own = nne.CudaContext(0)  # a context of its own: the setting must not leak into other tests
    shapes = [(1000, 512, True), (4096, 4096, False), (300, 2048, True)]
    layers, xs, ys, refs = build(nne, own, shapes, 1, 141)
    plan = nne.QLinearPlan(layers, [t.data_ptr() for t in xs], [t.data_ptr() for t in ys], 1, own)
    s = torch.cuda.current_stream().cuda_stream
    plan.run(s)
    torch.cuda.synchronize()
    base = [y.clone() for y in ys]
    for reserve in (8, 100, 147, 0):
        assert lib.nne_cuda_ctx_reserve_sms(own.handle, reserve) == 0
        for y in ys:
            y.fill_(float("nan"))
        plan.run(s)
        torch.cuda.synchronize()
        own.check()
        for y, b in zip(ys, base):
            assert torch.equal(y.view(torch.int32), b.view(torch.int32)), f"reserve={reserve}"
    assert lib.nne_cuda_ctx_reserve_sms(own.handle, -1) != 0
    assert lib.nne_cuda_ctx_reserve_sms(own.handle, 100000) != 0
    plan.close()
