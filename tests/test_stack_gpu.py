"""Config 4 of the benchmark plan: a LLaMA-2-7B-shaped decoder stack of QLinears (32 layers of
q/k/v/o 4096->4096, gate/up 4096->11008, down 11008->4096; 224 layers, 6.5 GB of int8 codes), one
decode step at batch 1 and batch 8, each layer fed by the one before it.

The weights are drawn on the device (the CPU generator would need minutes for 6.5 G values), so
parity is checked two ways that do not need them on the host:
  * against the oracle on SAMPLED layers (first and last), with the codes downloaded through the C
    ABI and the layer's actual device input copied back;
  * through a size-independent property over the whole 224-layer chain: row r of the batch-8 step
    (small-batch tensor-core kernel) equals, bit for bit, the batch-1 step of that row alone
    (streaming GEMV) - any error in either kernel is amplified by the 32 layers behind it."""
import ctypes as C
import time

import numpy as np
import pytest

import oracle

pytestmark = pytest.mark.gpu

H, F, LAYERS = 4096, 11008, 32
NAMES = [("q", H, H), ("k", H, H), ("v", H, H), ("o", H, H), ("gate", F, H), ("up", F, H), ("down", H, F)]


def graph_time_ms(torch, issue, reps=5):
    """Device time of one replay of a CUDA graph holding everything `issue(stream)` launches: the
    chain as the GPU runs it, without the host's per-launch cost (Python + ctypes, about as long as
    a decode-sized kernel)."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        issue(torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps


def test_config4_decoder_stack(nne, ctx):
    import torch
    lib = nne.load()
    dev = torch.device("cuda", 0)
    gen = torch.Generator(device=dev)
    gen.manual_seed(4)
    stream = torch.cuda.current_stream().cuda_stream
    stack = []
    for _ in range(LAYERS):
        layer = {}
        for name, n, k in NAMES:
            w = torch.randn(n, k, generator=gen, device=dev) * 0.02
            h = C.c_void_p()
            assert lib.nne_qlinear_create_from_f32_dev(ctx.handle, w.data_ptr(), None, n, k, stream,
                                                       C.byref(h)) == 0
            layer[name] = h
            del w
        stack.append(layer)
    torch.cuda.synchronize()
    total_bytes = sum(lib.nne_qlinear_memory_bytes(h) for layer in stack for h in layer.values())
    assert total_bytes == LAYERS * (4 * (H * H + 4 * H) + 3 * (H * F) + 2 * 4 * F + 4 * H)

    def fwd(h, x, m, k, y):
        assert lib.nne_qlinear_forward_dev(h, x.data_ptr(), m, k, y.data_ptr(), stream) == 0

    def decode_step(x0, keep=None):
        """x0 [b, H] on the device -> hidden state after 32 layers; `keep` collects (input, output)
        of sampled projections."""
        b = x0.shape[0]
        hcur = x0.clone()
        q, kk, v, o, d = (torch.empty(b, H, device=dev) for _ in range(5))
        g, u = (torch.empty(b, F, device=dev) for _ in range(2))
        for li, layer in enumerate(stack):
            fwd(layer["q"], hcur, b, H, q)
            fwd(layer["k"], hcur, b, H, kk)
            fwd(layer["v"], hcur, b, H, v)
            fwd(layer["o"], q, b, H, o)          # q stands in for the attention output
            fwd(layer["gate"], o, b, H, g)
            fwd(layer["up"], o, b, H, u)
            fwd(layer["down"], g, b, F, d)
            if keep is not None and li in (0, LAYERS - 1):
                keep[(li, "q")] = (hcur.cpu().numpy().copy(), q.cpu().numpy().copy())
                keep[(li, "down")] = (g.cpu().numpy().copy(), d.cpu().numpy().copy())
            hcur, d = d, hcur
        torch.cuda.synchronize()
        return hcur

    x8 = torch.randn(8, H, generator=gen, device=dev)
    keep = {}
    out8 = decode_step(x8, keep)
    ctx.check()
    assert bool(torch.isfinite(out8).all())

    # (1) sampled layers against the oracle
    for (li, name), (xin, yout) in keep.items():
        n, k = (H, H) if name == "q" else (H, F)
        qw = np.empty((n, k), dtype=np.int8)
        sc = np.empty(n, dtype=np.float32)
        assert lib.nne_qlinear_download(stack[li][name], qw.ctypes.data_as(C.c_void_p),
                                        sc.ctypes.data_as(C.c_void_p)) == 0
        y_ref = oracle.forward(qw, sc, None, xin)
        tol, _ = oracle.tolerance(qw, sc, xin)
        ratio = float((np.abs(yout - y_ref) / tol).max())
        print(f"config4 layer {li} {name}: max err/tol {ratio:.3e}")
        assert ratio <= 1.0

    # (2) batch invariance over the whole chain: different kernels, identical bits
    for r in (0, 5):
        out1 = decode_step(x8[r:r + 1].contiguous())
        assert torch.equal(out1.view(torch.int32)[0], out8.view(torch.int32)[r]), f"row {r} differs"
    ctx.check()

    # informational: linear-layer time of one decode step (224 dependent forwards, issued eagerly)
    for b in (1, 8):
        xb = x8[:b].contiguous()
        decode_step(xb)
        t0 = time.perf_counter()
        decode_step(xb)
        dt = time.perf_counter() - t0
        print(f"config4 batch {b}: {dt * 1e3:.2f} ms per decode step of the linear layers, "
              f"{b / dt:.0f} tokens/s, {total_bytes / dt / 1e9:.0f} GB/s of weights")
    # The same step with the independent projections of a layer grouped into plans
    # ([q, k, v], [o], [gate, up], [down]: 4 launches or launch pairs per layer instead of 7);
    # the result must not change by a bit.
    for b in (1, 8):
        xb = x8[:b].contiguous()
        want = decode_step(xb)
        bufs = {name: torch.empty(b, n, device=dev) for name, n, _ in NAMES}
        hid = [torch.empty(b, H, device=dev), torch.empty(b, H, device=dev)]
        plans = []
        for li, layer in enumerate(stack):
            src, dst = hid[li % 2], hid[(li + 1) % 2]
            groups = [(("q", "k", "v"), src, None), (("o",), bufs["q"], None),
                      (("gate", "up"), bufs["o"], None), (("down",), bufs["gate"], dst)]
            for names, xin, out in groups:
                cnt = len(names)
                hs = (C.c_void_p * cnt)(*[layer[nm] for nm in names])
                xs = (C.c_void_p * cnt)(*[xin.data_ptr()] * cnt)
                ys = (C.c_void_p * cnt)(*[(out if out is not None else bufs[nm]).data_ptr() for nm in names])
                p = C.c_void_p()
                assert lib.nne_qlinear_plan_create(ctx.handle, cnt, hs, xs, ys, b, C.byref(p)) == 0
                plans.append(p)

        def plan_step():
            hid[0].copy_(xb)
            for p in plans:
                assert lib.nne_qlinear_plan_run(p, stream) == 0
            torch.cuda.synchronize()
            return hid[LAYERS % 2]

        got = plan_step()
        ctx.check()
        assert torch.equal(got.view(torch.int32), want.view(torch.int32))
        t0 = time.perf_counter()
        plan_step()
        dt = time.perf_counter() - t0
        # (the graph resets the hidden state like plan_step does: fed its own output again and again,
        # a chain without norms overflows to Inf and every forward takes the kernels' IEEE slow path)
        gms = graph_time_ms(torch, lambda st: [hid[0].copy_(xb)] + [lib.nne_qlinear_plan_run(p, st) for p in plans])
        print(f"config4 batch {b}, grouped into plans: {dt * 1e3:.2f} ms per decode step issued from "
              f"Python, {gms:.3f} ms as a CUDA graph ({b / gms * 1e3:.0f} tokens/s, "
              f"{total_bytes / gms / 1e6:.0f} GB/s of weights)")
        for p in plans:
            lib.nne_qlinear_plan_destroy(p)
    # The same stack as a chain of decoder BLOCKS with the element-wise steps of the reference's
    # Llama2Block (src/models/llama.rs:377-392; attention itself is not part of this path, v stands
    # in for its output): q/k/v read RMSNorm(h), o adds the residual h, gate/up read RMSNorm(h2),
    # down reads silu(gate) * up and adds the residual h2.  (a) fused plans: at batch 1 every launch
    # is the decode kernel, nothing else runs between layers; (b) the same steps as standalone
    # kernels around plain plans.  Batch 8 must agree bit for bit (the fused plan runs the very same
    # kernels), batch 1 within 1e-3 of the hidden state's size after 32 layers (rrms is summed in
    # another order inside the decode kernel).
    g_attn = [torch.ones(H, device=dev) + 0.05 * torch.randn(H, generator=gen, device=dev) for _ in range(LAYERS)]
    g_ffn = [torch.ones(H, device=dev) + 0.05 * torch.randn(H, generator=gen, device=dev) for _ in range(LAYERS)]
    eps = 1e-5
    for b in (1, 8):
        xb = x8[:b].contiguous()
        bufs = {name: torch.empty(b, n, device=dev) for name, n, _ in NAMES}
        hid = [torch.empty(b, H, device=dev), torch.empty(b, H, device=dev)]
        h2 = torch.empty(b, H, device=dev)
        norm, act = torch.empty(b, H, device=dev), torch.empty(b, F, device=dev)
        fused = []
        for li, layer in enumerate(stack):
            src, dst = hid[li % 2], hid[(li + 1) % 2]
            L = {nm: type("L", (), {"_live_handle": (lambda self, h=layer[nm]: h), "_ctx": ctx})() for nm, _, _ in NAMES}
            ga, gf = g_attn[li].data_ptr(), g_ffn[li].data_ptr()
            fused.append(nne.FusedPlan([{"layer": L[nm], "x": src.data_ptr(), "y": bufs[nm].data_ptr(),
                                         "rmsnorm": (ga, eps)} for nm in ("q", "k", "v")], b, ctx))
            fused.append(nne.FusedPlan([{"layer": L["o"], "x": bufs["v"].data_ptr(), "y": h2.data_ptr(),
                                         "residual": src.data_ptr()}], b, ctx))
            fused.append(nne.FusedPlan([{"layer": L[nm], "x": h2.data_ptr(), "y": bufs[nm].data_ptr(),
                                         "rmsnorm": (gf, eps)} for nm in ("gate", "up")], b, ctx))
            fused.append(nne.FusedPlan([{"layer": L["down"], "x": bufs["gate"].data_ptr(), "y": dst.data_ptr(),
                                         "silu_mul": bufs["up"].data_ptr(), "residual": h2.data_ptr()}], b, ctx))
        launches = sum(p.launches for p in fused)

        def fused_step():
            hid[0].copy_(xb)
            for p in fused:
                p.run(stream)
            torch.cuda.synchronize()
            return hid[LAYERS % 2].clone()

        def unfused_step():
            hid[0].copy_(xb)
            for li, layer in enumerate(stack):
                src, dst = hid[li % 2], hid[(li + 1) % 2]
                nne.rmsnorm_device(ctx, src.data_ptr(), g_attn[li].data_ptr(), eps, b, H, norm.data_ptr(), stream)
                for nm in ("q", "k", "v"):
                    fwd(layer[nm], norm, b, H, bufs[nm])
                fwd(layer["o"], bufs["v"], b, H, h2)
                nne.add_device(ctx, h2.data_ptr(), src.data_ptr(), b * H, h2.data_ptr(), stream)
                nne.rmsnorm_device(ctx, h2.data_ptr(), g_ffn[li].data_ptr(), eps, b, H, norm.data_ptr(), stream)
                fwd(layer["gate"], norm, b, H, bufs["gate"])
                fwd(layer["up"], norm, b, H, bufs["up"])
                nne.silu_mul_device(ctx, bufs["gate"].data_ptr(), bufs["up"].data_ptr(), b * F, act.data_ptr(), stream)
                fwd(layer["down"], act, b, F, dst)
                nne.add_device(ctx, dst.data_ptr(), h2.data_ptr(), b * H, dst.data_ptr(), stream)
            torch.cuda.synchronize()
            return hid[LAYERS % 2].clone()

        want = unfused_step()
        got = fused_step()
        ctx.check()
        assert bool(torch.isfinite(got).all()) and bool(torch.isfinite(want).all())
        rel = float((got - want).abs().max() / want.abs().max())
        if b == 8:
            assert torch.equal(got.view(torch.int32), want.view(torch.int32))
        else:
            assert rel <= 1e-3, rel
        t0 = time.perf_counter()
        fused_step()
        dt_f = time.perf_counter() - t0
        t0 = time.perf_counter()
        unfused_step()
        dt_u = time.perf_counter() - t0
        gms = graph_time_ms(torch, lambda st: [hid[0].copy_(xb)] + [p.run(st) for p in fused])
        print(f"config4 batch {b}, decoder blocks with RMSNorm / SiLU*mul / residuals: fused plans "
              f"{dt_f * 1e3:.2f} ms issued from Python, {gms:.3f} ms as a CUDA graph ({launches} launches, "
              f"{b / gms * 1e3:.0f} tokens/s, {total_bytes / gms / 1e6:.0f} GB/s of weights); standalone "
              f"element-wise kernels + one forward per layer {dt_u * 1e3:.2f} ms from Python; "
              f"max |diff| / max |h| = {rel:.2e}")
        # (c) the whole step - all 224 items - as ONE plan: the library finds which items consume
        # which outputs.  Batch 1: a single launch of the decode kernel whose grid meets between the
        # groups while the weight stream runs on; batch 8: the groups one after another.  Same
        # kernels, same arithmetic: the hidden state must not change by a bit.
        items = []
        for li, layer in enumerate(stack):
            src, dst = hid[li % 2], hid[(li + 1) % 2]
            L = {nm: type("L", (), {"_live_handle": (lambda self, h=layer[nm]: h), "_ctx": ctx})() for nm, _, _ in NAMES}
            ga, gf = g_attn[li].data_ptr(), g_ffn[li].data_ptr()
            items += [{"layer": L[nm], "x": src.data_ptr(), "y": bufs[nm].data_ptr(), "rmsnorm": (ga, eps)}
                      for nm in ("q", "k", "v")]
            items.append({"layer": L["o"], "x": bufs["v"].data_ptr(), "y": h2.data_ptr(), "residual": src.data_ptr()})
            items += [{"layer": L[nm], "x": h2.data_ptr(), "y": bufs[nm].data_ptr(), "rmsnorm": (gf, eps)}
                      for nm in ("gate", "up")]
            items.append({"layer": L["down"], "x": bufs["gate"].data_ptr(), "y": dst.data_ptr(),
                          "silu_mul": bufs["up"].data_ptr(), "residual": h2.data_ptr()})
        whole = nne.FusedPlan(items, b, ctx)
        assert whole.launches == (1 if b == 1 else launches)
        hid[0].copy_(xb)
        whole.run(stream)
        torch.cuda.synchronize()
        ctx.check()
        assert torch.equal(hid[LAYERS % 2].view(torch.int32), got.view(torch.int32))
        wms = graph_time_ms(torch, lambda st: [hid[0].copy_(xb), whole.run(st)])
        print(f"config4 batch {b}, the same decoder blocks as ONE plan of {len(items)} items: "
              f"{whole.launches} launch(es), {wms:.3f} ms as a CUDA graph ({b / wms * 1e3:.0f} tokens/s, "
              f"{total_bytes / wms / 1e6:.0f} GB/s of weights)")
        whole.close()
        for p in fused:
            p.close()
    # The 224 layers as INDEPENDENT forwards, each fed its own N(0,1) activation, all in one plan:
    # tokens/s = batch / time of the 224 forwards.
    flat = [(layer[name], n, k) for layer in stack for name, n, k in NAMES]
    cnt = len(flat)
    for b in (1, 8):
        xs = [torch.randn(b, k, generator=gen, device=dev) for _, _, k in flat]
        ys = [torch.empty(b, n, device=dev) for _, n, _ in flat]
        p = C.c_void_p()
        assert lib.nne_qlinear_plan_create(ctx.handle, cnt, (C.c_void_p * cnt)(*[h for h, _, _ in flat]),
                                           (C.c_void_p * cnt)(*[x.data_ptr() for x in xs]),
                                           (C.c_void_p * cnt)(*[y.data_ptr() for y in ys]), b,
                                           C.byref(p)) == 0
        assert lib.nne_qlinear_plan_launches(p) == (1 if b == 1 else 2)
        for _ in range(2):
            assert lib.nne_qlinear_plan_run(p, stream) == 0
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(5):
            assert lib.nne_qlinear_plan_run(p, stream) == 0
        e1.record()
        torch.cuda.synchronize()
        ctx.check()
        dt = e0.elapsed_time(e1) * 1e-3 / 5
        print(f"config4 batch {b}, 224 independent forwards as one plan: {dt * 1e3:.3f} ms, "
              f"{b / dt:.0f} tokens/s, {total_bytes / dt / 1e9:.0f} GB/s of weights")
        for i in (0, 3, 4, 6, 100, 223):   # one of every shape, first and last layer
            h, n, k = flat[i]
            y1 = torch.empty(b, n, device=dev)
            fwd(h, xs[i], b, k, y1)
            torch.cuda.synchronize()
            assert torch.equal(y1.view(torch.int32), ys[i].view(torch.int32)), f"layer {i} differs"
        lib.nne_qlinear_plan_destroy(p)
        del xs, ys
    for layer in stack:
        for h in layer.values():
            lib.nne_qlinear_destroy(h)
