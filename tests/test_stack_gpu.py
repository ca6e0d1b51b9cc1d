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
        print(f"config4 batch {b}, grouped into plans: {dt * 1e3:.2f} ms per decode step, "
              f"{b / dt:.0f} tokens/s, {total_bytes / dt / 1e9:.0f} GB/s of weights")
        for p in plans:
            lib.nne_qlinear_plan_destroy(p)
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
