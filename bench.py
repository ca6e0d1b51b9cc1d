#!/usr/bin/env python
"""Benchmark of the int8 quantized-linear hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl native|reference]

Workload (config.workload): the decode sweep on LLaMA-2-7B-shaped projections at M=1 -
QLinear K->N in {4096->4096, 4096->11008, 11008->4096}, weights ~ N(0, 0.02) quantized per
output channel to int8, f32 activations ~ N(0, 1).  One step = one M=1 forward of every layer
of a rotation set (several independently drawn copies of each shape, > L2 in total) so the
weights come from HBM, not L2.  The layers of a step do not depend on each other, so the step is
issued as one plan (nne_qlinear_plan_run: one kernel launch that streams all the layers); the
same step issued as one launch per layer is reported beside it under "per_layer_launches".
metric = int8-weight streaming rate in GB/s, counting the algorithmic bytes
N*K + 4N + 4K + 4N per forward.  The same line carries the decode batch sweep (M in 1..16, one
forward per layer) under "decode_batch_sweep" and the M=2048 prefill figure (TFLOP/s) under
"prefill".

N > 1 (torchrun, one rank per GPU): every rank holds its own column shard of N-times-wider layers
(weak scaling: per-GPU weight bytes fixed) and a step ends with the gathered outputs on every rank.
The exchange is the library's (nne_qlinear_plan_create_sharded): the decode kernel stores its
results into every rank's window over peer-mapped memory; the NCCL all-gather route is timed beside
it (NNE_BENCH_ROUTE=nccl makes it the headline) and both are checked bit for bit.  "config5" carries
the 70B-shaped FFN sharded over the same GPUs at M=1 and M=2048.

--impl reference times the CPU restatement of the reference's Rayon/AVX2 path (oracle/) on the
host cores: at M=1 the reference's row split gives exactly one task, hence one thread.
"""
import argparse
import ctypes as C
import importlib
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SHAPES = [(4096, 4096), (11008, 4096), (4096, 11008)]  # (N, K)
REPLICAS = 4  # copies of each shape in the rotation set: 4 * 107 MB = 428 MB > 126 MB L2
PREFILL_SHAPES = [(11008, 4096), (4096, 11008)]
DECODE_SWEEP_M = (1, 2, 4, 8, 16)
PREFILL_M = 2048
PREFILL_OTHER_M = (128, 512)
REPEATS_PER_STEP = 100  # plan launches per reported step
CONFIG5_SHAPES = [(28672, 8192), (8192, 28672)]  # LLaMA-70B-shaped FFN: gate/up and down
CONFIG5_M = 2048
# dram__bytes_read.sum + dram__bytes_write.sum of one qgemv_stream_kernel launch over the rotation
# set (read 428.5 MB + write 5.1 MB), from an ncu capture of this kernel on this workload.
DRAM_TRAFFIC_PER_LAUNCH = 433.6e6


def algorithmic_bytes(n, k, m, bias=False):
    return n * k + 4 * n + (4 * n if bias else 0) + 4 * m * k + 4 * m * n


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
            "source": "fallback"}


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-lms", "10", "-i", str(self.gpu_index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, pw, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [t.strip() for t in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            try:
                pw.append(float(f[3]))
            except ValueError:
                pass
            for nm, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "samples": len(sm),
                "power_w_max": max(pw) if pw else None, "reasons": sorted(reasons)}


# ---------------------------------------------------------------------------------------------
# reference arm: the CPU restatement of the reference's path, on the host cores
# ---------------------------------------------------------------------------------------------
def cpu_forward_rate(seconds_budget, reps_cap=1000):
    """Times M=1 forwards of one layer of each shape with the oracle (AVX2 path, one thread: the
    reference parallelises over input rows only, src/nn/quantized.rs:179-182).  Returns
    (GB/s, cores, sample text, seconds of CPU work)."""
    import numpy as np
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle
    rng = np.random.default_rng(2)
    layers = []
    for (n, k) in SHAPES:
        q = rng.integers(-127, 128, size=(n, k), dtype=np.int8)
        s = (np.abs(rng.standard_normal(n)) * 1e-3 + 1e-4).astype(np.float32)
        x = rng.standard_normal((1, k)).astype(np.float32)
        layers.append((q, s, x))
    for (q, s, x) in layers:  # warm-up, also pages the arrays in
        oracle.forward(q, s, None, x, threads=1, use_avx2=-1)
    total_bytes, total_t, reps = 0, 0.0, 0
    while total_t < seconds_budget and reps < reps_cap:
        for (q, s, x) in layers:
            t0 = time.perf_counter()
            oracle.forward(q, s, None, x, threads=1, use_avx2=-1)
            total_t += time.perf_counter() - t0
            total_bytes += algorithmic_bytes(q.shape[0], q.shape[1], 1)
        reps += 1
    avx = bool(oracle.lib().nne_ref_has_avx2_fma())
    sample = (f"{reps} passes of one M=1 forward per shape {SHAPES} "
              f"({'AVX2/FMA' if avx else 'portable'} dot, 1 thread = all the reference's row "
              f"split allows at M=1; host has {os.cpu_count()} cores)")
    return total_bytes / total_t / 1e9, 1, sample, total_t


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import numpy as np
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle
    rng = np.random.default_rng(2)
    layers = []
    for (n, k) in SHAPES:
        q = rng.integers(-127, 128, size=(n, k), dtype=np.int8)
        s = (np.abs(rng.standard_normal(n)) * 1e-3 + 1e-4).astype(np.float32)
        x = rng.standard_normal((1, k)).astype(np.float32)
        layers.append((q, s, x))
    step_bytes = sum(algorithmic_bytes(n, k, 1) for (n, k) in SHAPES)

    def step():
        for (q, s, x) in layers:
            oracle.forward(q, s, None, x, threads=1, use_avx2=-1)

    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = time.perf_counter() - t0
    value = step_bytes * args.steps / dt / 1e9
    sample = ("each step = one M=1 forward of one layer per shape (bounded sample of the rotation "
              "set: 1 of 4 copies); C restatement of the reference's Rayon/AVX2 path, 1 thread "
              f"(the row split gives one task at M=1); host has {os.cpu_count()} cores")
    print(json.dumps({
        "impl": "reference", "metric": "qlinear_int8_weight_stream_rate_m1", "value": value,
        "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "config2-decode-7B-projections-M1", "shapes_NK": SHAPES, "m": 1},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": 1, "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


# ---------------------------------------------------------------------------------------------
# native arm
# ---------------------------------------------------------------------------------------------
def device_time_ms(torch, stream, fn, iters, warm=3):
    """Device time of `iters` calls of fn issued back to back on `stream` (CUDA events)."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(iters):
        fn()
    e1.record(stream)
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def run_native(args):
    import numpy as np
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run, one rank per GPU")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        # the NCCL route moves 0.3 MB per rank and step: the low-latency protocol
        # (N = 8, us per step: default 107.5, LL128 84.2, LL 107.7)
        os.environ.setdefault("NCCL_PROTO", "LL128")
        dist.init_process_group("nccl", device_id=dev)

    nne = importlib.import_module("neural-network-engine_b200")
    lib = nne.load()
    ctx = nne.CudaContext(local_rank)
    peaks = measured_peaks()
    stream = torch.cuda.current_stream()

    def ok(status):
        if status != 0:
            raise RuntimeError(nne._lib.last_error())

    def make_layer(n, k, seed, std=0.02):
        g = torch.Generator(device=dev)
        g.manual_seed(seed)
        w = torch.randn(n, k, generator=g, device=dev, dtype=torch.float32) * std
        h = C.c_void_p()
        ok(lib.nne_qlinear_create_from_f32_dev(ctx.handle, w.data_ptr(), None, n, k,
                                               stream.cuda_stream, C.byref(h)))
        torch.cuda.synchronize()
        del w
        return h

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(v):
        if world == 1:
            return v
        t = torch.tensor([v], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # Rotation set: REPLICAS independently drawn copies of each shape.  N > 1: every layer is this
    # rank's column shard (rows [rank*n, (rank+1)*n)) of a layer `world` times wider - weak scaling -
    # and a step ends with every rank holding the gathered [1, world*n] output of every layer.
    specs = [(n, k) for _ in range(REPLICAS) for (n, k) in SHAPES]
    nl = len(specs)
    y_total = sum(n for n, _ in specs)
    group = None
    route_names = {0: "peer stores from the forward kernel", 1: "ncclAllGather"}
    head_route = 1 if os.environ.get("NNE_BENCH_ROUTE", "").startswith("n") else 0
    if world > 1:
        window = 4 * (12 * world * y_total + 2 * CONFIG5_M * sum(n for n, _ in CONFIG5_SHAPES)) + (64 << 20)
        group = nne.ShardGroup(ctx, rank, world, window)
        group.use_nccl()
    layers = []
    for i, (n, k) in enumerate(specs):
        h = make_layer(n, k, 2 + 1000 * rank + i)
        g = torch.Generator(device=dev)
        g.manual_seed(100 + i)  # activations are replicated: the same on every rank
        x = torch.randn(1, k, generator=g, device=dev, dtype=torch.float32)
        layers.append({"h": h, "n": n, "k": k, "x": x})
    step_bytes = sum(algorithmic_bytes(L["n"], L["k"], 1) for L in layers)
    hs = (C.c_void_p * nl)(*[L["h"] for L in layers])
    xs = (C.c_void_p * nl)(*[L["x"].data_ptr() for L in layers])

    # The step as ONE launch: a plan over the whole rotation set.  One GPU: an ordinary plan.
    # N > 1: sharded plans over AREAS output areas of the window, used in turn.  A run never waits
    # for another rank: the kernel stores its results into every rank's window and announces the
    # rank's previous run; the timed region ends with nne_shard_group_wait, after which every rank
    # holds every slice of every step.  Nothing reads the gathered outputs inside the timed region,
    # so the areas only keep consecutive steps from writing the same addresses.
    AREAS = 4

    def sharded_plans(route, x_ptrs=None, count=AREAS):
        plans, areas = [], []
        for _ in range(count):
            base = group.alloc(world * y_total)
            ptrs, off = [], 0
            for L in layers:
                ptrs.append(base + 4 * off)
                off += world * L["n"]
            p = C.c_void_p()
            rb = (C.c_size_t * nl)(*[rank * L["n"] for L in layers])
            nt = (C.c_size_t * nl)(*[world * L["n"] for L in layers])
            ok(lib.nne_qlinear_plan_create_sharded(group.handle, nl, hs, rb, nt, x_ptrs or xs,
                                                   (C.c_void_p * nl)(*ptrs), 1, route, C.byref(p)))
            plans.append(p)
            areas.append((base, ptrs))
        return plans, areas

    y_local = torch.zeros(y_total, device=dev, dtype=torch.float32)
    yl_ptrs, off = [], 0
    for L in layers:
        L["y_local"] = y_local[off:off + L["n"]]
        yl_ptrs.append(y_local.data_ptr() + 4 * off)
        off += L["n"]
    local_plan = C.c_void_p()
    ok(lib.nne_qlinear_plan_create(ctx.handle, nl, hs, xs, (C.c_void_p * nl)(*yl_ptrs), 1, C.byref(local_plan)))
    if world > 1:
        plans_by_route = {0: sharded_plans(0), 1: sharded_plans(1)}
        plans, areas = plans_by_route[head_route]
    else:
        plans, areas = [local_plan], None
    launches_per_step = lib.nne_qlinear_plan_launches(plans[0])

    def stepper(plan_list, wait=False):
        """Runs the plans in turn on the main stream.  Peer-store route: a run only stores; each run
        announces its predecessor from inside the kernel, and `drain` (nne_shard_group_wait)
        completes the exchange of everything issued so far."""
        turn = [0]

        def step():
            ok(lib.nne_qlinear_plan_run(plan_list[turn[0] % len(plan_list)], stream.cuda_stream))
            turn[0] += 1

        def drain():
            if wait:
                ok(lib.nne_shard_group_wait(group.handle, stream.cuda_stream))
        step.drain = drain
        return step

    step = stepper(plans, wait=(world > 1 and head_route == 0))
    R = max(1, args.repeats)
    for _ in range(max(args.warmup, 3)):
        step()
    step.drain()
    barrier()

    # device-timed region: K steps of R plan launches each, back to back on one stream
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.2)
    launches0 = lib.nne_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record(stream)
    h0 = time.perf_counter()
    marks = []  # an event after every reported step: shows how the rate develops over the timed region
    # Flow control on the host: at most 8 x 32 launches are queued ahead of the GPU.  With some 500
    # launches queued the driver's launch queue fills up, an enqueue then costs the host as long as a
    # kernel runs (55 us instead of 6), and the next launch no longer reaches the GPU before the
    # running kernel lets its dependents go: the programmatic overlap between launches is lost and
    # every launch takes 6-11 us longer (measured per step: 6.62 ms for the first 500 launches, 7.19
    # up to 1000, 7.7 after).  A host that stays 256 launches ahead never starves the GPU.
    pace = []
    for i in range(args.steps * R):
        step()
        if (i + 1) % 32 == 0:
            pe = torch.cuda.Event()
            pe.record(stream)
            pace.append(pe)
            if len(pace) > 8:
                pace.pop(0).synchronize()
        if (i + 1) % R == 0 and (i + 1) < args.steps * R and len(marks) < 63:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record(stream)
            marks.append(ev)
    host_us_per_launch = (time.perf_counter() - h0) * 1e6 / (args.steps * R)  # enqueue only
    step.drain()  # the last runs' slices have arrived on this rank too
    e1.record(stream)
    barrier()
    launches = lib.nne_launch_count() - launches0
    ms = max_over_ranks(e0.elapsed_time(e1))
    edges = [e0] + marks + ([e1] if len(marks) == args.steps - 1 else [])
    step_ms = [round(edges[i].elapsed_time(edges[i + 1]), 4) for i in range(len(edges) - 1)]
    clocks = sampler.stop() if rank == 0 else None
    passes = args.steps * R
    value = step_bytes * world * passes / (ms * 1e-3) / 1e9
    per_launch_us = ms * 1e3 / (passes * launches_per_step)
    achieved = step_bytes * passes / (ms * 1e-3) / 1e9  # one GPU's kernels

    # N > 1, outside the timed region: (1) the same step with no exchange and through the other
    # route, (2) a check of what the exchange delivered.  For (2) every rank draws NEW activations
    # (so that nothing left over from the timed steps can pass), runs one step, and recomputes on
    # its own GPU the slices that two OTHER ranks own in three layers (their weights from the same
    # seeds): those slices of its gathered outputs, and its own, must be bit-identical - channel j
    # reads row j only (src/nn/quantized.rs:184-192), so a shard computes what the full layer would.
    multi = parity = None
    if world > 1:
        iters = max(20, min(passes, 400))
        t_local = max_over_ranks(device_time_ms(torch, stream, stepper([local_plan]), iters))
        barrier()
        other = 1 - head_route
        st_other = stepper(plans_by_route[other][0], wait=(other == 0))

        def other_step():
            st_other()
        t_other = max_over_ranks(device_time_ms(torch, stream, other_step, iters))
        st_other.drain()
        barrier()
        serial_turn = [0]

        def serial_step():
            pl = plans_by_route[0][0]
            ok(lib.nne_qlinear_plan_run(pl[serial_turn[0] % len(pl)], stream.cuda_stream))
            ok(lib.nne_shard_group_wait(group.handle, stream.cuda_stream))
            serial_turn[0] += 1
        t_serial = max_over_ranks(device_time_ms(torch, stream, serial_step, iters))
        barrier()
        multi = {"kernel_only_us_per_step": t_local * 1e3,
                 "peer_stores_run_then_wait_in_one_stream_us_per_step": t_serial * 1e3,
                 "kernel_plus_exchange_us_per_step": ms * 1e3 / passes,
                 "route": route_names[head_route],
                 "other_route": {"route": route_names[other], "us_per_step": t_other * 1e3,
                                 "GB/s": step_bytes * world / (t_other * 1e-3) / 1e9}}
        for i, L in enumerate(layers):
            g = torch.Generator(device=dev)
            g.manual_seed(9000 + i)
            L["x"].copy_(torch.randn(1, L["k"], generator=g, device=dev, dtype=torch.float32))
        checked, identical = 0, True
        for route in (0, 1):
            pl, ar = plans_by_route[route]
            barrier()
            ok(lib.nne_qlinear_plan_run(pl[0], stream.cuda_stream))
            ok(lib.nne_shard_group_wait(group.handle, stream.cuda_stream))
            barrier()
            ctx.check()
            for i in (0, 1, 2):
                L = layers[i]
                got = torch.as_tensor(nne.DeviceArray(ar[0][1][i], (world * L["n"],)), device=dev)
                for r in sorted({rank, (rank + 1) % world, (rank + 2) % world}):
                    h = L["h"] if r == rank else make_layer(L["n"], L["k"], 2 + 1000 * r + i)
                    want = torch.empty(L["n"], device=dev, dtype=torch.float32)
                    ok(lib.nne_qlinear_forward_dev(h, L["x"].data_ptr(), 1, L["k"], want.data_ptr(),
                                                   stream.cuda_stream))
                    torch.cuda.synchronize()
                    same = torch.equal(got[r * L["n"]:(r + 1) * L["n"]].view(torch.int32), want.view(torch.int32))
                    identical = identical and same
                    checked += 1
                    if r != rank:
                        lib.nne_qlinear_destroy(h)
        t = torch.tensor([1 if identical else 0], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        parity = {"checked": checked * world, "identical": bool(int(t.item())),
                  "what": "both routes, fresh activations, 3 layers: own slice and the slices of two other "
                          "ranks recomputed locally from their seeds, bit for bit, on every rank"}
        if not parity["identical"]:
            if rank == 0:
                print(json.dumps({"error": "gathered output differs from the locally recomputed slices",
                                  "parity": parity}))
            sys.exit(3)

    # The same step issued layer by layer (one launch per QLinear, replayed as a CUDA graph so the
    # host's launch cost stays out): what a caller gets without a plan.
    per_layer = None
    if world == 1:
        def per_layer_step():
            s = torch.cuda.current_stream().cuda_stream
            for L in layers:
                ok(lib.nne_qlinear_forward_dev(L["h"], L["x"].data_ptr(), 1, L["k"], L["y_local"].data_ptr(), s))

        for _ in range(3):
            per_layer_step()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(stream)
        with torch.cuda.graph(graph, stream=side):
            per_layer_step()  # launches on torch's current stream, which is `side` here
        torch.cuda.synchronize()
        gms = device_time_ms(torch, stream, graph.replay, max(20, min(passes, 400)))
        per_layer = {"value": step_bytes / (gms * 1e-3) / 1e9, "unit": "GB/s",
                     "frac_of_measured_hbm": step_bytes / (gms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                     "launches_per_step": nl, "avg_launch_us": gms * 1e3 / nl,
                     "launch": "CUDA graph replay of 12 single-layer launches"}

    # end-to-end: host buffers in, host buffers out, H2D and D2H inside every timed step.
    # (1) the step as the plan runs it: nne_qlinear_plan_run_host over one pinned x slab and one
    #     pinned y slab (one copy each way around the one launch); N > 1: the sharded plan, so the
    #     exchange is inside and the GATHERED outputs come back (two plans alternate output areas);
    # (2) layer by layer through nne_qlinear_forward_host (what QLinear::forward binds to).
    x_total = sum(L["k"] for L in layers)
    xslab = torch.empty(x_total, device=dev, dtype=torch.float32)
    xh_all = torch.empty(x_total, dtype=torch.float32).pin_memory()
    yh_all = torch.empty(world * y_total, dtype=torch.float32).pin_memory()
    xo = 0
    xps = []
    for L in layers:
        xh_all[xo:xo + L["k"]].copy_(L["x"].view(-1).cpu())
        xps.append(xslab.data_ptr() + 4 * xo)
        xo += L["k"]
    xps_c = (C.c_void_p * nl)(*xps)
    if world > 1:
        hplans, _ = sharded_plans(head_route, xps_c, count=2)
    else:
        yslab = torch.empty(y_total, device=dev, dtype=torch.float32)
        yps, yo = [], 0
        for L in layers:
            yps.append(yslab.data_ptr() + 4 * yo)
            yo += L["n"]
        hp = C.c_void_p()
        ok(lib.nne_qlinear_plan_create(ctx.handle, nl, hs, xps_c, (C.c_void_p * nl)(*yps), 1, C.byref(hp)))
        hplans = [hp]
    e2e_turn = [0]

    def e2e_step():
        p = hplans[e2e_turn[0] % len(hplans)]
        e2e_turn[0] += 1
        ok(lib.nne_qlinear_plan_run_host(p, xh_all.data_ptr(), yh_all.data_ptr()))

    host = []
    for L in layers:
        xh = torch.empty(1, L["k"], dtype=torch.float32).pin_memory()
        xh.copy_(L["x"].cpu())
        yh = torch.empty(1, L["n"], dtype=torch.float32).pin_memory()
        host.append((xh, yh))

    def e2e_layer_step():
        for L, (xh, yh) in zip(layers, host):
            ok(lib.nne_qlinear_forward_host(L["h"], xh.data_ptr(), 1, L["k"], yh.data_ptr()))

    def time_host(fn, steps):
        for _ in range(3):
            fn()
        barrier()
        t0 = time.perf_counter()
        for _ in range(steps):
            fn()
        torch.cuda.synchronize()
        return max_over_ranks(time.perf_counter() - t0)

    e2e_steps = max(min(passes, 500), 20)
    e2e_s = time_host(e2e_step, e2e_steps)
    e2e_value = step_bytes * world * e2e_steps / e2e_s / 1e9
    e2e_layer_steps = min(e2e_steps, 100)
    e2e_layer = None
    if world == 1:
        e2e_layer_s = time_host(e2e_layer_step, e2e_layer_steps)
        e2e_layer = {"value": step_bytes * e2e_layer_steps / e2e_layer_s / 1e9, "unit": "GB/s",
                     "api": "nne_qlinear_forward_host, 12 calls per step (per call H2D + launch + D2H + sync)"}
        # the two routes must agree bit for bit
        got = torch.cat([yh.view(-1) for _, yh in host])
        if not torch.equal(got.view(torch.int32), yh_all.view(torch.int32)):
            raise RuntimeError("plan and per-layer host results differ")
    else:
        # the gathered outputs that came back must hold this rank's own slices where they belong
        e2e_layer_step()
        off = 0
        for L, (_, yh) in zip(layers, host):
            mine = yh_all[off + rank * L["n"]: off + (rank + 1) * L["n"]]
            if not torch.equal(mine.view(torch.int32), yh.view(-1).view(torch.int32)):
                raise RuntimeError("gathered host result does not hold this rank's slice")
            off += world * L["n"]
    for p in hplans:
        lib.nne_qlinear_plan_destroy(p)
    h2d = sum(4 * L["k"] for L in layers)
    d2h = 4 * world * y_total

    sweep = prefill = stack = quant = config5 = None
    want = set(args.sections.split(","))

    def on(name):
        return "all" in want or name in want
    if world == 1:
        if on("sweep"):
            sweep = run_decode_sweep(nne, lib, ctx, dev, layers, args)          # config 2, M in 1..16
        if on("prefill"):
            prefill = run_prefill(nne, lib, ctx, dev, make_layer, peaks, args)  # config 3
        if on("stack"):
            stack = run_stack(nne, lib, ctx, dev, make_layer, peaks, args)      # config 4
        if on("quantize"):
            quant = run_quantize(nne, lib, ctx, dev, peaks, args)               # QLinear::from_linear
    if on("config5"):
        config5 = run_config5(nne, lib, ctx, dev, group, rank, world, make_layer, peaks, args,
                              barrier, max_over_ranks)

    out = None
    if rank == 0:
        cpu_v, cpu_cores, cpu_sample, _ = cpu_forward_rate(seconds_budget=8.0)
        out = {
            "metric": "qlinear_int8_weight_stream_rate_m1", "value": value, "unit": "GB/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "s8", "data": "synthetic",
            "dtype_note": "int8 weights x int8 digit planes of the f32 activations -> exact int32/int64 "
                          "sums (dp4a), one rounding to f32, f32 scale and bias",
            "config": {"workload": "config2-decode-7B-projections-M1", "shapes_NK": SHAPES,
                       "m": 1, "replicas_per_shape": REPLICAS, "layers_per_pass": len(layers),
                       "passes_per_step": R,
                       "step": f"{R} passes over the rotation set, one plan launch (nne_qlinear_plan_run) per "
                               "pass, back to back: long enough for the clock sampler to see load",
                       "weight_bytes_per_pass_per_gpu": sum(L["n"] * L["k"] for L in layers),
                       "l2": "rotation set of distinct weights larger than the 126 MB L2",
                       "parallelism": "1 GPU" if world == 1 else
                       f"column shards over {world} GPUs, output slices exchanged by {route_names[head_route]}"
                       + ("; steps back to back, one wait for all arrivals closes the timed region"
                          if head_route == 0 else "")},
            "roofline": {"bound": "hbm", "kernel": "qgemv_stream_kernel", "achieved": achieved,
                         "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": achieved / peaks["hbm_gbs"], "peak_source": peaks["source"],
                         "frac_of_nominal_8000": achieved / 8000.0,
                         "avg_launch_us": per_launch_us,
                         "median_launch_us": (statistics.median(step_ms) * 1e3 / (R * launches_per_step)) if step_ms else None,
                         "best_launch_us": (min(step_ms) * 1e3 / (R * launches_per_step)) if step_ms else None,
                         "launches_per_pass": launches_per_step,
                         "algorithmic_bytes_per_launch": step_bytes / launches_per_step,
                         "traffic": DRAM_TRAFFIC_PER_LAUNCH,
                         "traffic_source": "ncu capture of this kernel on this workload at one GPU (a constant, "
                                           "not measured in this run)"},
            "cpu_baseline": {"value": cpu_v, "unit": "GB/s", "cores": cpu_cores, "kind": "port",
                             "sample": cpu_sample},
            "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "steps": e2e_steps,
                    "api": "nne_qlinear_plan_run_host (pinned host x and y slabs; x host->device, one launch"
                           + (", exchange of the output slices" if world > 1 else "")
                           + ", y device->host, sync in every pass; at one GPU the two copies are made by "
                             "copy kernels reading and writing the pinned memory over PCIe, chained to the forward)"},
            "gpu_launches": int(launches),
            "host_enqueue_us_per_launch": host_us_per_launch,
            "step_ms": step_ms,
            "clocks": clocks,
        }
        if e2e_layer is not None:
            out["e2e"]["per_layer"] = e2e_layer
        for key, val in (("multi_gpu", multi), ("parity", parity), ("per_layer_launches", per_layer),
                         ("decode_batch_sweep", sweep), ("prefill", prefill), ("decoder_stack", stack),
                         ("quantize", quant), ("config5", config5)):
            if val is not None:
                out[key] = val
        print(json.dumps(out))
    torch.cuda.synchronize()
    lib.nne_qlinear_plan_destroy(local_plan)
    if world > 1:
        for route in (0, 1):
            for p in plans_by_route[route][0]:
                lib.nne_qlinear_plan_destroy(p)
    for L in layers:
        lib.nne_qlinear_destroy(L["h"])
    if world > 1:
        barrier()
        group.close()
        dist.destroy_process_group()


def run_decode_sweep(nne, lib, ctx, dev, layers, args):
    """M in {1, 2, 4, 8, 16}: forwards of the 12-layer rotation set, (a) issued one layer at a time
    back to back on one stream, (b) as one plan over the 12 layers; GB/s = algorithmic bytes /
    device time."""
    import torch
    stream = torch.cuda.current_stream()
    cases = []
    for m in DECODE_SWEEP_M:
        xs = [torch.randn(m, L["k"], device=dev, dtype=torch.float32) for L in layers]
        ys = [torch.empty(m, L["n"], device=dev, dtype=torch.float32) for L in layers]

        def sweep_step():
            for L, x, y in zip(layers, xs, ys):
                if lib.nne_qlinear_forward_dev(L["h"], x.data_ptr(), m, L["k"], y.data_ptr(),
                                               stream.cuda_stream) != 0:
                    raise RuntimeError(nne._lib.last_error())

        for _ in range(3):
            sweep_step()
        torch.cuda.synchronize()
        iters = 20 if args.steps >= 20 else max(3, args.steps)
        l0 = lib.nne_launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(iters):
            sweep_step()
        e1.record(stream)
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / iters
        nbytes = sum(algorithmic_bytes(L["n"], L["k"], m) for L in layers)
        launches = (lib.nne_launch_count() - l0) / (iters * len(layers))
        # (b) the same 12 forwards as one plan
        nl = len(layers)
        plan = C.c_void_p()
        if lib.nne_qlinear_plan_create(ctx.handle, nl, (C.c_void_p * nl)(*[L["h"] for L in layers]),
                                       (C.c_void_p * nl)(*[x.data_ptr() for x in xs]),
                                       (C.c_void_p * nl)(*[y.data_ptr() for y in ys]), m, C.byref(plan)) != 0:
            raise RuntimeError(nne._lib.last_error())
        for _ in range(3):
            lib.nne_qlinear_plan_run(plan, stream.cuda_stream)
        torch.cuda.synchronize()
        p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        p0.record(stream)
        for _ in range(iters):
            if lib.nne_qlinear_plan_run(plan, stream.cuda_stream) != 0:
                raise RuntimeError(nne._lib.last_error())
        p1.record(stream)
        torch.cuda.synchronize()
        pms = p0.elapsed_time(p1) / iters
        plan_launches = lib.nne_qlinear_plan_launches(plan)
        lib.nne_qlinear_plan_destroy(plan)
        cases.append({"m": m, "GB/s": nbytes / (ms * 1e-3) / 1e9, "us_per_layer": ms * 1e3 / len(layers),
                      "kernel": int(lib.nne_qlinear_kernel_for(layers[0]["h"], m)),
                      "launches_per_layer": launches,
                      "plan_GB/s": nbytes / (pms * 1e-3) / 1e9, "plan_us_per_step": pms * 1e3,
                      "plan_launches_per_step": int(plan_launches)})
    return {"cases": cases, "launch": "GB/s: one forward per layer, back to back (no plan, no graph); "
                                      "plan_GB/s: the 12 forwards as one plan",
            "kernels": {"1": "qgemv_stream_kernel", "4": "qlinear_skinny_i8_kernel"}}


def run_stack(nne, lib, ctx, dev, make_layer, peaks, args):
    """Config 4: 32 layers x {q, k, v, o: 4096->4096; gate, up: 4096->11008; down: 11008->4096} = 224
    QLinears (6.5 GB of int8 codes), each fed its own N(0,1) activation of B rows, all 224 forwards
    in one plan; tokens/s = B / device time."""
    import torch
    shapes = ([(4096, 4096)] * 4 + [(11008, 4096)] * 2 + [(4096, 11008)]) * 32
    hs = [make_layer(n, k, 4000 + i) for i, (n, k) in enumerate(shapes)]
    cnt = len(hs)
    wbytes = sum(n * k for n, k in shapes)
    stream = torch.cuda.current_stream()
    cases = []
    for b in (1, 8):
        xs = [torch.randn(b, k, device=dev, dtype=torch.float32) for _, k in shapes]
        ys = [torch.empty(b, n, device=dev, dtype=torch.float32) for n, _ in shapes]
        plan = C.c_void_p()
        if lib.nne_qlinear_plan_create(ctx.handle, cnt, (C.c_void_p * cnt)(*hs),
                                       (C.c_void_p * cnt)(*[x.data_ptr() for x in xs]),
                                       (C.c_void_p * cnt)(*[y.data_ptr() for y in ys]), b, C.byref(plan)) != 0:
            raise RuntimeError(nne._lib.last_error())
        for _ in range(3):
            lib.nne_qlinear_plan_run(plan, stream.cuda_stream)
        torch.cuda.synchronize()
        iters = 10 if args.steps >= 10 else max(3, args.steps)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(iters):
            if lib.nne_qlinear_plan_run(plan, stream.cuda_stream) != 0:
                raise RuntimeError(nne._lib.last_error())
        e1.record(stream)
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / iters
        nbytes = sum(algorithmic_bytes(n, k, b) for n, k in shapes)
        gbs = nbytes / (ms * 1e-3) / 1e9
        cases.append({"batch": b, "ms": ms, "tokens_per_s": b / (ms * 1e-3), "GB/s": gbs,
                      "frac_of_measured_hbm": gbs / peaks["hbm_gbs"],
                      "launches": int(lib.nne_qlinear_plan_launches(plan))})
        lib.nne_qlinear_plan_destroy(plan)
        del xs, ys
    # The same 224 layers as what a decode step really is: a CHAIN of 32 decoder blocks, every
    # layer fed by the ones before it, with the block's RMSNorm / SiLU*mul / residual steps
    # (reference src/models/llama.rs:377-392, 343-346) fused into the forwards - ONE plan of 224
    # dependent items (attention itself is not part of this path: v stands in for its output).
    chained = []
    H, F = 4096, 11008
    gam = [torch.ones(H, device=dev) + 0.05 * torch.randn(H, device=dev) for _ in range(64)]
    try:
        for b in (1, 8):
            x0 = torch.randn(b, H, device=dev)
            hid = [torch.empty(b, H, device=dev), torch.empty(b, H, device=dev)]
            h2 = torch.empty(b, H, device=dev)
            buf = {nm: torch.empty(b, n, device=dev) for nm, n in (("q", H), ("k", H), ("v", H), ("gate", F), ("up", F))}
            items = (nne._lib.PlanItem * cnt)()
            for li in range(32):
                src, dst = hid[li % 2], hid[(li + 1) % 2]
                q, k, v, o, gate, up, down = hs[7 * li:7 * li + 7]
                spec = [(q, src, buf["q"], 1, gam[2 * li], None, None), (k, src, buf["k"], 1, gam[2 * li], None, None),
                        (v, src, buf["v"], 1, gam[2 * li], None, None), (o, buf["v"], h2, 0, None, None, src),
                        (gate, h2, buf["gate"], 1, gam[2 * li + 1], None, None), (up, h2, buf["up"], 1, gam[2 * li + 1], None, None),
                        (down, buf["gate"], dst, 2, None, buf["up"], h2)]
                for j, (h, x, y, op, g, x2, res) in enumerate(spec):
                    it = items[7 * li + j]
                    it.layer, it.x, it.y, it.input_op, it.eps = getattr(h, "value", h), x.data_ptr(), y.data_ptr(), op, 1e-5
                    it.gamma = g.data_ptr() if g is not None else None
                    it.x2 = x2.data_ptr() if x2 is not None else None
                    it.residual = res.data_ptr() if res is not None else None
            plan = C.c_void_p()
            if lib.nne_qlinear_plan_create_fused(ctx.handle, cnt, items, b, C.byref(plan)) != 0:
                raise RuntimeError(nne._lib.last_error())

            def step():
                hid[0].copy_(x0)
                if lib.nne_qlinear_plan_run(plan, stream.cuda_stream) != 0:
                    raise RuntimeError(nne._lib.last_error())
            for _ in range(3):
                step()
            torch.cuda.synchronize()
            iters = 10 if args.steps >= 10 else max(3, args.steps)
            ms = device_time_ms(torch, stream, step, iters)
            finite = bool(torch.isfinite(hid[0]).all())
            nbytes = sum(algorithmic_bytes(n, k, b) for n, k in shapes)
            chained.append({"batch": b, "ms": ms, "tokens_per_s": b / (ms * 1e-3), "GB/s": nbytes / (ms * 1e-3) / 1e9,
                            "launches": int(lib.nne_qlinear_plan_launches(plan)), "finite": finite})
            lib.nne_qlinear_plan_destroy(plan)
    except RuntimeError as e:  # reported, not fatal: the headline figures above stand on their own
        chained.append({"unavailable": str(e)[:200]})
    for h in hs:
        lib.nne_qlinear_destroy(h)
    return {"layers": cnt, "weight_bytes": wbytes, "cases": cases, "chained": chained,
            "note": "cases: 224 independent forwards as one plan (batch 1: streaming GEMV; batch 8: small-batch "
                    "tensor-core kernel).  chained: the same layers as 32 decoder blocks in dependency order "
                    "with RMSNorm, SiLU*mul and residuals fused, one plan of 224 dependent items issued from "
                    "the host (batch 1: one launch; batch 8: its groups one after another)"}


def run_prefill(nne, lib, ctx, dev, make_layer, peaks, args):
    """Config 3.  M = 2048 forward of the two FFN shapes, TFLOP/s = 2*M*N*K / device time, timed
    (a) as a burst of 20 forwards, (b) looped for more than a second with the SM clock sampled
    (against the sustained bf16 figure), (c) end to end from pinned host memory; M = 128 and 512
    beside it."""
    import torch
    res = {"m": PREFILL_M, "shapes_NK": PREFILL_SHAPES, "cases": []}
    stream = torch.cuda.current_stream()
    tot_flops, tot_ms = 0.0, 0.0
    hs = []
    for si, (n, k) in enumerate(PREFILL_SHAPES):
        h = make_layer(n, k, 3 + si)
        kind = lib.nne_qlinear_kernel_for(h, PREFILL_M)
        if kind != 2:
            lib.nne_qlinear_destroy(h)
            return {"unavailable": "tensor-core kernel not built for this shape", "kernel": kind}
        hs.append(h)
    xs = [torch.randn(PREFILL_M, k, device=dev, dtype=torch.float32) for _, k in PREFILL_SHAPES]
    ys = [torch.empty(PREFILL_M, n, device=dev, dtype=torch.float32) for n, _ in PREFILL_SHAPES]

    def fwd(i, m=PREFILL_M):
        n, k = PREFILL_SHAPES[i]
        if lib.nne_qlinear_forward_dev(hs[i], xs[i].data_ptr(), m, k, ys[i].data_ptr(), stream.cuda_stream) != 0:
            raise RuntimeError(nne._lib.last_error())

    iters = 20 if args.steps >= 20 else max(3, args.steps)
    for i, (n, k) in enumerate(PREFILL_SHAPES):
        ms = device_time_ms(torch, stream, lambda: fwd(i), iters)
        flops = 2.0 * PREFILL_M * n * k
        res["cases"].append({"n": n, "k": k, "ms": ms, "tflops": flops / (ms * 1e-3) / 1e12})
        tot_flops += flops
        tot_ms += ms
    tf = tot_flops / (tot_ms * 1e-3) / 1e12
    res["roofline"] = {"bound": "tensor", "kernel": "qlinear_prefill_i8_kernel", "achieved": tf,
                       "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                       "frac": tf / peaks["bf16_tflops"], "peak_source": peaks["source"],
                       "frac_of_nominal_2250": tf / 2250.0,
                       "timing": f"burst: {iters} forwards per shape back to back",
                       "note": "peak = measured cuBLAS bf16 GEMM; two int8 digit MMAs at twice the "
                               "bf16 rate cost what one bf16 MMA would"}
    res["value"] = tf
    res["unit"] = "TFLOP/s"
    res["dtype"] = "s8 x s8 -> s32 (tcgen05 kind::i8; x as two int8 digit planes), f32 epilogue"

    # (b) sustained: both shapes alternating for > 1 s, clocks sampled meanwhile
    per_pair_ms = tot_ms
    loops = max(10, int(1200.0 / per_pair_ms)) if args.steps >= 20 else 10
    sampler = ClockSampler(dev.index or 0)
    sampler.start()
    time.sleep(0.1)

    def pair():
        fwd(0)
        fwd(1)

    sms = device_time_ms(torch, stream, pair, loops, warm=2)
    clocks = sampler.stop()
    stf = tot_flops / (sms * 1e-3) / 1e12
    res["sustained"] = {"value": stf, "unit": "TFLOP/s", "seconds": sms * loops * 1e-3, "forwards": 2 * loops,
                        "peak": peaks["bf16_tflops_sustained"], "frac": stf / peaks["bf16_tflops_sustained"],
                        "frac_of_burst_peak": stf / peaks["bf16_tflops"], "frac_of_nominal_2250": stf / 2250.0,
                        "peak_source": peaks["source"] + " (cuBLAS bf16, seconds-long loop)", "clocks": clocks}

    # (c) end to end from pinned host memory through nne_qlinear_forward_host (4096 -> 11008)
    n, k = PREFILL_SHAPES[0]
    xh = torch.randn(PREFILL_M, k, dtype=torch.float32).pin_memory()
    yh = torch.empty(PREFILL_M, n, dtype=torch.float32).pin_memory()
    reps = 5 if args.steps >= 20 else 2
    for _ in range(2):
        lib.nne_qlinear_forward_host(hs[0], xh.data_ptr(), PREFILL_M, k, yh.data_ptr())
    t0 = time.perf_counter()
    for _ in range(reps):
        if lib.nne_qlinear_forward_host(hs[0], xh.data_ptr(), PREFILL_M, k, yh.data_ptr()) != 0:
            raise RuntimeError(nne._lib.last_error())
    sec = (time.perf_counter() - t0) / reps
    res["e2e"] = {"value": 2.0 * PREFILL_M * n * k / sec / 1e12, "unit": "TFLOP/s", "ms": sec * 1e3,
                  "h2d_bytes_per_step": 4 * PREFILL_M * k, "d2h_bytes_per_step": 4 * PREFILL_M * n,
                  "api": "nne_qlinear_forward_host, 4096->11008, pinned host x and y"}

    # the smaller batches of config 3 (same layers, first M rows of the same activations)
    res["other_m"] = []
    for m in PREFILL_OTHER_M:
        f, t = 0.0, 0.0
        for i, (n, k) in enumerate(PREFILL_SHAPES):
            ms = device_time_ms(torch, stream, lambda: fwd(i, m), iters)
            f += 2.0 * m * n * k
            t += ms
        v = f / (t * 1e-3) / 1e12
        res["other_m"].append({"m": m, "tflops": v, "frac": v / peaks["bf16_tflops"], "us_both_shapes": t * 1e3})
    for h in hs:
        lib.nne_qlinear_destroy(h)
    return res


def run_quantize(nne, lib, ctx, dev, peaks, args):
    """QLinear::from_linear's row loop on the device (nne_quantize_rows_dev): f32 [N, K] in, int8
    codes and f32 scales out; algorithmic bytes 4NK + NK + 4N; launches back to back over three
    matrices of each shape so that the input comes from HBM."""
    import torch
    stream = torch.cuda.current_stream()
    cases = []
    for (n, k) in ((11008, 4096), (4096, 11008), (28672, 8192)):
        ws = [torch.randn(n, k, device=dev, dtype=torch.float32) * 0.02 for _ in range(3)]
        q = torch.empty(n, k, device=dev, dtype=torch.int8)
        sc = torch.empty(n, device=dev, dtype=torch.float32)
        turn = [0]

        def run():
            w = ws[turn[0] % 3]
            turn[0] += 1
            if lib.nne_quantize_rows_dev(ctx.handle, w.data_ptr(), n, k, q.data_ptr(), sc.data_ptr(),
                                         stream.cuda_stream) != 0:
                raise RuntimeError(nne._lib.last_error())

        ms = device_time_ms(torch, stream, run, 12)
        nbytes = 5 * n * k + 4 * n
        gbs = nbytes / (ms * 1e-3) / 1e9
        cases.append({"n": n, "k": k, "us": ms * 1e3, "GB/s": gbs, "frac_of_measured_hbm": gbs / peaks["hbm_gbs"]})
        del ws, q, sc
    return {"kernel": "quantize_rows_bulk_kernel", "cases": cases,
            "bytes": "4*N*K read + N*K + 4*N written per launch"}


def run_config5(nne, lib, ctx, dev, group, rank, world, make_layer, peaks, args, barrier, max_over_ranks):
    """Config 5: LLaMA-70B-shaped FFN projections (8192 -> 28672, 28672 -> 8192; weights N(0, 0.015)),
    column-sharded over the run's GPUs (strong scaling: the layer is fixed, a rank owns 1/N of its
    rows), at M = 1 and M = 2048.  Per case: the forward kernels alone, and forward + exchange through
    both routes; the gathered output is checked against a local recomputation of another rank's
    slice (bit for bit)."""
    import torch
    stream = torch.cuda.current_stream()
    cases = []
    for si, (n_total, k) in enumerate(CONFIG5_SHAPES):
        n = n_total // world
        h = make_layer(n, k, 5000 + 100 * si + rank, std=0.015)
        peer = (rank + 1) % world
        h_peer = make_layer(n, k, 5000 + 100 * si + peer, std=0.015) if world > 1 else None
        g = torch.Generator(device=dev)
        g.manual_seed(50 + si)
        x = torch.randn(CONFIG5_M, k, generator=g, device=dev, dtype=torch.float32)
        y_local = torch.empty(CONFIG5_M, n, device=dev, dtype=torch.float32)
        areas = None
        if world > 1:
            areas = [group.alloc(CONFIG5_M * n_total) for _ in range(2)]
        for m in (1, CONFIG5_M):
            def local():
                if lib.nne_qlinear_forward_dev(h, x.data_ptr(), m, k, y_local.data_ptr(), stream.cuda_stream) != 0:
                    raise RuntimeError(nne._lib.last_error())

            iters = 20 if args.steps >= 20 else 3
            barrier()
            t_local = max_over_ranks(device_time_ms(torch, stream, local, iters))
            case = {"n_total": n_total, "k": k, "m": m, "rows_per_gpu": n,
                    "kernel": int(lib.nne_qlinear_kernel_for(h, m)), "kernel_only_us": t_local * 1e3}
            flops = 2.0 * m * n_total * k
            nbytes = algorithmic_bytes(n_total, k, m)
            if world > 1:
                for route, name in ((0, "peer_stores"), (1, "nccl")):
                    plans = []
                    for a in areas:
                        p = C.c_void_p()
                        if lib.nne_qlinear_plan_create_sharded(
                                group.handle, 1, (C.c_void_p * 1)(h), (C.c_size_t * 1)(rank * n),
                                (C.c_size_t * 1)(n_total), (C.c_void_p * 1)(x.data_ptr()),
                                (C.c_void_p * 1)(a), m, route, C.byref(p)) != 0:
                            raise RuntimeError(nne._lib.last_error())
                        plans.append(p)
                    turn = [0]

                    def run():
                        # run, then the arrival wait on the same stream: what a consumer of the
                        # gathered output sees (nothing is overlapped with the next forward)
                        p = plans[turn[0] & 1]
                        turn[0] += 1
                        if lib.nne_qlinear_plan_run(p, stream.cuda_stream) != 0:
                            raise RuntimeError(nne._lib.last_error())
                        if route == 0 and lib.nne_shard_group_wait(group.handle, stream.cuda_stream) != 0:
                            raise RuntimeError(nne._lib.last_error())

                    barrier()
                    t = max_over_ranks(device_time_ms(torch, stream, run, iters))
                    barrier()
                    ctx.check()
                    case[name + "_us"] = t * 1e3
                    # the last run went to area (turn-1)&1: the peer's slice there against a local recomputation
                    got = torch.as_tensor(nne.DeviceArray(areas[(turn[0] - 1) & 1], (m, n_total)), device=dev)
                    want = torch.empty(m, n, device=dev, dtype=torch.float32)
                    if lib.nne_qlinear_forward_dev(h_peer, x.data_ptr(), m, k, want.data_ptr(), stream.cuda_stream) != 0:
                        raise RuntimeError(nne._lib.last_error())
                    torch.cuda.synchronize()
                    same = torch.equal(got[:, peer * n:(peer + 1) * n].contiguous().view(torch.int32),
                                       want.view(torch.int32))
                    flag = torch.tensor([1 if same else 0], device=dev)
                    import torch.distributed as dist
                    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
                    case[name + "_identical"] = bool(int(flag.item()))
                    for p in plans:
                        lib.nne_qlinear_plan_destroy(p)
                    barrier()
                if not (case["peer_stores_identical"] and case["nccl_identical"]):
                    if rank == 0:
                        print(json.dumps({"error": "config 5: gathered output differs", "case": case}))
                    sys.exit(3)
            t_best = case.get("peer_stores_us", case["kernel_only_us"]) * 1e-6
            if m == 1:
                case["GB/s_kernel_only"] = nbytes / (case["kernel_only_us"] * 1e-6) / 1e9
                case["GB/s"] = nbytes / t_best / 1e9
                case["frac_of_measured_hbm_per_gpu"] = case["GB/s"] / world / peaks["hbm_gbs"]
            else:
                case["TFLOP/s_kernel_only"] = flops / (case["kernel_only_us"] * 1e-6) / 1e12
                case["TFLOP/s"] = flops / t_best / 1e12
                case["frac_of_measured_bf16_per_gpu"] = case["TFLOP/s"] / world / peaks["bf16_tflops"]
                if world > 1:
                    # what the exchange must move: every rank receives the other ranks' slices
                    recv = 4.0 * m * (n_total - n)
                    case["nvlink_floor_us"] = recv / 770e9 * 1e6
            cases.append(case)
        lib.nne_qlinear_destroy(h)
        if h_peer is not None:
            lib.nne_qlinear_destroy(h_peer)
        del x, y_local
    return {"n_gpus": world, "scaling": "strong", "cases": cases,
            "note": "us = max over ranks of the device time per forward (+ exchange); GB/s and TFLOP/s are "
                    "whole-layer figures over that time; nvlink_floor_us = bytes a rank must receive / 770 GB/s"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--repeats", type=int, default=REPEATS_PER_STEP,
                    help="plan launches per reported step (1 for a short run under a profiler)")
    ap.add_argument("--sections", default="all",
                    help="comma list of the extra sections to run besides the headline workload: "
                         "sweep,prefill,stack,quantize,config5 (a short list keeps a profiler capture small)")
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_native(args)


if __name__ == "__main__":
    main()
