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
(weak scaling: per-GPU weight bytes fixed), computes its output slices and the step's slices are
all-gathered over NCCL.

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
RESERVED_SMS = 8  # N > 1: SMs left to the all-gather that runs beside the next step's kernel
PREFILL_M = 2048
# dram__bytes_read.sum + dram__bytes_write.sum of one qgemv_stream_kernel launch over the rotation
# set (read 428.5 MB + write 5.1 MB), from the ncu capture summarised in
# profiles/qgemv_stream_kernel__decode_rotation_set.md.
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
                 "-lms", "20", "-i", str(self.gpu_index)],
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
        sm, mx, reasons = [], [], set()
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
            for nm, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "samples": len(sm),
                "reasons": sorted(reasons)}


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
class RawNccl:
    """ncclAllGather called straight through ctypes on the NCCL library torch has loaded, with a
    communicator of its own (unique id broadcast over torch.distributed).  The c10d wrapper costs
    tens of microseconds of host time per call - more than is left per 73 us step once eight ranks
    share the host's cores; the direct call costs a few."""

    def __init__(self, torch, dist, rank, world, dev):
        path = os.path.join(os.path.dirname(torch.__file__), "..", "nvidia", "nccl", "lib", "libnccl.so.2")
        self.lib = C.CDLL(path if os.path.exists(path) else "libnccl.so.2")

        class UniqueId(C.Structure):
            _fields_ = [("internal", C.c_byte * 128)]

        uid = UniqueId()
        if rank == 0 and self.lib.ncclGetUniqueId(C.byref(uid)) != 0:
            raise RuntimeError("ncclGetUniqueId failed")
        t = torch.tensor(list(bytes(uid)), dtype=torch.uint8, device=dev)
        dist.broadcast(t, 0)
        C.memmove(C.byref(uid), bytes(t.cpu().tolist()), 128)
        self.lib.ncclCommInitRank.argtypes = [C.POINTER(C.c_void_p), C.c_int, UniqueId, C.c_int]
        self.lib.ncclAllGather.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_void_p, C.c_void_p]
        self.comm = C.c_void_p()
        if self.lib.ncclCommInitRank(C.byref(self.comm), world, uid, rank) != 0:
            raise RuntimeError("ncclCommInitRank failed")

    def all_gather_f32(self, send_ptr, recv_ptr, count, stream_ptr):
        if self.lib.ncclAllGather(send_ptr, recv_ptr, count, 7, self.comm, stream_ptr) != 0:  # 7 = ncclFloat32
            raise RuntimeError("ncclAllGather failed")

    def close(self):
        if self.comm:
            self.lib.ncclCommDestroy.argtypes = [C.c_void_p]
            self.lib.ncclCommDestroy(self.comm)
            self.comm = C.c_void_p()


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
        # The all-gather runs beside the next step's kernel on the SMs that kernel leaves free
        # (RESERVED_SMS): cap the collective's CTAs at that number, or it waits for the kernel to
        # end (measured at N = 8 without the cap: 102.8 us per step against 72.7 on one GPU).
        os.environ.setdefault("NCCL_MAX_CTAS", str(RESERVED_SMS))
        # 0.3 MB per rank: the low-latency protocol.  N = 8, us per step: default 107.5, LL128 84.2, LL 107.7.
        os.environ.setdefault("NCCL_PROTO", "LL128")
        dist.init_process_group("nccl", device_id=dev)

    nne = importlib.import_module("neural-network-engine_b200")
    lib = nne.load()
    ctx = nne.CudaContext(local_rank)
    peaks = measured_peaks()

    def make_layer(n, k, seed):
        g = torch.Generator(device=dev)
        g.manual_seed(seed)
        w = torch.randn(n, k, generator=g, device=dev, dtype=torch.float32) * 0.02
        h = C.c_void_p()
        st = lib.nne_qlinear_create_from_f32_dev(ctx.handle, w.data_ptr(), None, n, k,
                                                 torch.cuda.current_stream().cuda_stream, C.byref(h))
        if st != 0:
            raise RuntimeError(f"layer create failed: {nne._lib.last_error()}")
        torch.cuda.synchronize()
        del w
        return h

    # rotation set: REPLICAS independently drawn copies of each shape (this rank's shard when N>1).
    # Outputs of all layers live in one slab per rank, so that N > 1 gathers a step's output
    # slices with a single NCCL all-gather.  N > 1 alternates two slabs: the gather of step i runs
    # on a second stream beside the kernel of step i+1, which writes the other slab.
    specs = [(n, k) for _ in range(REPLICAS) for (n, k) in SHAPES]
    slab_len = sum(n for n, _ in specs)
    overlap = world > 1
    nslabs = 2 if overlap else 1
    gathered = [torch.zeros(world, slab_len, device=dev, dtype=torch.float32) for _ in range(nslabs)]
    own = [g[rank] for g in gathered]
    layers, off = [], 0
    for i, (n, k) in enumerate(specs):
        h = make_layer(n, k, 2 + 1000 * rank + i)
        g = torch.Generator(device=dev)
        g.manual_seed(100 + i)  # activations are replicated: the same on every rank
        x = torch.randn(1, k, generator=g, device=dev, dtype=torch.float32)
        layers.append({"h": h, "n": n, "k": k, "x": x, "off": off, "y_own": own[0][off:off + n]})
        off += n
    step_bytes = sum(algorithmic_bytes(L["n"], L["k"], 1) for L in layers)
    stream = torch.cuda.current_stream()

    # The step as ONE launch: a plan over the whole rotation set (nne_qlinear_plan_*), one plan
    # per output slab.
    nl = len(layers)
    hs = (C.c_void_p * nl)(*[L["h"] for L in layers])
    xs = (C.c_void_p * nl)(*[L["x"].data_ptr() for L in layers])
    plans = []
    for sl in range(nslabs):
        ys = (C.c_void_p * nl)(*[own[sl][L["off"]:L["off"] + L["n"]].data_ptr() for L in layers])
        p = C.c_void_p()
        if lib.nne_qlinear_plan_create(ctx.handle, nl, hs, xs, ys, 1, C.byref(p)) != 0:
            raise RuntimeError(nne._lib.last_error())
        plans.append(p)
    launches_per_step = lib.nne_qlinear_plan_launches(plans[0])
    if overlap:
        # The persistent streaming kernel leaves a few SMs to the collective's CTAs.  Measured at
        # N = 2, microseconds per step: gather on the same stream 83.9; second stream with 0 / 8 / 16
        # SMs left free 80.6 / 80.1 / 82.4.
        if lib.nne_cuda_ctx_reserve_sms(ctx.handle, RESERVED_SMS) != 0:
            raise RuntimeError(nne._lib.last_error())
    comm = torch.cuda.Stream() if overlap else None
    raw = None
    if overlap:
        # every rank must take the same route: agree on whether the direct communicator came up
        try:
            raw = RawNccl(torch, dist, rank, world, dev)
            good = 1
        except Exception:
            raw, good = None, 0
        flag = torch.tensor([good], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if int(flag.item()) == 0:
            if raw is not None:
                raw.close()
            raw = None
    plan_done = [torch.cuda.Event() for _ in range(nslabs)]
    gather_done = [torch.cuda.Event() for _ in range(nslabs)]
    step_no = [0]

    def step():
        sl = step_no[0] % nslabs
        if overlap and step_no[0] >= nslabs:
            stream.wait_event(gather_done[sl])  # the gather that last read this slab is over
        step_no[0] += 1
        if lib.nne_qlinear_plan_run(plans[sl], stream.cuda_stream) != 0:
            raise RuntimeError(nne._lib.last_error())
        if overlap:
            plan_done[sl].record(stream)
            comm.wait_event(plan_done[sl])
            if raw is not None:  # in place: this rank's slice already sits in its slot
                raw.all_gather_f32(own[sl].data_ptr(), gathered[sl].data_ptr(), slab_len, comm.cuda_stream)
            else:
                with torch.cuda.stream(comm):
                    dist.all_gather_into_tensor(gathered[sl].view(-1), own[sl])
            gather_done[sl].record(comm)
        elif world > 1:
            dist.all_gather_into_tensor(gathered[0].view(-1), own[0])

    def drain():
        if overlap:
            for sl in range(min(nslabs, step_no[0])):
                stream.wait_event(gather_done[sl])

    def per_layer_step():
        s = torch.cuda.current_stream().cuda_stream
        for L in layers:
            if lib.nne_qlinear_forward_dev(L["h"], L["x"].data_ptr(), 1, L["k"],
                                           L["y_own"].data_ptr(), s) != 0:
                raise RuntimeError(nne._lib.last_error())

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    drain()
    barrier()

    # device-timed region: K steps back to back on one stream
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    launches0 = lib.nne_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record(stream)
    h0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    host_us_per_step = (time.perf_counter() - h0) * 1e6 / args.steps  # enqueue only, nothing waited for
    drain()
    e1.record(stream)
    barrier()
    launches = lib.nne_launch_count() - launches0
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    clocks = sampler.stop() if rank == 0 else None
    value = step_bytes * world * args.steps / (ms * 1e-3) / 1e9
    per_launch_us = ms * 1e3 / (args.steps * launches_per_step)
    achieved = step_bytes * args.steps / (ms * 1e-3) / 1e9  # one GPU's kernels

    # The same step issued layer by layer (one launch per QLinear, replayed as a CUDA graph so the
    # host's launch cost stays out): what a caller gets without a plan.
    per_layer = None
    if world == 1:
        for _ in range(3):
            per_layer_step()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(stream)
        with torch.cuda.graph(graph, stream=side):
            per_layer_step()  # launches on torch's current stream, which is `side` here
        torch.cuda.synchronize()
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record(stream)
        for _ in range(args.steps):
            graph.replay()
        g1.record(stream)
        torch.cuda.synchronize()
        gms = g0.elapsed_time(g1)
        per_layer = {"value": step_bytes * args.steps / (gms * 1e-3) / 1e9, "unit": "GB/s",
                     "launches_per_step": nl, "avg_launch_us": gms * 1e3 / (args.steps * nl),
                     "launch": "CUDA graph replay of 12 single-layer launches"}

    # end-to-end: host buffers in, host buffers out, H2D and D2H inside every timed step.
    # (1) the step as the plan runs it: nne_qlinear_plan_run_host over one pinned x slab and one
    #     pinned y slab (one copy each way around the one launch);
    # (2) layer by layer through nne_qlinear_forward_host (what QLinear::forward binds to).
    x_total = sum(L["k"] for L in layers)
    y_total = sum(L["n"] for L in layers)
    xslab = torch.empty(x_total, device=dev, dtype=torch.float32)
    yslab = torch.empty(y_total, device=dev, dtype=torch.float32)
    xh_all = torch.empty(x_total, dtype=torch.float32).pin_memory()
    yh_all = torch.empty(y_total, dtype=torch.float32).pin_memory()
    xo = yo = 0
    xps, yps = [], []
    for L in layers:
        xh_all[xo:xo + L["k"]].copy_(L["x"].view(-1).cpu())
        xps.append(xslab.data_ptr() + 4 * xo)
        yps.append(yslab.data_ptr() + 4 * yo)
        xo += L["k"]
        yo += L["n"]
    hplan = C.c_void_p()
    if lib.nne_qlinear_plan_create(ctx.handle, nl, hs, (C.c_void_p * nl)(*xps), (C.c_void_p * nl)(*yps), 1,
                                   C.byref(hplan)) != 0:
        raise RuntimeError(nne._lib.last_error())

    def e2e_step():
        if lib.nne_qlinear_plan_run_host(hplan, xh_all.data_ptr(), yh_all.data_ptr()) != 0:
            raise RuntimeError(nne._lib.last_error())

    host = []
    for L in layers:
        xh = torch.empty(1, L["k"], dtype=torch.float32).pin_memory()
        xh.copy_(L["x"].cpu())
        yh = torch.empty(1, L["n"], dtype=torch.float32).pin_memory()
        host.append((xh, yh))

    def e2e_layer_step():
        for L, (xh, yh) in zip(layers, host):
            st = lib.nne_qlinear_forward_host(L["h"], xh.data_ptr(), 1, L["k"], yh.data_ptr())
            if st != 0:
                raise RuntimeError(nne._lib.last_error())

    def time_host(fn, steps):
        for _ in range(3):
            fn()
        barrier()
        t0 = time.perf_counter()
        for _ in range(steps):
            fn()
        torch.cuda.synchronize()
        sec = time.perf_counter() - t0
        if world > 1:
            t = torch.tensor([sec], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            sec = float(t.item())
        return sec

    e2e_steps = max(args.steps, 5)
    e2e_s = time_host(e2e_step, e2e_steps)
    e2e_layer_s = time_host(e2e_layer_step, min(e2e_steps, 200))
    e2e_value = step_bytes * world * e2e_steps / e2e_s / 1e9
    e2e_layer_value = step_bytes * world * min(e2e_steps, 200) / e2e_layer_s / 1e9
    # the two routes must agree bit for bit
    got = torch.cat([yh.view(-1) for _, yh in host])
    if not torch.equal(got.view(torch.int32), yh_all.view(torch.int32)):
        raise RuntimeError("plan and per-layer host results differ")
    lib.nne_qlinear_plan_destroy(hplan)
    h2d = sum(4 * L["k"] for L in layers)
    d2h = sum(4 * L["n"] for L in layers)

    # decode batch sweep (config 2): one forward per layer over the rotation set, M rows each
    sweep = None
    if world == 1:
        sweep = run_decode_sweep(nne, lib, ctx, dev, layers, args)

    # prefill (M = 2048) on the tensor-core kernel, when it is built in
    prefill = None
    if world == 1:
        prefill = run_prefill(nne, lib, ctx, dev, make_layer, peaks, args)

    # config 4: the 224 QLinears of a 7B-shaped decoder stack as independent forwards in one plan
    stack = None
    if world == 1:
        stack = run_stack(nne, lib, ctx, dev, make_layer, peaks, args)

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
                       "m": 1, "replicas_per_shape": REPLICAS, "layers_per_step": len(layers),
                       "weight_bytes_per_step_per_gpu": sum(L["n"] * L["k"] for L in layers),
                       "l2": "rotation set of distinct weights larger than the 126 MB L2",
                       "launch": "one plan launch per step (nne_qlinear_plan_run), steps back to back",
                       "parallelism": "1 GPU" if world == 1 else
                       f"column shards over {world} GPUs + one NCCL all-gather of the step's output slices"
                       + (f", on a second stream beside the next step's kernel ({RESERVED_SMS} SMs left free for it)"
                          if overlap else "")},
            "roofline": {"bound": "hbm", "kernel": "qgemv_stream_kernel", "achieved": achieved,
                         "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": achieved / peaks["hbm_gbs"], "peak_source": peaks["source"],
                         "frac_of_nominal_8000": achieved / 8000.0,
                         "avg_launch_us": per_launch_us, "launches_per_step": launches_per_step,
                         "algorithmic_bytes_per_launch": step_bytes / launches_per_step,
                         "traffic": DRAM_TRAFFIC_PER_LAUNCH},
            "cpu_baseline": {"value": cpu_v, "unit": "GB/s", "cores": cpu_cores, "kind": "port",
                             "sample": cpu_sample},
            "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "steps": e2e_steps,
                    "api": "nne_qlinear_plan_run_host (pinned host x and y slabs; H2D, one launch, D2H, "
                           "sync in every step)",
                    "per_layer": {"value": e2e_layer_value, "unit": "GB/s",
                                  "api": "nne_qlinear_forward_host, 12 calls per step (per call H2D + "
                                         "launch + D2H + sync)"}},
            "gpu_launches": int(launches),
            "host_enqueue_us_per_step": host_us_per_step,
            "collective": None if world == 1 else ("ncclAllGather called directly (ctypes)" if raw is not None
                                                    else "torch.distributed all_gather_into_tensor"),
            "clocks": clocks,
        }
        if per_layer is not None:
            out["per_layer_launches"] = per_layer
        if sweep is not None:
            out["decode_batch_sweep"] = sweep
        if prefill is not None:
            out["prefill"] = prefill
        if stack is not None:
            out["decoder_stack"] = stack
        print(json.dumps(out))
    if raw is not None:
        torch.cuda.synchronize()
        raw.close()
    for p in plans:
        lib.nne_qlinear_plan_destroy(p)
    for L in layers:
        lib.nne_qlinear_destroy(L["h"])
    if world > 1:
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
    for h in hs:
        lib.nne_qlinear_destroy(h)
    return {"layers": cnt, "weight_bytes": wbytes, "cases": cases,
            "note": "224 independent forwards as one plan (batch 1: streaming GEMV; batch 8: small-batch "
                    "tensor-core kernel)"}


def run_prefill(nne, lib, ctx, dev, make_layer, peaks, args):
    """M = 2048 forward of the two FFN shapes; TFLOP/s = 2*M*N*K / device time."""
    import torch
    res = {"m": PREFILL_M, "shapes_NK": PREFILL_SHAPES, "cases": []}
    stream = torch.cuda.current_stream()
    tot_flops, tot_ms = 0.0, 0.0
    for si, (n, k) in enumerate(PREFILL_SHAPES):
        h = make_layer(n, k, 3 + si)
        kind = lib.nne_qlinear_kernel_for(h, PREFILL_M)
        if kind != 2:
            lib.nne_qlinear_destroy(h)
            return {"unavailable": "tensor-core kernel not built for this shape", "kernel": kind}
        x = torch.randn(PREFILL_M, k, device=dev, dtype=torch.float32)
        y = torch.empty(PREFILL_M, n, device=dev, dtype=torch.float32)

        def fwd():
            st = lib.nne_qlinear_forward_dev(h, x.data_ptr(), PREFILL_M, k, y.data_ptr(),
                                             stream.cuda_stream)
            if st != 0:
                raise RuntimeError(nne._lib.last_error())

        for _ in range(3):
            fwd()
        torch.cuda.synchronize()
        iters = 20 if args.steps >= 20 else max(3, args.steps)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(iters):
            fwd()
        e1.record(stream)
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / iters
        flops = 2.0 * PREFILL_M * n * k
        res["cases"].append({"n": n, "k": k, "ms": ms, "tflops": flops / (ms * 1e-3) / 1e12})
        tot_flops += flops
        tot_ms += ms
        lib.nne_qlinear_destroy(h)
        del x, y
    tf = tot_flops / (tot_ms * 1e-3) / 1e12
    res["roofline"] = {"bound": "tensor", "kernel": "qlinear_prefill_i8_kernel", "achieved": tf,
                       "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                       "frac": tf / peaks["bf16_tflops"], "peak_source": peaks["source"],
                       "frac_of_nominal_2250": tf / 2250.0}
    res["value"] = tf
    res["unit"] = "TFLOP/s"
    res["dtype"] = "s8 x s8 -> s32 (tcgen05 kind::i8; x as two int8 digit planes), f32 epilogue"
    res["roofline"]["note"] = ("peak = measured cuBLAS bf16 GEMM; two int8 digit MMAs at twice the "
                               "bf16 rate cost what one bf16 MMA would")
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_native(args)


if __name__ == "__main__":
    main()
