"""Column shards on two GPUs, one process per GPU (torchrun), through the library's shard API:
every rank quantizes and runs its own slice on its own GPU and the slices are exchanged by peer
stores (route 0: fused into the decode kernel at m = 1, a copy kernel otherwise) or by
ncclAllGather (route 1).  The gathered result on EVERY rank must equal the single-GPU forward bit
for bit (same kernels, same per-row arithmetic), run after run with changing activations, and the
shard's codes must equal the full layer's rows.  Skipped on a box with fewer than two GPUs."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r'''
import importlib, os, sys
import numpy as np, torch, torch.distributed as dist
sys.path.insert(0, os.path.join(ROOT, "tests")); sys.path.insert(0, ROOT)
import oracle
nne = importlib.import_module("neural-network-engine_b200")
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dev = torch.device("cuda", rank)
dist.init_process_group("nccl", device_id=dev)
ctx = nne.CudaContext(rank)
group = nne.ShardGroup(ctx, rank, world, 64 << 20)
group.use_nccl()
stream = torch.cuda.current_stream().cuda_stream
ok = True
# (n, k, m): decode kernel with fused stores (m = 1), small-batch and prefill kernels + copy kernel,
# unequal slices and unaligned slice starts (n = 515)
# (m > 16: the tensor-core kernel's epilogue stores its tiles into every window itself)
for (n, k, m) in ((1000, 1024, 1), (4096, 4096, 1), (4096, 4096, 2), (1024, 2048, 8), (768, 512, 40),
                  (1000, 1024, 130), (515, 512, 1), (515, 512, 5), (515, 512, 40)):
    w = oracle.normal(300, n, (n, k), 0.0, 0.015)
    b = oracle.normal(300, n + 1, (n,), 0.0, 0.1)
    full = nne.QLinear.from_linear(nne.Linear(w, b), ctx)
    routes = (nne.ROUTE_PEER_STORES, nne.ROUTE_NCCL) if n % world == 0 else (nne.ROUTE_PEER_STORES,)
    for route in routes:
        sh = nne.ShardedQLinear(nne, w, b, group, max_m=max(64, m), route=route)
        codes = np.array_equal(sh.local.qweight, full.qweight.reshape(n, k)[sh.begin:sh.end].reshape(-1))
        same = True
        for it in range(4):                     # four runs: both output areas twice, new x each time
            x = oracle.normal(301, 10 * m + it, (m, k))
            xd = torch.from_numpy(x).to(dev)
            y = sh.forward(xd, stream)
            torch.cuda.synchronize()
            ctx.check()
            y_one = full.forward(x)
            same = same and np.array_equal(y.cpu().numpy().view(np.uint32), y_one.view(np.uint32))
            dist.barrier()                       # the peer may still read this area: keep runs in step
        ok = ok and same and codes
        print(f"rank {rank}: {k}->{n} M={m} route {route} identical={same} shard codes identical={codes}",
              flush=True)
        sh.close()
# the host entry point of a sharded plan returns the gathered outputs
n, k, m = 2048, 1024, 1
w = oracle.normal(302, 0, (n, k), 0.0, 0.015)
sh = nne.ShardedQLinear(nne, w, None, group, max_m=4)
xbuf = torch.zeros(m, k, device=dev)
plan = nne.ShardedPlan(group, [sh.local], [sh.begin], [n], [xbuf.data_ptr()], [sh._areas[0]], m)
x = oracle.normal(302, 1, (m, k))
y = plan.run_host(x).reshape(m, n)
y_one = nne.QLinear.from_linear(nne.Linear(w, None), ctx).forward(x)
same = np.array_equal(y.view(np.uint32), y_one.view(np.uint32))
print(f"rank {rank}: run_host identical={same}", flush=True)
ok = ok and same
dist.barrier()
plan.close(); sh.close()
torch.cuda.synchronize()
group.close()
dist.destroy_process_group()
sys.exit(0 if ok else 1)
'''


def test_two_gpu_shards_match_single_gpu():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    code = "ROOT = %r\n" % ROOT + CHILD
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
                        "--nproc-per-node=2", "--master-addr", "127.0.0.1", "--master-port", "29611",
                        "--no-python", sys.executable, "-c", code],
                       capture_output=True, text=True, timeout=600, env=env)
    print(r.stdout[-6000:], r.stderr[-3000:])
    assert r.returncode == 0


def test_two_devices_in_one_process(nne):
    """The same exchange with ONE process driving both devices (windows mapped by peer access
    instead of IPC handles): the kernels of the two ranks are launched one after the other from
    this thread and meet on the GPUs."""
    import ctypes as C

    import numpy as np
    import torch

    import oracle
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    lib = nne.load()
    world = 2
    ctxs = [nne.CudaContext(d) for d in range(world)]
    groups = [nne.ShardGroup(ctxs[r], r, world, 8 << 20, connect=False) for r in range(world)]
    table = (C.c_void_p * world)(*[g.handle for g in groups])
    for g in groups:
        assert lib.nne_shard_group_connect_local(g.handle, table) == 0, nne._lib.last_error()
    n, k = 1536, 1024
    w = oracle.normal(310, 0, (n, k), 0.0, 0.02)
    b = oracle.normal(310, 1, (n,), 0.0, 0.1)
    full = nne.QLinear.from_linear(nne.Linear(w, b), ctxs[0])
    shards = [nne.ShardedQLinear(nne, w, b, g, max_m=32) for g in groups]
    for m in (1, 6, 24):
        # one activation buffer per rank, plans and workspaces made before any kernel waits for a peer
        xds = []
        for r in range(world):
            with torch.cuda.device(r):
                xds.append(torch.zeros(m, k, device=f"cuda:{r}"))
                shards[r].prepare(xds[r])
                shards[r].local.forward(np.zeros((m, k), np.float32))
        for it in range(2):
            x = oracle.normal(311, 10 * m + it, (m, k))
            for r in range(world):
                with torch.cuda.device(r):
                    xds[r].copy_(torch.from_numpy(x))
                    torch.cuda.synchronize()
            outs = []
            for r in range(world):
                with torch.cuda.device(r):
                    outs.append((xds[r], shards[r].forward(xds[r], torch.cuda.current_stream().cuda_stream)))
            for r in range(world):
                with torch.cuda.device(r):
                    torch.cuda.synchronize()
                ctxs[r].check()
            y_one = full.forward(x)
            for r in range(world):
                assert np.array_equal(outs[r][1].cpu().numpy().view(np.uint32), y_one.view(np.uint32)), \
                    f"rank {r} m={m} run {it}"
    for s in shards:
        s.close()
    for g in groups:
        g.close()
