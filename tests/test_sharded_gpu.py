"""Two-GPU run of the column-sharded layer: every rank quantizes and runs its own slice on its own
GPU, the slices are all-gathered over NCCL, and the result must equal the single-GPU forward bit
for bit (same kernel, same per-row arithmetic).  Skipped on a box with fewer than two GPUs."""
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
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
ctx = nne.CudaContext(rank)
ok = True
for (n, k, m) in ((1000, 1024, 1), (4096, 4096, 2), (515, 512, 40)):
    w = oracle.normal(300, n, (n, k), 0.0, 0.015)
    b = oracle.normal(300, n + 1, (n,), 0.0, 0.1)
    x = oracle.normal(301, m, (m, k))
    sh = nne.ShardedQLinear(nne, w, b, rank, world, ctx)
    y = sh.forward(torch.from_numpy(x).cuda(), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    full = nne.QLinear.from_linear(nne.Linear(w, b), ctx)
    y_one = full.forward(x)
    same = np.array_equal(y.cpu().numpy().view(np.uint32), y_one.view(np.uint32))
    codes = np.array_equal(sh.local.qweight, full.qweight.reshape(n, k)[sh.begin:sh.end].reshape(-1))
    ok = ok and same and codes
    print(f"rank {rank}: {k}->{n} M={m} identical={same} shard codes identical={codes}", flush=True)
dist.barrier()
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
    print(r.stdout[-3000:], r.stderr[-3000:])
    assert r.returncode == 0
