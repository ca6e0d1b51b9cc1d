"""Host-side logic of the multi-GPU path on CPU: the row partition, and a world_size-2 gloo run in
which each rank computes its column slice with the CPU oracle, the slices are all-gathered and
the assembled output must equal the unsharded oracle output bit for bit (same per-row arithmetic)."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle


def test_shard_rows_partition(nne):
    for n in (1, 7, 8, 4096, 11008, 28672, 5):
        for world in (1, 2, 3, 4, 8):
            spans = [nne.shard_rows(n, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [e - b for b, e in spans]
            assert max(sizes) - min(sizes) <= 1 and sizes == nne.shard_sizes(n, world)
    with pytest.raises(ValueError):
        nne.shard_rows(8, 2, 2)


def _worker(rank, world, port, n, k, m, ret):
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import importlib
    nne = importlib.import_module("neural-network-engine_b200")
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    w = oracle.normal(200, 0, (n, k), 0.0, 0.015)
    bias = oracle.normal(200, 1, (n,), 0.0, 0.1)
    x = oracle.normal(200, 2, (m, k))
    b, e = nne.shard_rows(n, world, rank)
    q, s = oracle.quantize_rows(w[b:e])                    # a shard quantizes on its own
    y_local = oracle.forward(q, s, bias[b:e], x)           # [m, e-b]
    width = max(nne.shard_sizes(n, world))
    mine = torch.zeros(m, width)
    mine[:, : e - b] = torch.from_numpy(y_local)
    gathered = torch.empty(world, m, width)
    dist.all_gather_into_tensor(gathered.view(-1), mine.view(-1))
    full = nne.assemble(gathered.numpy(), n, world, m)
    qf, sf = oracle.quantize_rows(w)
    y_ref = oracle.forward(qf, sf, bias, x)
    ok = np.array_equal(full.view(np.uint32), y_ref.view(np.uint32)) and \
        np.array_equal(q, qf[b:e]) and np.array_equal(s.view(np.uint32), sf[b:e].view(np.uint32))
    ret[rank] = bool(ok)
    dist.destroy_process_group()


@pytest.mark.parametrize("n,k,m", [(37, 64, 1), (64, 128, 3)])
def test_two_rank_gloo_gather_matches_unsharded(n, k, m):
    world = 2
    port = 29500 + (os.getpid() % 2000)
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, port, n, k, m, ret), nprocs=world, join=True)
        assert all(ret.get(r) for r in range(world))
