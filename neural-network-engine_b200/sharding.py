"""Column sharding of a QLinear over the ranks of one node.

The path shards by output channel: channel j of QLinear::forward reads only row j of `qweight`,
`scales[j]` and `bias[j]` (reference src/nn/quantized.rs:184-192), and the quantize step is per
row (:107-127), so a shard quantized on its own holds bit-identical codes.  Rank g of G owns the
rows [g*N/G, (g+1)*N/G) (the first N % G ranks one more); outputs are exchanged with one NCCL
all-gather (torch.distributed is used for the plumbing only)."""
from __future__ import annotations

from typing import List, Optional, Tuple

import numpy as np


def shard_rows(n: int, world: int, rank: int) -> Tuple[int, int]:
    """[begin, end) of the output rows rank `rank` owns."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad rank {rank} of {world}")
    per, rem = divmod(n, world)
    begin = rank * per + min(rank, rem)
    return begin, begin + per + (1 if rank < rem else 0)


def shard_sizes(n: int, world: int) -> List[int]:
    return [shard_rows(n, world, r)[1] - shard_rows(n, world, r)[0] for r in range(world)]


def assemble(gathered: np.ndarray, n: int, world: int, m: int) -> np.ndarray:
    """Rank-major gathered slices -> row-major [m, n].

    `gathered` is what an all-gather of equally sized (padded) per-rank buffers returns:
    [world, m, width] with width = max shard size; rank g's valid columns are its shard size."""
    width = max(shard_sizes(n, world))
    g = np.asarray(gathered).reshape(world, m, width)
    out = np.empty((m, n), dtype=g.dtype)
    for r in range(world):
        b, e = shard_rows(n, world, r)
        out[:, b:e] = g[r, :, : e - b]
    return out


class ShardedQLinear:
    """One rank's column slice of a QLinear plus the gather.  `forward(x)` returns the full
    [m, out_features] output on every rank."""

    def __init__(self, nne, weight: np.ndarray, bias: Optional[np.ndarray], rank: int, world: int,
                 ctx=None):
        self.out_features, self.in_features = weight.shape
        self.rank, self.world = rank, world
        b, e = shard_rows(self.out_features, world, rank)
        self.begin, self.end = b, e
        self.width = max(shard_sizes(self.out_features, world))
        self.local = nne.QLinear.from_linear(
            nne.Linear(weight[b:e], None if bias is None else bias[b:e]), ctx)

    def forward(self, x_dev, stream: int = 0):
        """x_dev: torch CUDA tensor [m, in_features] (replicated on every rank)."""
        import torch
        import torch.distributed as dist
        m = x_dev.shape[0]
        mine = torch.zeros(m, self.width, device=x_dev.device, dtype=torch.float32)
        if self.end > self.begin:
            self.local.forward_device(x_dev.data_ptr(), m, mine.data_ptr(), stream, ldy=self.width)
        if self.world == 1:
            return mine[:, : self.out_features]
        gathered = torch.empty(self.world, m, self.width, device=x_dev.device, dtype=torch.float32)
        dist.all_gather_into_tensor(gathered.view(-1), mine.view(-1))
        out = torch.empty(m, self.out_features, device=x_dev.device, dtype=torch.float32)
        for r in range(self.world):
            b, e = shard_rows(self.out_features, self.world, r)
            out[:, b:e] = gathered[r, :, : e - b]
        return out
