"""Column sharding of a QLinear over the GPUs of one node: host mirror of the library's shard API.

The path shards by output channel: channel j of QLinear::forward reads only row j of `qweight`,
`scales[j]` and `bias[j]` (reference src/nn/quantized.rs:184-192), and the quantize step is per
row (:107-127), so a shard quantized on its own holds bit-identical codes.  Rank g of G owns the
rows [g*N/G, (g+1)*N/G) (the first N % G ranks one more).

Everything that computes or moves data is the library's (`nne_shard_group_*`,
`nne_qlinear_plan_create_sharded`): the forward kernels store their output slices into every
rank's window over peer-mapped memory, or - route 1 - the slices are exchanged with
`ncclAllGather`.  `torch.distributed` is used here only to carry the 64-byte window handles and
the NCCL unique id from rank to rank."""
from __future__ import annotations

import ctypes as C
import os
from typing import List, Optional, Tuple

import numpy as np

from . import _lib
from ._lib import NneError, check, load

ROUTE_PEER_STORES, ROUTE_NCCL = 0, 1


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


class DeviceArray:
    """A view of device memory for consumers of the CUDA array interface
    (`torch.as_tensor(DeviceArray(ptr, shape), device="cuda")` aliases it without a copy)."""

    def __init__(self, ptr: int, shape, typestr: str = "<f4"):
        self.__cuda_array_interface__ = {"shape": tuple(int(s) for s in shape), "typestr": typestr,
                                         "data": (int(ptr), False), "version": 2}


class NcclComm:
    """An NCCL communicator of this rank, made through ctypes on the NCCL library the process has
    loaded (torch's); the unique id travels over torch.distributed.  Host plumbing for route 1:
    the library receives the communicator as an opaque pointer."""

    def __init__(self, rank: int, world: int, device):
        import torch
        import torch.distributed as dist
        path = os.path.join(os.path.dirname(torch.__file__), "..", "nvidia", "nccl", "lib", "libnccl.so.2")
        self.lib = C.CDLL(path if os.path.exists(path) else "libnccl.so.2")

        class UniqueId(C.Structure):
            _fields_ = [("internal", C.c_byte * 128)]

        uid = UniqueId()
        if rank == 0 and self.lib.ncclGetUniqueId(C.byref(uid)) != 0:
            raise RuntimeError("ncclGetUniqueId failed")
        t = torch.tensor(list(bytes(uid)), dtype=torch.uint8, device=device)
        dist.broadcast(t, 0)
        C.memmove(C.byref(uid), bytes(t.cpu().tolist()), 128)
        self.lib.ncclCommInitRank.argtypes = [C.POINTER(C.c_void_p), C.c_int, UniqueId, C.c_int]
        self.comm = C.c_void_p()
        if self.lib.ncclCommInitRank(C.byref(self.comm), world, uid, rank) != 0:
            raise RuntimeError("ncclCommInitRank failed")

    def close(self):
        if self.comm:
            self.lib.ncclCommDestroy.argtypes = [C.c_void_p]
            self.lib.ncclCommDestroy(self.comm)
            self.comm = C.c_void_p()


class ShardGroup:
    """One rank's end of the exchange (`nne_shard_group`): a window of device memory every peer
    maps.  `alloc` hands out window space; ranks that allocate in the same order get the same
    offsets, which is what the gathered outputs need."""

    def __init__(self, ctx, rank: int, world: int, window_bytes: int, connect: bool = True):
        self.ctx, self.rank, self.world = ctx, rank, world
        h = C.c_void_p()
        check(load().nne_shard_group_create(ctx.handle, rank, world, window_bytes, C.byref(h)))
        self._h = h
        base, size = C.c_void_p(), C.c_size_t()
        check(load().nne_shard_group_window(h, C.byref(base), C.byref(size)))
        self.base, self.bytes = int(base.value), int(size.value)
        self._top = 0
        self._nccl = None
        if connect and world > 1:
            self.connect_over_torch_distributed()

    @property
    def handle(self):
        return self._h

    def export_handle(self) -> bytes:
        buf = C.create_string_buffer(64)
        check(load().nne_shard_group_handle(self._h, buf))
        return buf.raw

    def connect(self, handles: List[bytes]) -> None:
        """`handles[p]` = rank p's `export_handle()` (any transport may have carried them)."""
        table = b"".join(handles)
        assert len(table) == 64 * self.world
        check(load().nne_shard_group_connect(self._h, table))

    def connect_over_torch_distributed(self) -> None:
        import torch
        import torch.distributed as dist
        mine = torch.tensor(list(self.export_handle()), dtype=torch.uint8, device=f"cuda:{self.ctx.device}")
        every = torch.empty(self.world * 64, dtype=torch.uint8, device=mine.device)
        dist.all_gather_into_tensor(every, mine)
        raw = bytes(every.cpu().tolist())
        self.connect([raw[64 * p: 64 * (p + 1)] for p in range(self.world)])
        dist.barrier()  # every rank has mapped every window before anybody stores into one

    def use_nccl(self, comm: Optional[NcclComm] = None) -> None:
        """Gives the group a communicator for route 1 (made here unless one is passed)."""
        self._nccl = comm or NcclComm(self.rank, self.world, f"cuda:{self.ctx.device}")
        check(load().nne_shard_group_set_nccl(self._h, self._nccl.comm))

    def wait(self, stream: int = 0) -> None:
        """Enqueues the wait for the arrival of every sharded run issued so far (peer-store route)."""
        check(load().nne_shard_group_wait(self._h, stream))

    def alloc(self, nfloats: int) -> int:
        """Device pointer to `nfloats` f32 of window space (256-byte aligned)."""
        off = (self._top + 255) & ~255
        if off + 4 * nfloats > self.bytes:
            raise MemoryError("shard window exhausted")
        self._top = off + 4 * nfloats
        return self.base + off

    def close(self):
        if getattr(self, "_h", None) is not None:
            load().nne_shard_group_destroy(self._h)
            self._h = None
        if self._nccl is not None:
            self._nccl.close()
            self._nccl = None


class ShardedPlan:
    """`nne_qlinear_plan_create_sharded`: a list of column shards run together; afterwards the
    gathered outputs [m, n_total_i] sit in this rank's window at `y_full_ptrs[i]`."""

    def __init__(self, group: ShardGroup, shards, row_begins, n_totals, x_ptrs, y_full_ptrs, m: int,
                 route: int = ROUTE_PEER_STORES):
        n = len(shards)
        hs = (C.c_void_p * n)(*[s._live_handle() for s in shards])
        rb = (C.c_size_t * n)(*[int(v) for v in row_begins])
        nt = (C.c_size_t * n)(*[int(v) for v in n_totals])
        xs = (C.c_void_p * n)(*[int(p) for p in x_ptrs])
        ys = (C.c_void_p * n)(*[int(p) for p in y_full_ptrs])
        h = C.c_void_p()
        check(load().nne_qlinear_plan_create_sharded(group.handle, n, hs, rb, nt, xs, ys, m, route, C.byref(h)))
        self._h, self._keep = h, (group, list(shards))
        self.m, self.n_totals, self.k = int(m), [int(v) for v in n_totals], [s.in_features for s in shards]

    @property
    def launches(self) -> int:
        return int(load().nne_qlinear_plan_launches(self._h))

    def run(self, stream: int = 0) -> None:
        check(load().nne_qlinear_plan_run(self._h, stream))

    def run_host(self, x_all: np.ndarray, y_all: Optional[np.ndarray] = None) -> np.ndarray:
        x_all = np.ascontiguousarray(x_all, dtype=np.float32).reshape(-1)
        assert x_all.size == sum(self.m * k for k in self.k)
        if y_all is None:
            y_all = np.empty(sum(self.m * n for n in self.n_totals), dtype=np.float32)
        check(load().nne_qlinear_plan_run_host(self._h, x_all.ctypes.data_as(C.c_void_p),
                                               y_all.ctypes.data_as(C.c_void_p)))
        return y_all

    def close(self):
        if getattr(self, "_h", None) is not None:
            load().nne_qlinear_plan_destroy(self._h)
            self._h = None


class ShardedQLinear:
    """One rank's column slice of a QLinear.  `forward(x)` returns the full [m, out_features]
    output on every rank (a torch tensor aliasing the group's window; valid until the forward after
    next, because two output areas alternate)."""

    def __init__(self, nne, weight: np.ndarray, bias: Optional[np.ndarray], group: ShardGroup,
                 max_m: int = 16, route: int = ROUTE_PEER_STORES):
        self.out_features, self.in_features = weight.shape
        self.group, self.route = group, route
        b, e = shard_rows(self.out_features, group.world, group.rank)
        self.begin, self.end = b, e
        self.local = nne.QLinear.from_linear(
            nne.Linear(weight[b:e], None if bias is None else bias[b:e]), group.ctx)
        self.max_m = max_m
        self._areas = [group.alloc(max_m * self.out_features) for _ in range(2)]
        self._plans = {}
        self._turn = 0

    def _plan(self, x_ptr: int, m: int, area: int) -> ShardedPlan:
        if m > self.max_m:
            raise ValueError(f"m = {m} above the {self.max_m} rows the output areas were sized for")
        key = (m, area, x_ptr)
        plan = self._plans.get(key)
        if plan is None:
            plan = ShardedPlan(self.group, [self.local], [self.begin], [self.out_features],
                               [x_ptr], [self._areas[area]], m, self.route)
            self._plans[key] = plan
        return plan

    def prepare(self, x_dev) -> None:
        """Builds the plans a later `forward(x_dev)` needs (plan creation allocates; a caller that
        drives several devices from one thread does it before the first rank's kernel waits)."""
        for area in (0, 1):
            self._plan(x_dev.data_ptr(), int(x_dev.shape[0]), area)

    def forward(self, x_dev, stream: int = 0):
        """x_dev: torch CUDA tensor [m, in_features] (replicated on every rank, contiguous f32)."""
        import torch
        m = int(x_dev.shape[0])
        area = self._turn & 1
        self._turn += 1
        plan = self._plan(x_dev.data_ptr(), m, area)
        plan.run(stream)
        if self.route == ROUTE_PEER_STORES:
            self.group.wait(stream)  # the reader of the result follows on this stream
        return torch.as_tensor(DeviceArray(self._areas[area], (m, self.out_features)),
                               device=f"cuda:{self.group.ctx.device}")

    def close(self):
        for p in self._plans.values():
            p.close()
        self._plans = {}
