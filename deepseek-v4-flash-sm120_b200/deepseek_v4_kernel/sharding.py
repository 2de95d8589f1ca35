"""Multi-GPU partitioning of the sparse-MLA path (one process per GPU).

Three ways the path shards, none of which needs a collective inside the kernels:
  * decode by request: contiguous slices of the batch; every rank holds only
    its own requests' pages (request-parallel, no communication);
  * decode by heads (tensor-parallel style): h_q / tp heads per rank over a
    replicated cache, followed by ONE all-gather of the per-head outputs;
  * prefill by query blocks, balanced by the modelled time of each query row
    (tiles of its causal top-k list plus a fixed cost per row) rather than by row count.
The reference has none of this in-tree: SGLang supplies tensor parallelism and
the kernel just sees a smaller h_q (its launch script sets
--tensor-parallel-size 4).
"""
from __future__ import annotations

from typing import List, Tuple

import torch
import torch.distributed as dist


def request_slice(n_requests: int, world: int, rank: int) -> slice:
    """Contiguous, near-equal slice of the batch owned by `rank`."""
    base, extra = divmod(n_requests, world)
    start = rank * base + min(rank, extra)
    return slice(start, start + base + (1 if rank < extra else 0))


def head_slice(h_q: int, world: int, rank: int) -> slice:
    if h_q % world:
        raise ValueError(f"h_q={h_q} is not divisible by the tensor-parallel size {world}")
    per = h_q // world
    return slice(rank * per, (rank + 1) * per)


def causal_pairs(s_q: int, topk: int, row0: int = 0) -> torch.Tensor:
    """Pairs attended by each query row of a causal top-k prefill: min(i + 1, topk)."""
    rows = torch.arange(row0, row0 + s_q, dtype=torch.int64)
    return torch.clamp(rows + 1, max=topk)


TILE_ROWS = 128               # index entries the attention kernel handles per tile
ROW_FIXED_TILES = 1.5         # set-up and epilogue of one query row, in tile times (measured)


def row_cost(pairs: torch.Tensor) -> torch.Tensor:
    """Modelled time of a prefill query row in tile units: the kernel walks a row's list in
    tiles of 128 entries (a partly filled tile costs a whole one) and pays a fixed set-up and
    epilogue per row, so short rows are dearer than their pair count says."""
    tiles = (pairs + TILE_ROWS - 1) // TILE_ROWS
    return tiles.to(torch.float64) + ROW_FIXED_TILES


def balanced_query_blocks(s_q: int, topk: int, world: int) -> List[Tuple[int, int]]:
    """Contiguous [begin, end) query blocks of near-equal modelled time (`row_cost` of the
    causal pair counts)."""
    csum = torch.cumsum(row_cost(causal_pairs(s_q, topk)), 0)
    total = float(csum[-1])
    bounds = [0]
    for r in range(1, world):
        target = torch.tensor(total * r / world, dtype=torch.float64)
        bounds.append(int(torch.searchsorted(csum, target, right=False)))
    bounds.append(s_q)
    return [(bounds[r], max(bounds[r], bounds[r + 1])) for r in range(world)]


def all_gather_heads(out_local: torch.Tensor, lse_local: torch.Tensor, group=None):
    """One all-gather of per-head results after head-sharded decode.

    out_local [b, s_q, h_q/tp, 512], lse_local [b, h_q/tp, s_q] ->
    (out [b, s_q, h_q, 512], lse [b, h_q, s_q]) on every rank.  Uses the backend
    of the process group (NCCL over NVLink on GPUs, gloo on CPU).
    """
    world = dist.get_world_size(group)
    b, s_q, h_loc, d = out_local.shape
    out_all = torch.empty((world,) + tuple(out_local.shape), dtype=out_local.dtype,
                          device=out_local.device)
    lse_all = torch.empty((world,) + tuple(lse_local.shape), dtype=lse_local.dtype,
                          device=lse_local.device)
    dist.all_gather_into_tensor(out_all.view(-1), out_local.contiguous().view(-1), group=group)
    dist.all_gather_into_tensor(lse_all.view(-1), lse_local.contiguous().view(-1), group=group)
    out = out_all.permute(1, 2, 0, 3, 4).reshape(b, s_q, world * h_loc, d)
    lse = lse_all.permute(1, 0, 2, 3).reshape(b, world * h_loc, s_q)
    return out, lse


class HeadGather:
    """All-gather of head-sharded decode results through NVLink peer memory
    (`dsv4_gather_heads`): one kernel per rank instead of two library collectives.

    The gathered buffers live in symmetric memory (every rank maps every rank's copy).
    Two buffer sets alternate between steps; `gather` returns views of the set just
    filled, valid until the call after next.  All ranks must call `gather` the same
    number of times.  CUDA only; needs the in-tree library and peer access between the
    GPUs of the group.
    """

    def __init__(self, b: int, s_q: int, h_q: int, device, group=None):
        import ctypes as C
        import os
        # plain peer loads and stores only: no NVLink multicast object is bound to the buffers
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm
        from . import _native as N
        self._N, self._C = N, C
        group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if h_q % self.world:
            raise ValueError(f"h_q={h_q} is not divisible by the tensor-parallel size {self.world}")
        if self.world > N.MAX_PEERS:
            raise ValueError(f"at most {N.MAX_PEERS} ranks")
        self.b, self.s_q, self.h_q, self.h_local = b, s_q, h_q, h_q // self.world
        out_bytes = b * s_q * h_q * 512 * 2
        lse_bytes = (b * h_q * s_q * 4 + 255) // 256 * 256
        set_bytes = out_bytes + lse_bytes
        self._offsets = [(k * set_bytes, k * set_bytes + out_bytes) for k in range(2)]
        self._flag_off = 2 * set_bytes
        total = self._flag_off + 256
        self.buf = symm.empty(total, dtype=torch.uint8, device=device)
        self.buf.zero_()
        torch.cuda.synchronize(device)
        self.hdl = symm.rendezvous(self.buf, group.group_name)
        self.peer_base = [int(p) for p in self.hdl.buffer_ptrs]
        self.counter = torch.zeros(1, dtype=torch.int32, device=device)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        self.step = 0
        self.views = []
        for o_off, l_off in self._offsets:
            out = self.buf[o_off:o_off + out_bytes].view(torch.bfloat16).view(b, s_q, h_q, 512)
            lse = self.buf[l_off:l_off + b * h_q * s_q * 4].view(torch.float32).view(b, h_q, s_q)
            self.views.append((out, lse))
        dist.barrier(group)                     # every rank has zeroed its flags before any step
        torch.cuda.synchronize(device)

    def _args_for(self, k: int):
        N = self._N
        a = N.GatherArgs()
        a.world, a.rank, a.b, a.s_q, a.h_local = self.world, self.rank, self.b, self.s_q, self.h_local
        o_off, l_off = self._offsets[k]
        for r in range(self.world):
            a.peer_out[r] = self.peer_base[r] + o_off
            a.peer_lse[r] = self.peer_base[r] + l_off
            a.peer_flags[r] = self.peer_base[r] + self._flag_off
        a.counter, a.status = self.counter.data_ptr(), self.status.data_ptr()
        return a

    def gather(self, out_local: torch.Tensor, lse_local: torch.Tensor, stream: int):
        """Queue the exchange of this rank's shard on `stream`; returns (out, lse) views of
        the gathered buffers [b, s_q, h_q, 512] / [b, h_q, s_q], complete once the kernel
        has run."""
        if not hasattr(self, "_args"):
            self._args = [self._args_for(0), self._args_for(1)]
        assert out_local.is_contiguous() and lse_local.is_contiguous()
        self.step += 1
        k = self.step & 1
        a = self._args[k]
        a.step = self.step
        a.out_local, a.lse_local = out_local.data_ptr(), lse_local.data_ptr()
        rc = self._N.lib.dsv4_gather_heads(self._C.byref(a), stream)
        if rc:
            self._N.check(rc, "dsv4_gather_heads")
        return self.views[k]

    def decode_gather(self, call, stream: int):
        """Decode this rank's head shard with the prepared launch `call` (a cuda.DecodeCall
        over h_q / world heads) and exchange the result in the same call
        (`dsv4_sparse_decode_gather`): the exchange kernel is queued behind the decode with
        programmatic dependent launch.  Returns (out, lse) views like `gather`."""
        if not hasattr(self, "_args"):
            self._args = [self._args_for(0), self._args_for(1)]
        self.step += 1
        k = self.step & 1
        a = self._args[k]
        a.step = self.step
        rc = self._N.lib.dsv4_sparse_decode_gather(self._C.byref(call.args), self._C.byref(a), stream)
        if rc:
            self._N.check(rc, "dsv4_sparse_decode_gather")
        return self.views[k]

    def timed_out(self) -> bool:
        """True when a bounded wait for a peer's shard ran out (synchronises)."""
        return bool(self.status.item() != 0)
