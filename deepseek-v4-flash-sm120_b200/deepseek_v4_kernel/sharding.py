"""Multi-GPU partitioning of the sparse-MLA path (one process per GPU).

Three ways the path shards, none of which needs a collective inside the kernels:
  * decode by request: contiguous slices of the batch; every rank holds only
    its own requests' pages (request-parallel, no communication);
  * decode by heads (tensor-parallel style): h_q / tp heads per rank over a
    replicated cache, followed by ONE all-gather of the per-head outputs;
  * prefill by query blocks, balanced by the number of (query, key) pairs a
    causal top-k gives each query rather than by row count.
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


def balanced_query_blocks(s_q: int, topk: int, world: int) -> List[Tuple[int, int]]:
    """Contiguous [begin, end) query blocks with near-equal pair counts."""
    csum = torch.cumsum(causal_pairs(s_q, topk), 0)
    total = int(csum[-1])
    bounds = [0]
    for r in range(1, world):
        target = total * r // world
        bounds.append(int(torch.searchsorted(csum, torch.tensor(target), right=False)))
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
