"""Host-side multi-GPU logic, run as two gloo ranks on CPU: request slices,
head shards with the single all-gather, pair-balanced prefill blocks, and a
rank that fails before the collective."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from deepseek_v4_kernel import sharding as SH
from oracle import sparse_mla as O
from util import load_golden


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_request_slices_cover_the_batch():
    for n, w in [(128, 8), (16, 1), (10, 4), (3, 8)]:
        seen = []
        for r in range(w):
            sl = SH.request_slice(n, w, r)
            seen += list(range(n))[sl]
        assert seen == list(range(n))
    sizes = [len(range(128)[SH.request_slice(128, 8, r)]) for r in range(8)]
    assert sizes == [16] * 8


def test_prefill_blocks_balance_modelled_time_not_rows():
    s_q, topk = 8192, 2048
    pairs = SH.causal_pairs(s_q, topk)
    assert int(pairs.sum()) == 14_681_088            # the benchmark configuration's pair count
    for world in (2, 4, 8):
        blocks = SH.balanced_query_blocks(s_q, topk, world)
        assert blocks[0][0] == 0 and blocks[-1][1] == s_q
        assert all(blocks[i][1] == blocks[i + 1][0] for i in range(world - 1))
        cost = SH.row_cost(pairs)
        work = [float(cost[a:b].sum()) for a, b in blocks]
        assert max(work) <= 1.01 * (sum(work) / world)        # equal modelled time
        pair_work = [int(pairs[a:b].sum()) for a, b in blocks]
        assert max(pair_work) <= 1.10 * (sum(pair_work) / world)
        assert blocks[0][1] - blocks[0][0] > s_q // world     # early queries are cheaper


def _head_shard_worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = load_golden("decode_h16_topk256")
        hs = SH.head_slice(16, world, rank)
        q_loc = g["q"][:, :, hs].contiguous()
        out_loc, lse_loc = O.sparse_decode(q_loc, g["kv_pages"], g["indices"], None, None,
                                           g["sm_scale"], 64)
        out, lse = SH.all_gather_heads(out_loc, lse_loc.transpose(1, 2).contiguous())
        ok = torch.equal(out, g["out"]) and torch.allclose(lse.transpose(1, 2), g["lse"], atol=1e-6)
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_head_sharded_decode_all_gather_two_ranks():
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_head_shard_worker, args=(r, 2, port, ret)) for r in range(2)]
    [p.start() for p in procs]
    [p.join(120) for p in procs]
    assert all(p.exitcode == 0 for p in procs)
    assert ret.get(0) is True and ret.get(1) is True


def _failing_worker(rank, world, port, ret):
    import datetime
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=5))
    if rank == 1:
        ret[1] = "left before the collective"
        os._exit(0)                      # the rank goes away between steps
    try:
        x = torch.zeros(1, 1, 8, 512, dtype=torch.bfloat16)
        SH.all_gather_heads(x, torch.zeros(1, 8, 1))
        ret[0] = "no error"
    except Exception as exc:  # noqa: BLE001  the surviving rank must see an error, not hang
        ret[0] = "error: " + type(exc).__name__


def test_peer_leaving_surfaces_as_an_error_not_a_hang():
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_failing_worker, args=(r, 2, port, ret)) for r in range(2)]
    [p.start() for p in procs]
    [p.join(90) for p in procs]
    for p in procs:
        if p.is_alive():
            p.terminate()
            pytest.fail("a rank hung after its peer left")
    assert str(ret.get(0, "")).startswith("error")
