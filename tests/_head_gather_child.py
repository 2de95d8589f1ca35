"""Child process of test_gpu_multi.py: one rank of a head-sharded decode whose per-head
results are exchanged with the peer-memory all-gather (and, as a cross-check, with the
library all-gather).  Started by torch.distributed.run; prints OK on success."""
import math
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path[:0] = [ROOT, os.path.join(ROOT, "deepseek-v4-flash-sm120_b200"), os.path.dirname(os.path.abspath(__file__))]

from deepseek_v4_kernel import cuda as K, sharding  # noqa: E402
from oracle import sparse_mla as O  # noqa: E402
import test_gpu_decode as T  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=dev)
    h_q, b = 64, 3
    q, pages, idx = T.fake_batch(b, h_q, 16, 512, seed=123, layout=O.V32)      # same on every rank
    sm = 1.0 / math.sqrt(576)
    kv4 = pages.to(dev).view(pages.size(0), 64, 1, O.V32.bytes_per_token)
    qd = q.to(dev)
    hs = sharding.head_slice(h_q, world, rank)
    gather = sharding.HeadGather(b, 1, h_q, dev)
    stream = torch.cuda.current_stream(dev).cuda_stream
    for step in range(4):                               # more steps than buffer sets
        idx_s = torch.roll(idx, shifts=step * 7, dims=2).to(dev)
        full_out, full_lse, _, _ = K.sparse_decode_fwd(qd, kv4, idx_s, None, None, None, None, None,
                                                       None, None, 512, sm)
        out_l, lse_l, _, _ = K.sparse_decode_fwd(qd[:, :, hs].contiguous(), kv4, idx_s, None, None,
                                                 None, None, None, None, None, 512, sm)
        g_out, g_lse = gather.gather(out_l.contiguous(), lse_l.contiguous(), stream)
        n_out, n_lse = sharding.all_gather_heads(out_l, lse_l)
        torch.cuda.synchronize(dev)
        assert not gather.timed_out(), "a peer's shard did not arrive"
        assert torch.equal(g_out, n_out) and torch.equal(g_lse, n_lse), f"step {step}: differs from NCCL"
        torch.testing.assert_close(g_out.float(), full_out.float(), atol=5e-3, rtol=5e-3)
        torch.testing.assert_close(g_lse, full_lse, atol=1e-3, rtol=1e-3)
        # decode and exchange in one call, for split plans with and without a combine step:
        # bit-identical to an all-gather of the same call's own local result
        for n_splits in (1, 3, 8):
            call = K.DecodeCall(qd[:, :, hs].contiguous(), kv4, idx_s, sm, n_splits=n_splits)
            f_out, f_lse = gather.decode_gather(call, stream)
            torch.cuda.synchronize(dev)
            assert not gather.timed_out(), "a peer's shard did not arrive (one-call path)"
            r_out, r_lse = sharding.all_gather_heads(call.out, call.lse)
            assert torch.equal(f_out, r_out) and torch.equal(f_lse, r_lse), "one-call path differs from NCCL"
            torch.testing.assert_close(f_out.float(), full_out.float(), atol=5e-3, rtol=5e-3)
            torch.testing.assert_close(f_lse, full_lse, atol=1e-3, rtol=1e-3)
    assert K.device_status() == 0
    dist.barrier()
    dist.destroy_process_group()
    print("OK", flush=True)


if __name__ == "__main__":
    main()
