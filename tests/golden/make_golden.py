"""Generate the golden vectors in this folder from the reference project itself.

Run once, where the reference checkout is available, as

    python tests/golden/make_golden.py /path/to/reference

It imports the reference's own `tests/reference.py` (torch, CPU), draws its
seeded fake batches, runs its decode / prefill reference functions and stores
inputs and outputs as `.npz` (BF16 tensors as their uint16 bit patterns).  The
test-suite replays these files against the CPU oracle and the CUDA kernels, so
nothing at test time needs the reference checkout.
"""
from __future__ import annotations

import math
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def bits(t: torch.Tensor) -> np.ndarray:
    if t.dtype == torch.bfloat16:
        return t.contiguous().view(torch.int16).numpy().view(np.uint16)
    return t.contiguous().numpy()


def main(ref_root: str) -> None:
    sys.path.insert(0, os.path.join(ref_root, "tests"))
    import reference as R  # the reference's own oracle

    sm = 1.0 / math.sqrt(512)

    def decode_case(name, *, b, h_q, num_blocks, topk, seed, lengths=None, sink_seed=None):
        q, pages, _view, idx = R.make_fake_batch(b=b, h_q=h_q, num_blocks=num_blocks,
                                                 page_block=64, topk=topk, seed=seed,
                                                 device="cpu")
        tk = torch.tensor(lengths, dtype=torch.int32) if lengths is not None else None
        sink = None
        if sink_seed is not None:
            sink = torch.randn(h_q, generator=torch.Generator().manual_seed(sink_seed))
        out, lse = R.sparse_decode_reference(q, pages, idx, tk, sink, sm, 64)
        dense = R._pages_to_bf16(pages, 64)
        arrays = dict(q=bits(q), kv_pages=bits(pages), indices=bits(idx), out=bits(out),
                      lse=bits(lse), dense_head=bits(dense[:64]),
                      sm_scale=np.float64(sm), page_block=np.int64(64))
        if tk is not None:
            arrays["topk_length"] = bits(tk)
        if sink is not None:
            arrays["attn_sink"] = bits(sink)
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **arrays)

    def prefill_case(name, *, s_q, h_q, s_kv, topk, seed, with_len, with_sink, lonely_row=None):
        q, kv, idx, sink, tl = R.make_fake_prefill_batch(
            s_q=s_q, h_q=h_q, s_kv=s_kv, topk=topk, with_topk_length=with_len,
            with_attn_sink=with_sink, seed=seed, device="cpu")
        if lonely_row is not None:
            idx[lonely_row] = -1
        out, mx, lse = R.sparse_prefill_reference(q, kv, idx, sm, 512, sink, tl)
        arrays = dict(q=bits(q), kv=bits(kv), indices=bits(idx), out=bits(out),
                      max_logits=bits(mx), lse=bits(lse), sm_scale=np.float64(sm))
        if sink is not None:
            arrays["attn_sink"] = bits(sink)
        if tl is not None:
            arrays["topk_length"] = bits(tl)
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **arrays)

    # The reference's own decode test shapes (tests/test_sparse_decode.py:27-67),
    # with h_q trimmed on all but one case to keep the files small.
    decode_case("decode_h64_topk64", b=2, h_q=64, num_blocks=8, topk=64, seed=0)
    decode_case("decode_h16_topk256", b=2, h_q=16, num_blocks=8, topk=256, seed=0)
    decode_case("decode_h16_topk2048", b=2, h_q=16, num_blocks=8, topk=2048, seed=0)
    decode_case("decode_h16_topk512_len", b=2, h_q=16, num_blocks=4, topk=512, seed=1,
                lengths=[64, 32])
    decode_case("decode_h16_topk128_sink_len0", b=2, h_q=16, num_blocks=4, topk=128, seed=2,
                lengths=[100, 0], sink_seed=7)
    # Prefill (tests/test_sparse_prefill.py:44-106), small s_kv.
    prefill_case("prefill_h16_topk128", s_q=16, h_q=16, s_kv=512, topk=128, seed=0,
                 with_len=False, with_sink=False, lonely_row=5)
    prefill_case("prefill_h16_topk256_len_sink", s_q=16, h_q=16, s_kv=512, topk=256, seed=2,
                 with_len=True, with_sink=True)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: make_golden.py <checkout of ambientlight/deepseek-v4-flash-sm120>")
    main(sys.argv[1])
