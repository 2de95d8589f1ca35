"""The CPU oracle against the golden vectors taken from the reference project,
plus properties of the parts the reference never tested (quantiser, combine,
576/644-byte layout)."""
import math

import pytest
import torch

from oracle import sparse_mla as O
from util import load_golden

DECODE_CASES = ["decode_h64_topk64", "decode_h16_topk256", "decode_h16_topk2048",
                "decode_h16_topk512_len", "decode_h16_topk128_sink_len0"]
PREFILL_CASES = ["prefill_h16_topk128", "prefill_h16_topk256_len_sink"]


@pytest.mark.parametrize("name", DECODE_CASES)
def test_decode_matches_reference_vectors(name):
    g = load_golden(name)
    out, lse = O.sparse_decode(g["q"], g["kv_pages"], g["indices"], g.get("topk_length"),
                               g.get("attn_sink"), g["sm_scale"], g["page_block"], O.MODEL1)
    assert torch.equal(out, g["out"])          # same arithmetic, same order: bit-exact
    torch.testing.assert_close(lse, g["lse"], atol=1e-6, rtol=1e-6)
    # row-gathering variant is the same arithmetic
    out2, lse2 = O.sparse_decode(g["q"], g["kv_pages"], g["indices"], g.get("topk_length"),
                                 g.get("attn_sink"), g["sm_scale"], g["page_block"], O.MODEL1,
                                 whole_arena=False)
    assert torch.equal(out2, out) and torch.equal(lse2, lse)


@pytest.mark.parametrize("name", DECODE_CASES[:2])
def test_dequant_is_bit_exact(name):
    g = load_golden(name)
    dense = O.pages_to_bf16(g["kv_pages"], g["page_block"], O.MODEL1)
    assert torch.equal(dense[:64].view(torch.int16), g["dense_head"].view(torch.int16))
    idx = torch.tensor([0, 5, 63, 17], dtype=torch.int32)
    assert torch.equal(O.gather_rows_bf16(g["kv_pages"], 64, O.MODEL1, idx), dense[idx.long()])


@pytest.mark.parametrize("name", PREFILL_CASES)
def test_prefill_matches_reference_vectors(name):
    g = load_golden(name)
    out, mx, lse = O.sparse_prefill(g["q"], g["kv"], g["indices"], g["sm_scale"], 512,
                                    g.get("attn_sink"), g.get("topk_length"))
    torch.testing.assert_close(out.float(), g["out"].float(), atol=2e-3, rtol=2e-2)
    fin = torch.isfinite(g["max_logits"])
    assert torch.equal(fin, torch.isfinite(mx))
    torch.testing.assert_close(mx[fin], g["max_logits"][fin], atol=1e-5, rtol=1e-5)
    assert torch.equal(torch.isposinf(lse), torch.isposinf(g["lse"]))
    fin = torch.isfinite(g["lse"])
    torch.testing.assert_close(lse[fin], g["lse"][fin], atol=1e-5, rtol=1e-5)


def test_minus_one_is_a_zero_row_not_a_mask():
    """Decode: an index of -1 adds exp(0 - max) to the denominator."""
    g = load_golden("decode_h16_topk256")
    idx = g["indices"].clone()
    assert (idx < 0).any()
    out_a, lse_a = O.sparse_decode(g["q"], g["kv_pages"], idx, None, None, g["sm_scale"], 64)
    out_b, lse_b = O.sparse_decode(g["q"], g["kv_pages"], idx, None, None, g["sm_scale"], 64,
                                   mask_invalid=True)
    assert (lse_a > lse_b).all()


@pytest.mark.parametrize("layout", [O.MODEL1, O.V32])
def test_quantiser_round_trip(layout):
    gen = torch.Generator().manual_seed(3)
    n = 256
    scale = torch.logspace(-3, 2, n).unsqueeze(1)
    k_nope = (torch.randn(n, layout.d_nope, generator=gen) * scale).bfloat16()
    k_nope[7] = 0                                   # all-zero tile row
    k_rope = torch.randn(n, 64, generator=gen).bfloat16()
    pages = O.build_pages(k_nope, k_rope, 64, layout)
    assert pages.shape == (n // 64, 64 * layout.bytes_per_token)
    dense = O.pages_to_bf16(pages, 64, layout)
    assert torch.equal(dense[:, layout.d_nope:], k_rope)          # RoPE kept bit-exact
    x = k_nope.float().view(n, layout.scale_active, layout.quant_tile)
    amax = x.abs().amax(-1)
    e = O.tile_exponent(amax)
    # the scale is the smallest power of two with amax / scale <= 448
    s = torch.pow(2.0, e.float())
    assert (amax.clamp(min=O.AMAX_FLOOR) / s <= 448).all()
    assert (amax.clamp(min=O.AMAX_FLOOR) / (s / 2) > 448).all()
    # e4m3 keeps 3 mantissa bits: relative error of a normal value <= 2^-4, plus the
    # subnormal step 2^-9 * scale near zero
    err = (dense[:, :layout.d_nope].float().view_as(x) - x).abs()
    bound = x.abs() * 2.0 ** -4 + s.unsqueeze(-1) * 2.0 ** -10 + 1e-30
    assert (err <= bound).all()
    # idempotent: re-quantising the dequantised values reproduces the same bytes
    pages2 = O.build_pages(dense[:, :layout.d_nope].contiguous(), k_rope, 64, layout)
    d2 = O.pages_to_bf16(pages2, 64, layout)
    assert torch.equal(d2, dense)


def test_combine_equals_unsplit_decode():
    gen = torch.Generator().manual_seed(5)
    g = load_golden("decode_h16_topk2048")
    q, pages, idx = g["q"], g["kv_pages"], g["indices"]
    sink = torch.randn(16, generator=gen)
    out_ref, lse_ref = O.sparse_decode(q, pages, idx, None, sink, g["sm_scale"], 64)
    n_splits, per = 5, 416
    b, _, h, _ = q.shape
    o_acc = torch.zeros(n_splits, b, h, 512)
    l_acc = torch.full((n_splits, b, h), float("-inf"))
    dense = O.pages_to_bf16(pages, 64, O.MODEL1).float()
    for s in range(n_splits):
        lo, hi = s * per, min(2048, (s + 1) * per)
        for bi in range(b):
            ids = idx[bi, 0, lo:hi]
            valid = (ids >= 0) & (ids < dense.size(0))
            k = torch.where(valid.unsqueeze(-1), dense[ids.clamp(min=0).long()], torch.zeros(1))
            o, l = O.decode_one(q[bi, 0].float(), k, valid, hi - lo, g["sm_scale"], False)
            o_acc[s, bi], l_acc[s, bi] = o, l
    out, lse = O.combine_splits(o_acc, l_acc, sink)
    torch.testing.assert_close(out.float(), out_ref[:, 0].float(), atol=1e-3, rtol=8e-3)
    torch.testing.assert_close(lse, lse_ref[:, 0], atol=1e-5, rtol=1e-5)
    # an all-empty row: out 0, lse = sink
    l_acc[:, 0, 3] = float("-inf")
    out, lse = O.combine_splits(o_acc, l_acc, sink)
    assert (out[0, 3] == 0).all() and lse[0, 3] == sink[3]
    out, lse = O.combine_splits(o_acc, l_acc, None)
    assert (out[0, 3] == 0).all() and lse[0, 3] == float("-inf")


def test_v32_layout_decode_consistency():
    """644-byte layout: decode over quantised pages equals dense attention over
    the dequantised rows (no reference vectors exist for this layout)."""
    gen = torch.Generator().manual_seed(11)
    n_tok, h, topk = 256, 8, 96
    pages = O.build_pages(torch.randn(n_tok, 512, generator=gen).bfloat16(),
                          torch.randn(n_tok, 64, generator=gen).bfloat16(), 64, O.V32)
    q = torch.randn(1, 1, h, 576, generator=gen).bfloat16()
    idx = torch.randperm(n_tok, generator=gen)[:topk].int().view(1, 1, topk)
    sm = 576 ** -0.5
    out, lse = O.sparse_decode(q, pages, idx, None, None, sm, 64, O.V32)
    k = O.pages_to_bf16(pages, 64, O.V32)[idx.view(-1).long()].float()
    s = (q[0, 0].float() @ k.t()) * sm
    torch.testing.assert_close(lse[0, 0], torch.logsumexp(s, -1))
    torch.testing.assert_close(out[0, 0].float(), (torch.softmax(s, -1) @ k[:, :512]),
                               atol=4e-3, rtol=1e-2)


def test_extra_kv_is_list_concatenation():
    g = load_golden("decode_h16_topk256")
    q, pages, idx = g["q"], g["kv_pages"], g["indices"]
    a, b_ = idx[..., :192].contiguous(), idx[..., 192:].contiguous()
    out_ref, lse_ref = O.sparse_decode(q, pages, idx, None, None, g["sm_scale"], 64)
    out, lse = O.sparse_decode(q, pages, a, None, None, g["sm_scale"], 64,
                               extra_kv_pages=pages, extra_indices=b_)
    assert torch.equal(out, out_ref)
    torch.testing.assert_close(lse, lse_ref)
