"""CPU oracle for the sparse-MLA attention path (TEST INFRASTRUCTURE ONLY).

This module restates, in plain torch-on-CPU, the arithmetic of the reference
project's own torch oracle so that the CUDA kernels can be checked against it.
It is imported by the test-suite, by the smoke check and by the CPU-baseline
leg of the benchmark, and by nothing else: the product path never calls it.

Parity status
-------------
* MODEL1 layout (448 FP8 + 64 BF16 RoPE, 7+1 UE8M0 bytes, 584 B/token): pinned.
  `tests/golden/` holds vectors produced by importing the reference's
  `tests/reference.py` itself; `tests/test_oracle.py` replays them.
* V32 layout (512 FP8 + 64 BF16 RoPE, 4 UE8M0 bytes, 644 B/token), decode
  `attn_sink`, `extra_kv`, the split-KV combine in isolation and the KV
  quantiser: parity unpinned (the reference has no implementation or test of
  them); the oracle here is the same arithmetic with other constants.

Reference functions followed (paths inside the reference project):
  tests/reference.py:40-42    UE8M0 byte -> scale               -> ue8m0_to_scale
  tests/reference.py:45-58    FP8 * scale -> BF16, concat RoPE  -> unpack_rows
  tests/reference.py:61-79    page arena -> dense BF16 rows     -> pages_to_bf16
  tests/reference.py:82-132   decode attention                  -> sparse_decode
  tests/reference.py:154-199  prefill attention                 -> sparse_prefill
  csrc/sm120/decode/split_kv_combine.cuh:23-110  merge partials -> combine_splits
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch

D_ROPE = 64
D_V = 512


@dataclass(frozen=True)
class KvLayout:
    """Byte layout of one token inside a KV page.

    A page of P tokens is two sections, not per-token records:
      [P x nope_rope_bytes]  FP8 e4m3 latent then BF16 RoPE, per token
      [P x scale_slots]      UE8M0 scale bytes, per token
    (reference: tests/reference.py:7-14 and :61-79).
    """
    name: str
    d_nope: int
    quant_tile: int
    scale_active: int
    scale_slots: int

    @property
    def d_qk(self) -> int:
        return self.d_nope + D_ROPE

    @property
    def nope_rope_bytes(self) -> int:
        return self.d_nope + 2 * D_ROPE

    @property
    def bytes_per_token(self) -> int:
        return self.nope_rope_bytes + self.scale_slots

    def page_bytes(self, page_block: int) -> int:
        return page_block * self.bytes_per_token


# The reference's real layout (tests/reference.py:27-37).
MODEL1 = KvLayout("MODEL1", d_nope=448, quant_tile=64, scale_active=7, scale_slots=8)
# The 576/644-byte layout the benchmark configurations are quoted on
# (csrc/common/params.h:12-15 documents it; nothing in the reference runs it).
V32 = KvLayout("V32", d_nope=512, quant_tile=128, scale_active=4, scale_slots=4)

LAYOUTS = {"MODEL1": MODEL1, "V32": V32}


def layout_for(d_qk: int) -> KvLayout:
    if d_qk == MODEL1.d_qk:
        return MODEL1
    if d_qk == V32.d_qk:
        return V32
    raise ValueError(f"no KV layout with d_qk={d_qk}")


# --------------------------------------------------------------------------
# Dequantisation
# --------------------------------------------------------------------------
def ue8m0_to_scale(b: torch.Tensor) -> torch.Tensor:
    """UE8M0 byte -> fp32 power of two, 2**(b-127); byte 0 gives 2**-127."""
    return torch.pow(2.0, b.to(torch.float32) - 127.0)


def unpack_rows(nope_u8: torch.Tensor, rope_u8: torch.Tensor, scale_u8: torch.Tensor,
                layout: KvLayout) -> torch.Tensor:
    """[n, d_nope] FP8 bytes, [n, 128] RoPE bytes, [n, slots] scales -> [n, d_qk] BF16.

    The product fp8 * 2**k is formed in fp32 and rounded to BF16; because e4m3
    carries four significant bits the rounding is exact unless it underflows.
    """
    n = nope_u8.size(0)
    fp8 = nope_u8.contiguous().view(torch.float8_e4m3fn).float()
    scale = ue8m0_to_scale(scale_u8[:, : layout.scale_active])
    nope = fp8.view(n, layout.scale_active, layout.quant_tile) * scale.unsqueeze(-1)
    nope = nope.view(n, layout.d_nope).to(torch.bfloat16)
    rope = rope_u8.contiguous().view(torch.bfloat16).view(n, D_ROPE)
    return torch.cat([nope, rope], dim=-1)


def split_page_sections(kv_pages: torch.Tensor, page_block: int, layout: KvLayout):
    """uint8 [num_blocks, >=page_bytes] -> (nope_rope [N, nrb], scales [N, slots])."""
    nb = kv_pages.size(0)
    nrb = layout.nope_rope_bytes
    body = kv_pages[:, : page_block * nrb].reshape(nb * page_block, nrb)
    scales = kv_pages[:, page_block * nrb: page_block * layout.bytes_per_token]
    return body, scales.reshape(nb * page_block, layout.scale_slots)


def pages_to_bf16(kv_pages: torch.Tensor, page_block: int, layout: KvLayout) -> torch.Tensor:
    """Every token of every page as dense BF16 [num_blocks*page_block, d_qk]."""
    assert kv_pages.dtype == torch.uint8 and kv_pages.dim() == 2
    assert kv_pages.size(1) >= layout.page_bytes(page_block)
    body, scales = split_page_sections(kv_pages, page_block, layout)
    return unpack_rows(body[:, : layout.d_nope], body[:, layout.d_nope:], scales, layout)


def gather_rows_bf16(kv_pages: torch.Tensor, page_block: int, layout: KvLayout,
                     idx: torch.Tensor) -> torch.Tensor:
    """Dequantise only the rows named by `idx` (all must be in range).

    Same arithmetic as pages_to_bf16(...)[idx]; used where the whole arena is
    too large to dequantise in a test.
    """
    idx = idx.long()
    page, row = idx // page_block, idx % page_block
    nrb = layout.nope_rope_bytes
    ar = torch.arange(nrb)
    body = kv_pages[page.unsqueeze(1), (row * nrb).unsqueeze(1) + ar]
    sa = torch.arange(layout.scale_slots)
    scales = kv_pages[page.unsqueeze(1),
                      (page_block * nrb + row * layout.scale_slots).unsqueeze(1) + sa]
    return unpack_rows(body[:, : layout.d_nope], body[:, layout.d_nope:], scales, layout)


# --------------------------------------------------------------------------
# Decode
# --------------------------------------------------------------------------
def _mix_sink(o: torch.Tensor, lse: torch.Tensor, sink: Optional[torch.Tensor]):
    """Fold a per-head sink logit into (o, lse): o *= sigmoid(lse - sink),
    lse = logaddexp(lse, sink) (tests/reference.py:124-129)."""
    if sink is None:
        return o, lse
    sink = sink.float()
    o = o * (1.0 / (1.0 + torch.exp(sink - lse))).unsqueeze(-1)
    m = torch.maximum(lse, sink)
    lse = m + torch.log(torch.exp(lse - m) + torch.exp(sink - m))
    return o, lse


def decode_one(q_bs: torch.Tensor, k: torch.Tensor, valid: torch.Tensor, length: int,
               sm_scale: float, mask_invalid: bool):
    """One (request, query token): q_bs [h, d_qk] fp32, k [n, d_qk] fp32 with
    invalid rows already zeroed.  Returns fp32 (o [h, 512], lse [h])."""
    n = k.size(0)
    logits = (q_bs @ k.t()) * sm_scale
    dead = torch.arange(n) >= length
    if mask_invalid:
        dead = dead | ~valid
    logits = logits.masked_fill(dead.unsqueeze(0), float("-inf"))
    lse = torch.logsumexp(logits, dim=-1)
    p = torch.softmax(logits, dim=-1)
    return p @ k[:, :D_V], lse


def sparse_decode(q: torch.Tensor, kv_pages: torch.Tensor, indices: torch.Tensor,
                  topk_length: Optional[torch.Tensor], attn_sink: Optional[torch.Tensor],
                  sm_scale: float, page_block: int, layout: Optional[KvLayout] = None,
                  *, mask_invalid: bool = False, whole_arena: bool = True,
                  extra_kv_pages: Optional[torch.Tensor] = None,
                  extra_indices: Optional[torch.Tensor] = None,
                  extra_topk_length: Optional[torch.Tensor] = None,
                  extra_page_block: Optional[int] = None,
                  ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Sparse MLA decode.  q [b, s_q, h_q, d_qk] bf16, kv_pages uint8
    [num_blocks, page_bytes], indices int32 [b, s_q, topk].

    Semantics kept from the reference oracle (tests/reference.py:105-131):
      * an index outside [0, num_tokens) gathers a ZERO row that still takes
        part in the softmax with logit 0 (it is not masked) unless
        `mask_invalid` asks for FlashMLA's own behaviour;
      * `topk_length[b]` masks positions >= length to -inf, and a length below
        one is raised to one;
      * V is the first 512 columns of the dequantised K row.
    Returns (out [b, s_q, h_q, 512] bf16, lse [b, s_q, h_q] fp32).

    `whole_arena=True` dequantises the complete cache per call exactly as the
    reference does (that cost is part of the CPU baseline); False dequantises
    only the gathered rows, which is the same arithmetic.
    The optional extra_* cache is a second (kv, indices, length) list appended
    to the first, as in csrc/sm120/decode/sparse_decode_kernel.cuh:468-478.
    """
    layout = layout or layout_for(q.size(-1))
    b, s_q, h_q, d_qk = q.shape
    assert d_qk == layout.d_qk and kv_pages.dtype == torch.uint8
    topk = indices.size(-1)
    n_tok = kv_pages.size(0) * page_block
    dense = pages_to_bf16(kv_pages, page_block, layout) if whole_arena else None
    if extra_kv_pages is not None:
        extra_page_block = extra_page_block or page_block
        n_tok_x = extra_kv_pages.size(0) * extra_page_block
        dense_x = pages_to_bf16(extra_kv_pages, extra_page_block, layout)

    def rows(table, pages, pblock, idx, ntok):
        valid = (idx >= 0) & (idx < ntok)
        safe = torch.where(valid, idx, torch.zeros_like(idx)).long()
        k = table[safe] if table is not None else gather_rows_bf16(pages, pblock, layout, safe)
        return torch.where(valid.unsqueeze(-1), k, torch.zeros_like(k)).float(), valid

    out = torch.zeros(b, s_q, h_q, D_V, dtype=torch.bfloat16)
    lse_out = torch.empty(b, s_q, h_q, dtype=torch.float32)
    for bi in range(b):
        length = int(topk_length[bi]) if topk_length is not None else topk
        length = max(length, 1)
        for si in range(s_q):
            k, valid = rows(dense, kv_pages, page_block, indices[bi, si], n_tok)
            if extra_kv_pages is not None:
                xtopk = extra_indices.size(-1)
                xlen = int(extra_topk_length[bi]) if extra_topk_length is not None else xtopk
                xlen = max(min(xlen, xtopk), 0)
                keep = min(length, topk)
                kx, vx = rows(dense_x, extra_kv_pages, extra_page_block,
                              extra_indices[bi, si], n_tok_x)
                k = torch.cat([k[:keep], kx[:xlen]])
                valid = torch.cat([valid[:keep], vx[:xlen]])
                eff = keep + xlen
            else:
                eff = length
            o, lse = decode_one(q[bi, si].float(), k, valid, eff, sm_scale, mask_invalid)
            if mask_invalid:
                o = torch.nan_to_num(o, nan=0.0)
            o, lse = _mix_sink(o, lse, attn_sink)
            out[bi, si] = o.to(torch.bfloat16)
            lse_out[bi, si] = lse
    return out, lse_out


# --------------------------------------------------------------------------
# Prefill (flat BF16 KV)
# --------------------------------------------------------------------------
def sparse_prefill(q: torch.Tensor, kv: torch.Tensor, indices: torch.Tensor, sm_scale: float,
                   d_v: int = D_V, attn_sink: Optional[torch.Tensor] = None,
                   topk_length: Optional[torch.Tensor] = None, *, row_block: int = 256,
                   ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Sparse MLA prefill.  q [s_q, h_q, d_qk] bf16, kv [s_kv, d_qk] bf16,
    indices int32 [s_q, topk]; an index < 0 or >= s_kv, or at a position
    >= topk_length[i], is masked to -inf (tests/reference.py:168-181).

    Returns (out bf16 [s_q, h_q, d_v], max_logits fp32, lse fp32), natural log;
    a row with nothing to attend to gives out 0, max_logits -inf, lse +inf, and
    the returned lse never includes the sink (tests/reference.py:183-199).
    Rows are processed `row_block` at a time to bound the dense gather.
    """
    s_q, h_q, d_qk = q.shape
    s_kv, topk = kv.size(0), indices.size(-1)
    out = torch.empty(s_q, h_q, d_v, dtype=torch.bfloat16)
    mx = torch.empty(s_q, h_q, dtype=torch.float32)
    lse = torch.empty(s_q, h_q, dtype=torch.float32)
    pos = torch.arange(topk).unsqueeze(0)
    for r0 in range(0, s_q, row_block):
        r1 = min(s_q, r0 + row_block)
        idx = indices[r0:r1].clone()
        if topk_length is not None:
            idx[pos >= topk_length[r0:r1].unsqueeze(1)] = -1
        bad = (idx < 0) | (idx >= s_kv)
        safe = torch.where(bad, torch.zeros_like(idx), idx).long()
        g = kv[safe.reshape(-1)].reshape(r1 - r0, topk, d_qk).float()
        s = torch.einsum("qhd,qtd->qht", q[r0:r1].float(), g) * sm_scale
        s = s.masked_fill(bad.unsqueeze(1), float("-inf"))
        l0 = torch.logsumexp(s, dim=-1)
        mx[r0:r1] = s.max(dim=-1).values
        if attn_sink is not None:
            l_o = torch.logaddexp(l0, attn_sink.float().unsqueeze(0).expand_as(l0))
        else:
            l_o = l0.clone()
        l_o[l_o == float("-inf")] = float("inf")
        p = torch.exp(s - l_o.unsqueeze(-1))
        out[r0:r1] = torch.einsum("qht,qtd->qhd", p, g[..., :d_v]).to(torch.bfloat16)
        l0 = l0.clone()
        l0[l0 == float("-inf")] = float("inf")
        lse[r0:r1] = l0
    return out, mx, lse


def sparse_prefill_paged(q, kv_pages, indices, sm_scale, page_block, layout=None,
                         attn_sink=None, topk_length=None):
    """Prefill over the FP8 paged cache: dequantise, then sparse_prefill."""
    layout = layout or layout_for(q.size(-1))
    return sparse_prefill(q, pages_to_bf16(kv_pages, page_block, layout), indices, sm_scale,
                          D_V, attn_sink, topk_length)


# --------------------------------------------------------------------------
# Split-KV combine
# --------------------------------------------------------------------------
def combine_splits(o_accum: torch.Tensor, lse_accum: torch.Tensor,
                   attn_sink: Optional[torch.Tensor] = None):
    """o_accum fp32 [n_splits, n, h, 512] (each locally normalised),
    lse_accum fp32 [n_splits, n, h] -> (out bf16 [n, h, 512], lse fp32 [n, h]).

    m = max_s lse_s; l = sum_s exp(lse_s - m); out = sum_s exp(lse_s - m) o_s / l;
    a row whose partials are all -inf gives out 0 and lse = sink or -inf
    (csrc/sm120/decode/split_kv_combine.cuh:51-106).
    """
    m = lse_accum.max(dim=0).values
    w = torch.exp(lse_accum - torch.where(torch.isfinite(m), m, torch.zeros_like(m)))
    w = torch.where(torch.isfinite(lse_accum), w, torch.zeros_like(w))
    l = w.sum(dim=0)
    o = (w.unsqueeze(-1) * torch.nan_to_num(o_accum, nan=0.0)).sum(dim=0)
    empty = l == 0
    o = o / torch.where(empty, torch.ones_like(l), l).unsqueeze(-1)
    lse = torch.where(empty, torch.full_like(l, float("-inf")), torch.log(l) + m)
    if attn_sink is not None:
        sink = attn_sink.float().expand_as(lse)
        o2, lse2 = _mix_sink(o, lse, attn_sink)
        o = torch.where(empty.unsqueeze(-1), torch.zeros_like(o), o2)
        lse = torch.where(empty, sink, lse2)
    else:
        o = torch.where(empty.unsqueeze(-1), torch.zeros_like(o), o)
    return o.to(torch.bfloat16), lse


# --------------------------------------------------------------------------
# KV store / quantise (no reference implementation exists: parity unpinned)
# --------------------------------------------------------------------------
FP8_MAX = 448.0
AMAX_FLOOR = 1e-4


def tile_exponent(amax: torch.Tensor) -> torch.Tensor:
    """ceil(log2(max(amax, 1e-4) / 448)) computed exactly through frexp."""
    r = torch.clamp(amax.float(), min=AMAX_FLOOR) / FP8_MAX
    mant, ex = torch.frexp(r)              # r = mant * 2**ex, mant in [0.5, 1)
    return torch.where(mant == 0.5, ex - 1, ex).to(torch.int32)


def quantize_rows(k_nope: torch.Tensor, k_rope: torch.Tensor, layout: KvLayout):
    """BF16 latent [n, d_nope] + BF16 RoPE [n, 64] -> (body uint8 [n, nope_rope_bytes],
    scales uint8 [n, scale_slots]).  Per tile: e = ceil(log2(amax/448)), scale
    byte e+127, fp8 = saturating round-to-nearest-even cast of x / 2**e; unused
    scale slots are zero."""
    n = k_nope.size(0)
    x = k_nope.float().view(n, layout.scale_active, layout.quant_tile)
    e = tile_exponent(x.abs().amax(dim=-1))
    y = torch.clamp(x * torch.pow(2.0, -e.float()).unsqueeze(-1), -FP8_MAX, FP8_MAX)
    fp8 = y.to(torch.float8_e4m3fn).view(n, layout.d_nope).view(torch.uint8)
    rope = k_rope.contiguous().view(torch.uint8).view(n, 2 * D_ROPE)
    scales = torch.zeros(n, layout.scale_slots, dtype=torch.uint8)
    scales[:, : layout.scale_active] = (e + 127).clamp(0, 254).to(torch.uint8)
    return torch.cat([fp8, rope], dim=1), scales


def store_rows(kv_pages: torch.Tensor, page_block: int, layout: KvLayout,
               slots: torch.Tensor, body: torch.Tensor, scales: torch.Tensor) -> None:
    """Scatter quantised rows into the page-sectioned arena in place; a
    negative slot is skipped."""
    nrb = layout.nope_rope_bytes
    for i, s in enumerate(slots.tolist()):
        if s < 0:
            continue
        p, r = divmod(s, page_block)
        kv_pages[p, r * nrb:(r + 1) * nrb] = body[i]
        o = page_block * nrb + r * layout.scale_slots
        kv_pages[p, o:o + layout.scale_slots] = scales[i]


def build_pages(k_nope: torch.Tensor, k_rope: torch.Tensor, page_block: int,
                layout: KvLayout, page_stride: Optional[int] = None) -> torch.Tensor:
    """Quantise n = num_blocks*page_block tokens in slot order into a fresh arena."""
    n = k_nope.size(0)
    assert n % page_block == 0
    nb = n // page_block
    body, scales = quantize_rows(k_nope, k_rope, layout)
    stride = page_stride or layout.page_bytes(page_block)
    pages = torch.zeros(nb, stride, dtype=torch.uint8)
    nrb = layout.nope_rope_bytes
    pages[:, : page_block * nrb] = body.view(nb, page_block * nrb)
    pages[:, page_block * nrb: page_block * layout.bytes_per_token] = \
        scales.view(nb, page_block * layout.scale_slots)
    return pages
