"""Seeded synthetic inputs with the shapes, sizes and value distributions of the
benchmark configurations (decode at serving scale, mixed-length throughput
decode, long-context split-KV decode, causal sparse prefill).  They stand in
for live serving traffic; nothing here reads a dataset.

All generators run on any torch device.  The cache is filled through a
`quantize(k_nope, k_rope, slots, kv)` callable supplied by the caller: the
benchmark passes this package's CUDA store kernel, the tests may pass a CPU
quantiser.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, List, Optional

import torch

PAGE = 64
LAYOUT_BYTES = {"MODEL1": (448, 584), "V32": (512, 644)}     # (d_nope, bytes per token)


def generator(device, seed: int) -> torch.Generator:
    return torch.Generator(device=device).manual_seed(seed)


def empty_cache(num_blocks: int, layout: str, device, page_stride: Optional[int] = None):
    """uint8 cache [num_blocks, PAGE, 1, bytes]; `page_stride` pads each page."""
    _, tok = LAYOUT_BYTES[layout]
    stride = page_stride or PAGE * tok
    arena = torch.zeros((num_blocks, stride), dtype=torch.uint8, device=device)
    return arena[:, : PAGE * tok].view(num_blocks, PAGE, 1, tok) if page_stride is None else \
        torch.as_strided(arena, (num_blocks, PAGE, 1, tok), (stride, tok, tok, 1))


def fill_cache(kv: torch.Tensor, layout: str, quantize: Callable, gen: torch.Generator,
               rope_std: float = 1.0, chunk_pages: int = 1024) -> None:
    """Latent ~ N(0,1), RoPE ~ N(0, rope_std), quantised per tile into `kv`."""
    d_nope, _ = LAYOUT_BYTES[layout]
    dev = kv.device
    nb = kv.size(0)
    for p0 in range(0, nb, chunk_pages):
        n = (min(nb, p0 + chunk_pages) - p0) * PAGE
        k_nope = torch.randn((n, d_nope), device=dev, generator=gen).to(torch.bfloat16)
        k_rope = (torch.randn((n, 64), device=dev, generator=gen) * rope_std).to(torch.bfloat16)
        slots = torch.arange(p0 * PAGE, p0 * PAGE + n, device=dev, dtype=torch.int64)
        quantize(k_nope, k_rope, slots, kv)


@dataclass
class DecodeWorkload:
    name: str
    layout: str
    q: torch.Tensor                    # [b, 1, h_q, d_qk] bf16
    kv: torch.Tensor                   # [num_blocks, PAGE, 1, bytes] uint8
    indices: List[torch.Tensor]        # one or more [b, 1, topk] int32 sets (rotated by the bench)
    sm_scale: float
    topk_length: Optional[torch.Tensor] = None
    attn_sink: Optional[torch.Tensor] = None
    force_splits: Optional[int] = None
    context_lens: List[int] = field(default_factory=list)

    @property
    def shape(self):
        b, _, h_q, d_qk = self.q.shape
        return b, h_q, d_qk, self.indices[0].size(-1)

    def n_valid(self, which: int = 0) -> int:
        """Index slots that gather a row (a negative index gathers nothing)."""
        idx = self.indices[which]
        ok = idx >= 0
        if self.topk_length is not None:
            pos = torch.arange(idx.size(-1), device=idx.device)
            ok = ok & (pos < self.topk_length.clamp(min=1).view(-1, 1, 1))
        return int(ok.sum())

    def algorithmic_bytes(self, which: int = 0) -> int:
        """Bytes one call must move: gathered KV once per request, the index
        list, q, out and lse.  Split-KV partials are overhead and not counted."""
        b, h_q, d_qk, topk = self.shape
        tok = LAYOUT_BYTES[self.layout][1]
        return (self.n_valid(which) * tok + b * topk * 4 + b * h_q * d_qk * 2
                + b * h_q * 512 * 2 + b * h_q * 4)

    def kv_gather_bytes(self, which: int = 0) -> int:
        return self.n_valid(which) * LAYOUT_BYTES[self.layout][1]

    def flops(self, which: int = 0) -> int:
        b, h_q, d_qk, _ = self.shape
        return self.n_valid(which) * h_q * 2 * (d_qk + 512)


def _paged_indices(ctx_lens, topk, page_table, gen, device, clustered_frac=0.0, pad_tail=0):
    """Per request: `topk` distinct logical positions < ctx mapped through the
    request's slice of `page_table` to physical token indices."""
    rows, page0 = [], 0
    for ctx in ctx_lens:
        pages = (ctx + PAGE - 1) // PAGE
        table = page_table[page0:page0 + pages]
        page0 += pages
        n_clu = int(topk * clustered_frac) // PAGE * PAGE
        if n_clu:
            # runs of PAGE consecutive positions starting at random, non-overlapping offsets
            n_runs = n_clu // PAGE
            starts = torch.randperm(ctx // PAGE - 1, device=device, generator=gen)[:n_runs] * PAGE
            starts = starts + torch.randint(0, PAGE, (n_runs,), device=device, generator=gen)
            clu = (starts.view(-1, 1) + torch.arange(PAGE, device=device)).view(-1)
            taken = torch.zeros(ctx, dtype=torch.bool, device=device)
            taken[clu] = True
            rest = torch.nonzero(~taken).view(-1)
            uni = rest[torch.randperm(rest.numel(), device=device, generator=gen)[: topk - n_clu]]
            logical = torch.cat([clu, uni])
            logical = logical[torch.randperm(topk, device=device, generator=gen)]
        else:
            logical = torch.randperm(ctx, device=device, generator=gen)[:topk]
        phys = table[logical // PAGE] * PAGE + logical % PAGE
        if pad_tail:
            phys[-pad_tail:] = -1
        rows.append(phys.to(torch.int32))
    return torch.stack(rows).view(len(ctx_lens), 1, topk)


def decode_workload(name: str, *, b: int, h_q: int, topk: int, ctx_lens, layout: str, device,
                    quantize: Callable, seed: int = 0, n_index_sets: int = 1, pad_tail: int = 0,
                    clustered_frac: float = 0.0, force_splits: Optional[int] = None,
                    q_std: float = 1.0) -> DecodeWorkload:
    """Build a paged FP8 cache holding `ctx_lens[i]` tokens per request behind a
    random page permutation, plus `n_index_sets` independent top-k index sets."""
    gen = generator(device, seed)
    d_qk = LAYOUT_BYTES[layout][0] + 64
    ctx_lens = list(ctx_lens)
    assert len(ctx_lens) == b
    num_blocks = sum((c + PAGE - 1) // PAGE for c in ctx_lens)
    kv = empty_cache(num_blocks, layout, device)
    fill_cache(kv, layout, quantize, gen)
    q = (torch.randn((b, 1, h_q, d_qk), device=device, generator=gen) * q_std).to(torch.bfloat16)
    page_table = torch.randperm(num_blocks, device=device, generator=gen)
    sets = [_paged_indices(ctx_lens, topk, page_table, gen, device, clustered_frac, pad_tail)
            for _ in range(n_index_sets)]
    return DecodeWorkload(name, layout, q, kv, sets, d_qk ** -0.5, force_splits=force_splits,
                          context_lens=ctx_lens)


def config1(device, quantize, layout="V32"):
    """b=1, h_q=16, 4096 cached tokens, top-k 128 with the last 8 entries -1."""
    return decode_workload("cfg1", b=1, h_q=16, topk=128, ctx_lens=[4096], layout=layout,
                           device=device, quantize=quantize, seed=0, pad_tail=8)


def config2(device, quantize, b=16, h_q=64, ctx=32768, topk=2048, layout="V32", n_index_sets=1,
            seed=0):
    """Decode at serving scale: b requests of `ctx` tokens, top-k 2048, no padding."""
    return decode_workload(f"cfg2_b{b}_h{h_q}", b=b, h_q=h_q, topk=topk, ctx_lens=[ctx] * b,
                           layout=layout, device=device, quantize=quantize, seed=seed,
                           n_index_sets=n_index_sets)


def config3(device, quantize, b=16, h_q=64, topk=2048, layout="V32", seed=0, n_index_sets=1,
            ctx_range=(4096, 65536)):
    """Throughput decode: context lengths uniform in ctx_range, half of each
    index list in runs of 64 consecutive positions, half uniform."""
    g = torch.Generator().manual_seed(seed + 1000)
    ctx = torch.randint(ctx_range[0], ctx_range[1] + 1, (b,), generator=g).tolist()
    return decode_workload(f"cfg3_b{b}", b=b, h_q=h_q, topk=topk, ctx_lens=ctx, layout=layout,
                           device=device, quantize=quantize, seed=seed, clustered_frac=0.5,
                           n_index_sets=n_index_sets)


def config4(device, quantize, h_q=64, ctx=131072, topk=2048, layout="V32", splits=128, seed=0):
    """Long-context single stream: 256 trailing -1 entries, forced split count."""
    return decode_workload("cfg4", b=1, h_q=h_q, topk=topk, ctx_lens=[ctx], layout=layout,
                           device=device, quantize=quantize, seed=seed, pad_tail=256,
                           force_splits=splits)


@dataclass
class PrefillWorkload:
    name: str
    q: torch.Tensor          # [s_q, h_q, d_qk]
    kv_bf16: Optional[torch.Tensor]   # [s_kv, d_qk] flat workspace (drop-in entry)
    kv_pages: Optional[torch.Tensor]  # paged FP8 cache (fp8 entry)
    indices: torch.Tensor    # [s_q, topk] int32, causal, -1 padded
    sm_scale: float
    layout: str

    def pairs(self) -> int:
        return int((self.indices >= 0).sum())

    def flops(self) -> int:
        s_q, h_q, d_qk = self.q.shape
        return self.pairs() * h_q * 2 * (d_qk + 512)


def causal_indices(s_q: int, topk: int, device, gen, row0: int = 0) -> torch.Tensor:
    """Query i (global row row0+i) gets min(i+1, topk) distinct positions from
    [0, i], in random order, then -1 padding."""
    rows = torch.arange(row0, row0 + s_q, device=device)
    keys = torch.rand((s_q, row0 + s_q), device=device, generator=gen)
    keys.masked_fill_(torch.arange(row0 + s_q, device=device).view(1, -1) > rows.view(-1, 1), 2.0)
    k = min(topk, row0 + s_q)
    val, idx = torch.topk(keys, k, dim=1, largest=False)
    idx = torch.where(val > 1.5, torch.full_like(idx, -1), idx).to(torch.int32)
    if k < topk:
        idx = torch.cat([idx, torch.full((s_q, topk - k), -1, dtype=torch.int32, device=device)], 1)
    return idx


def config5(device, quantize=None, s_q=8192, h_q=64, topk=2048, layout="V32", seed=0,
            with_pages=True, q_std=1.0):
    """Causal sparse prefill over s_kv = s_q tokens.  Holds both the flat BF16
    workspace and (optionally) the same tokens quantised into the paged cache."""
    gen = generator(device, seed)
    d_nope = LAYOUT_BYTES[layout][0]
    d_qk = d_nope + 64
    q = (torch.randn((s_q, h_q, d_qk), device=device, generator=gen) * q_std).to(torch.bfloat16)
    k_nope = torch.randn((s_q, d_nope), device=device, generator=gen).to(torch.bfloat16)
    k_rope = torch.randn((s_q, 64), device=device, generator=gen).to(torch.bfloat16)
    idx_rows = []
    for r0 in range(0, s_q, 1024):                       # bounded scratch for the top-k draw
        idx_rows.append(causal_indices(min(1024, s_q - r0), topk, device, gen, row0=r0))
    indices = torch.cat(idx_rows)
    kv_pages = None
    if with_pages:
        nb = (s_q + PAGE - 1) // PAGE
        kv_pages = empty_cache(nb, layout, device)
        quantize(k_nope, k_rope, torch.arange(s_q, device=device, dtype=torch.int64), kv_pages)
    kv_bf16 = torch.cat([k_nope, k_rope], dim=1)
    return PrefillWorkload(f"cfg5_s{s_q}", q, kv_bf16, kv_pages, indices, d_qk ** -0.5, layout)
