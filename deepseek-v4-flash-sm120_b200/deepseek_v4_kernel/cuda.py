"""Host launchers over the C-ABI library, exposed under the reference's extension
module name `deepseek_v4_kernel.cuda` with the same function names, argument
order and keyword names (reference: csrc/api/api.cpp:16-40).

Each function validates shapes the way the reference's host code does
(csrc/api/sparse_decode.cpp:43-75, csrc/api/sparse_prefill.cpp:37-86), allocates
outputs and split-KV scratch through torch (so the caching allocator and CUDA
graph pools apply), fills the POD argument block and queues the kernels on the
current stream.  Nothing here computes attention on the host and there is no
fallback path: without the native library this module cannot be imported.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional, Tuple

import torch

from . import _native as N

_KV_DTYPES = (torch.float8_e4m3fn, torch.uint8, torch.int8)
_SCHED_META_INT32S = 8        # 32-byte record kept for FlashMLA binary parity
_sm_count = {}


def _require(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def num_sms(device: torch.device) -> int:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _sm_count:
        sms = C.c_int(0)
        N.check(N.lib.dsv4_device_info(idx, None, None, C.byref(sms)), "dsv4_device_info")
        _sm_count[idx] = sms.value
    return _sm_count[idx]


def plan_splits(b: int, s_q: int, h_q: int, topk: int, extra_topk: int, sms: int) -> int:
    forced = os.environ.get("DSV4_FORCE_SPLITS")
    if forced:
        return max(1, int(forced))
    return N.lib.dsv4_plan_splits(b, s_q, h_q, topk, extra_topk, sms)


def _kv_format(d_qk: int, token_bytes: int) -> int:
    if d_qk == 512 and token_bytes == 584:
        return N.KV_MODEL1
    if d_qk == 576 and token_bytes == 644:
        return N.KV_V32
    raise RuntimeError(
        "unsupported cache layout: expected d_qk=512 with 584 bytes/token (448 FP8 + 7 UE8M0 "
        "+ 1 pad + 64 BF16 RoPE) or d_qk=576 with 644 bytes/token (512 FP8 + 4 UE8M0 + 64 BF16 "
        f"RoPE), got d_qk={d_qk}, {token_bytes} bytes/token")


def _flags() -> int:
    f = 0
    if os.environ.get("DSV4_MASK_INVALID", "0") == "1":
        f |= N.FLAG_MASK_INVALID
    return f


def sparse_decode_fwd(q, kv, indices, topk_length, attn_sink, tile_scheduler_metadata,
                      num_splits, extra_kv, extra_indices, extra_topk_length, d_v, sm_scale,
                      *, n_splits: Optional[int] = None, flags: int = 0):
    """Sparse MLA decode forward.  Same contract as the reference's
    `sparse_decode_fwd` (csrc/api/sparse_decode.cpp:27-41):

      q [b, s_q, h_q, d_qk] bf16; kv [num_blocks, page_block, 1, bytes] fp8/uint8/int8;
      indices [b, s_q, topk] int32 -> (out [b, s_q, h_q, 512] bf16, lse [b, h_q, s_q] fp32,
      tile_scheduler_metadata, num_splits)

    Beyond the reference: s_q > 1 is accepted, and the 576/644-byte layout.
    `n_splits` / `flags` are test hooks (forced split count, Dsv4Flags).
    """
    _require(q.is_cuda and kv.is_cuda, "q and kv must be CUDA tensors")
    _require(q.dim() == 4, "q must be 4-D [b, s_q, h_q, d_qk]")
    _require(kv.dim() == 4, "kv must be 4-D [num_blocks, page_block, h_kv, bytes]")
    _require(indices.dim() == 3, "indices must be 3-D [b, s_q, topk]")
    _require(q.dtype == torch.bfloat16, "q must be bf16")
    _require(kv.dtype in _KV_DTYPES, "kv must be fp8_e4m3 / uint8 / int8 (packed layout)")
    _require(indices.dtype == torch.int32, "indices must be int32")
    b, s_q, h_q, d_qk = q.shape
    num_blocks, page_block, h_kv, token_bytes = kv.shape
    topk = indices.size(2)
    _require(h_kv == 1, "Only MQA (h_kv=1) is supported for sparse decode")
    _require(int(d_v) == 512, "Only d_v=512 supported")
    _require(indices.size(0) == b and indices.size(1) == s_q, "indices must be [b, s_q, topk]")
    fmt = _kv_format(d_qk, token_bytes)
    _require(q.stride(3) == 1 and indices.stride(2) == 1, "q and indices must be dense in the last dim")
    _require(kv.stride(1) == token_bytes and kv.stride(3) == 1,
             "kv pages must be dense (only the page stride may be padded)")
    for name, t, n in (("topk_length", topk_length, b), ("extra_topk_length", extra_topk_length, b)):
        if t is not None:
            _require(t.dtype == torch.int32 and t.numel() == n and t.is_contiguous(),
                     f"{name} must be contiguous int32 [{n}]")
    if attn_sink is not None:
        _require(attn_sink.dtype == torch.float32 and attn_sink.numel() == h_q
                 and attn_sink.is_contiguous(), "attn_sink must be contiguous float32 [h_q]")
    x_blocks = x_page = x_topk = 0
    if extra_kv is not None:
        _require(extra_indices is not None, "extra_indices required when extra_kv is provided")
        _require(extra_kv.dim() == 4 and extra_kv.size(3) == token_bytes and extra_kv.size(2) == 1,
                 "extra_kv must use the same token layout as kv")
        _require(extra_indices.dtype == torch.int32 and extra_indices.dim() == 3
                 and extra_indices.stride(2) == 1, "extra_indices must be int32 [b, s_q, extra_topk]")
        x_blocks, x_page, x_topk = extra_kv.size(0), extra_kv.size(1), extra_indices.size(2)

    with torch.cuda.device(q.device):
        out = torch.empty((b, s_q, h_q, 512), dtype=torch.bfloat16, device=q.device)
        lse = torch.empty((b, h_q, s_q), dtype=torch.float32, device=q.device)
        if n_splits is None:
            n_splits = plan_splits(b, s_q, h_q, topk, x_topk, num_sms(q.device))
        o_accum = lse_accum = None
        if n_splits > 1:
            o_accum = torch.empty((n_splits, b * s_q, h_q, 512), dtype=torch.float32, device=q.device)
            lse_accum = torch.empty((n_splits, b * s_q, h_q), dtype=torch.float32, device=q.device)
        if tile_scheduler_metadata is None:
            tile_scheduler_metadata = torch.empty((1, _SCHED_META_INT32S), dtype=torch.int32,
                                                  device=q.device)
            num_splits = torch.empty((b + 1,), dtype=torch.int32, device=q.device)

        a = N.DecodeArgs()
        a.b, a.s_q, a.h_q, a.d_qk, a.d_v, a.topk = b, s_q, h_q, d_qk, 512, topk
        a.kv_format, a.num_blocks, a.page_block_size = fmt, num_blocks, page_block
        a.extra_num_blocks, a.extra_page_block_size, a.extra_topk = x_blocks, x_page, x_topk
        a.n_splits, a.flags, a.sm_scale = n_splits, flags | _flags(), float(sm_scale)
        a.q, a.kv, a.indices = q.data_ptr(), kv.data_ptr(), indices.data_ptr()
        a.topk_length, a.attn_sink = _ptr(topk_length), _ptr(attn_sink)
        a.extra_kv, a.extra_indices = _ptr(extra_kv), _ptr(extra_indices)
        a.extra_topk_length = _ptr(extra_topk_length)
        a.out, a.lse, a.o_accum, a.lse_accum = out.data_ptr(), lse.data_ptr(), _ptr(o_accum), _ptr(lse_accum)
        a.stride_q_b, a.stride_q_s, a.stride_q_h = q.stride(0), q.stride(1), q.stride(2)
        a.stride_kv_block = kv.stride(0)
        a.stride_indices_b, a.stride_indices_s = indices.stride(0), indices.stride(1)
        if extra_kv is not None:
            a.stride_extra_kv_block = extra_kv.stride(0)
            a.stride_extra_indices_b = extra_indices.stride(0)
            a.stride_extra_indices_s = extra_indices.stride(1)
        a.stride_o_b, a.stride_o_s, a.stride_o_h = out.stride(0), out.stride(1), out.stride(2)
        # lse is produced directly in the reference's returned [b, h_q, s_q] arrangement.
        a.stride_lse_b, a.stride_lse_h, a.stride_lse_s = lse.stride(0), lse.stride(1), lse.stride(2)
        stream = torch.cuda.current_stream(q.device).cuda_stream
        N.check(N.lib.dsv4_sparse_decode(C.byref(a), stream), "dsv4_sparse_decode")
    return out, lse, tile_scheduler_metadata, num_splits


def _prefill(q, kv, indices, sm_scale, d_v, attn_sink, topk_length, fmt, num_blocks, page_block,
             s_kv, stride_kv, flags):
    s_q, h_q, d_qk = q.shape
    topk = indices.size(1)
    with torch.cuda.device(q.device):
        out = torch.empty((s_q, h_q, 512), dtype=torch.bfloat16, device=q.device)
        max_logits = torch.empty((s_q, h_q), dtype=torch.float32, device=q.device)
        lse = torch.empty((s_q, h_q), dtype=torch.float32, device=q.device)
        a = N.PrefillArgs()
        a.s_q, a.s_kv, a.h_q, a.d_qk, a.d_v, a.topk = s_q, s_kv, h_q, d_qk, 512, topk
        a.kv_format, a.num_blocks, a.page_block_size = fmt, num_blocks, page_block
        a.flags, a.sm_scale = flags, float(sm_scale)
        a.q, a.kv, a.indices = q.data_ptr(), kv.data_ptr(), indices.data_ptr()
        a.attn_sink, a.topk_length = _ptr(attn_sink), _ptr(topk_length)
        a.out, a.max_logits, a.lse = out.data_ptr(), max_logits.data_ptr(), lse.data_ptr()
        a.stride_q_s, a.stride_q_h = q.stride(0), q.stride(1)
        a.stride_kv_row, a.stride_indices_s = stride_kv, indices.stride(0)
        a.stride_o_s, a.stride_o_h = out.stride(0), out.stride(1)
        a.stride_ml_s, a.stride_lse_s = max_logits.stride(0), lse.stride(0)
        stream = torch.cuda.current_stream(q.device).cuda_stream
        N.check(N.lib.dsv4_sparse_prefill(C.byref(a), stream), "dsv4_sparse_prefill")
    return out, max_logits, lse


def _prefill_common_checks(q, indices, d_v, attn_sink, topk_length):
    _require(q.is_cuda, "q must be a CUDA tensor")
    _require(q.dim() == 3, "q must be 3-D [s_q, h_q, d_qk]")
    _require(q.dtype == torch.bfloat16, "q must be bf16")
    _require(indices.dtype == torch.int32, "indices must be int32")
    idx2 = indices.squeeze(1) if indices.dim() == 3 else indices
    _require(idx2.dim() == 2, "indices must be [s_q, topk] (or [s_q,1,topk])")
    s_q, h_q, _ = q.shape
    _require(int(d_v) == 512, "Only d_v=512 supported")
    _require(idx2.size(0) == s_q, f"indices s_q ({idx2.size(0)}) must match q s_q ({s_q})")
    _require(q.stride(2) == 1, f"q must be contiguous in d_qk (stride(2)==1); got {q.stride(2)}")
    _require(idx2.stride(1) == 1,
             f"indices must be contiguous in topk (stride==1); got {idx2.stride(1)}")
    if attn_sink is not None:
        _require(attn_sink.dtype == torch.float32, "attn_sink must be float32")
        _require(attn_sink.numel() == h_q and attn_sink.is_contiguous(),
                 f"attn_sink must have h_q ({h_q}) elements; got {attn_sink.numel()}")
    if topk_length is not None:
        _require(topk_length.dtype == torch.int32, "topk_length must be int32")
        _require(topk_length.numel() == s_q and topk_length.is_contiguous(),
                 f"topk_length must have s_q ({s_q}) elements; got {topk_length.numel()}")
    return idx2


def sparse_prefill_fwd(q, kv, indices, sm_scale, d_v=512, attn_sink=None, topk_length=None,
                       *, flags: int = 0):
    """Sparse MLA prefill over a flat BF16 workspace; drop-in for the reference's
    `sparse_prefill_fwd` (csrc/api/sparse_prefill.cpp:27-35):

      q [s_q, h_q, d_qk] bf16; kv [s_kv, (1,) d_qk] bf16; indices [s_q, (1,) topk] int32
      -> (out [s_q, h_q, 512] bf16, max_logits [s_q, h_q] fp32, lse [s_q, h_q] fp32)
    """
    _require(kv.is_cuda, "q and kv must be CUDA tensors")
    _require(kv.dtype == torch.bfloat16, "kv must be bf16 (dequantised workspace)")
    idx2 = _prefill_common_checks(q, indices, d_v, attn_sink, topk_length)
    kv_flat = kv.squeeze(1) if kv.dim() == 3 else kv
    _require(kv_flat.dim() == 2, "kv must be [s_kv, d_qk] (or [s_kv,1,d_qk])")
    d_qk = q.size(2)
    _require(d_qk in (512, 576), f"expected d_qk=512 (or 576), got {d_qk}")
    _require(kv_flat.size(1) == d_qk, f"kv last dim must be {d_qk}, got {kv_flat.size(1)}")
    _require(kv_flat.stride(1) == 1,
             f"kv must be contiguous in d_qk (stride==1); got {kv_flat.stride(1)}")
    return _prefill(q, kv_flat, idx2, sm_scale, d_v, attn_sink, topk_length, N.KV_BF16, 0, 1,
                    kv_flat.size(0), kv_flat.stride(0), flags)


def sparse_prefill_fwd_fp8(q, kv, indices, sm_scale, d_v=512, attn_sink=None, topk_length=None,
                           *, flags: int = 0):
    """Sparse MLA prefill reading the FP8 paged cache directly (no BF16 workspace).
    kv [num_blocks, page_block, 1, bytes] as for decode; other arguments and the
    returns as sparse_prefill_fwd.  No counterpart in the reference, whose caller
    dequantises first (csrc/common/params.h:99-102)."""
    _require(kv.is_cuda and kv.dim() == 4 and kv.dtype in _KV_DTYPES and kv.size(2) == 1,
             "kv must be a CUDA [num_blocks, page_block, 1, bytes] fp8/uint8/int8 tensor")
    idx2 = _prefill_common_checks(q, indices, d_v, attn_sink, topk_length)
    fmt = _kv_format(q.size(2), kv.size(3))
    _require(kv.stride(1) == kv.size(3) and kv.stride(3) == 1, "kv pages must be dense")
    return _prefill(q, kv, idx2, sm_scale, d_v, attn_sink, topk_length, fmt, kv.size(0),
                    kv.size(1), kv.size(0) * kv.size(1), kv.stride(0), flags)


def kv_store(k_nope, k_rope, slots, kv) -> None:
    """Quantise and store tokens into the paged cache in place.
    k_nope [n, 448|512] bf16, k_rope [n, 64] bf16, slots [n] int64 (negative = skip),
    kv [num_blocks, page_block, 1, 584|644]."""
    _require(k_nope.is_cuda and kv.is_cuda and kv.dim() == 4, "k_nope / kv must be CUDA tensors")
    _require(k_nope.dtype == torch.bfloat16 and k_rope.dtype == torch.bfloat16, "inputs must be bf16")
    _require(slots.dtype == torch.int64 and slots.is_contiguous(), "slots must be contiguous int64")
    n = k_nope.size(0)
    fmt = _kv_format(k_nope.size(1) + 64, kv.size(3))
    _require(k_rope.shape == (n, 64) and slots.numel() == n, "k_rope [n,64], slots [n] expected")
    _require(k_nope.stride(1) == 1 and k_rope.stride(1) == 1, "inputs must be dense rows")
    _require(kv.dtype in _KV_DTYPES and kv.stride(1) == kv.size(3) and kv.stride(3) == 1,
             "kv pages must be dense fp8/uint8/int8")
    a = N.StoreArgs()
    a.n_tokens, a.kv_format, a.num_blocks, a.page_block_size = n, fmt, kv.size(0), kv.size(1)
    a.k_nope, a.k_rope, a.slots, a.kv = k_nope.data_ptr(), k_rope.data_ptr(), slots.data_ptr(), kv.data_ptr()
    a.stride_nope, a.stride_rope, a.stride_kv_block = k_nope.stride(0), k_rope.stride(0), kv.stride(0)
    with torch.cuda.device(kv.device):
        N.check(N.lib.dsv4_kv_store(C.byref(a), torch.cuda.current_stream(kv.device).cuda_stream),
                "dsv4_kv_store")


def kv_store_rows(k, loc, kv) -> None:
    """Quantise and store tokens given as the cache writer of the serving framework has
    them: k [n, d_qk] or [n, 1, d_qk] bf16 (latent values then the 64 RoPE values; any row
    stride that is a multiple of 8 elements, so a column slice of a wider projection output
    is taken as it is), loc [n] int32 or int64 cache slots (negative = skip),
    kv [num_blocks, page_block, 1, 584|644].  Same bytes as `kv_store`."""
    _require(k.is_cuda and kv.is_cuda and kv.dim() == 4, "k / kv must be CUDA tensors")
    _require(k.dtype == torch.bfloat16, "k must be bf16")
    if k.dim() == 3:
        _require(k.size(1) == 1, "k must be [n, d_qk] or [n, 1, d_qk]")
        k = k[:, 0]
    _require(k.dim() == 2 and k.stride(1) == 1, "k rows must be dense")
    _require(loc.dtype in (torch.int32, torch.int64) and loc.is_contiguous() and loc.numel() == k.size(0),
             "loc must be contiguous int32/int64 [n]")
    fmt = _kv_format(k.size(1), kv.size(3))
    _require(kv.dtype in _KV_DTYPES and kv.stride(1) == kv.size(3) and kv.stride(3) == 1,
             "kv pages must be dense fp8/uint8/int8")
    a = N.StoreRowsArgs()
    a.n_tokens, a.kv_format, a.num_blocks, a.page_block_size = k.size(0), fmt, kv.size(0), kv.size(1)
    a.k, a.loc, a.kv = k.data_ptr(), loc.data_ptr(), kv.data_ptr()
    a.stride_k, a.stride_kv_block = (k.stride(0) if k.size(0) > 1 else k.size(1)), kv.stride(0)
    a.loc_is_int64 = int(loc.dtype == torch.int64)
    with torch.cuda.device(kv.device):
        N.check(N.lib.dsv4_kv_store_rows(C.byref(a), torch.cuda.current_stream(kv.device).cuda_stream),
                "dsv4_kv_store_rows")


def gather_dequant(kv, indices, method: int = 0) -> torch.Tensor:
    """Dequantised BF16 rows [n, d_qk] of the tokens named by int32 `indices` [n]."""
    _require(kv.is_cuda and kv.dim() == 4 and indices.dtype == torch.int32, "bad arguments")
    d_qk = 512 if kv.size(3) == 584 else 576
    fmt = _kv_format(d_qk, kv.size(3))
    idx = indices.contiguous().view(-1)
    rows = torch.empty((idx.numel(), d_qk), dtype=torch.bfloat16, device=kv.device)
    with torch.cuda.device(kv.device):
        N.check(N.lib.dsv4_gather_dequant(kv.data_ptr(), kv.stride(0), fmt, kv.size(0), kv.size(1),
                                          idx.data_ptr(), idx.numel(), rows.data_ptr(), method,
                                          torch.cuda.current_stream(kv.device).cuda_stream),
                "dsv4_gather_dequant")
    return rows


def split_combine(o_accum, lse_accum, attn_sink=None, s_q: int = 1):
    """Merge split-KV partials: o_accum fp32 [n_splits, n_rows, h_q, 512], lse_accum fp32
    [n_splits, n_rows, h_q] -> (out bf16 [n_rows, h_q, 512], lse fp32 [n_rows, h_q])."""
    _require(o_accum.is_cuda and o_accum.dtype == torch.float32 and o_accum.is_contiguous()
             and lse_accum.dtype == torch.float32 and lse_accum.is_contiguous(), "bad partials")
    n_splits, n_rows, h_q, d_v = o_accum.shape
    _require(d_v == 512 and lse_accum.shape == (n_splits, n_rows, h_q), "bad partial shapes")
    out = torch.empty((n_rows, h_q, 512), dtype=torch.bfloat16, device=o_accum.device)
    lse = torch.empty((n_rows, h_q), dtype=torch.float32, device=o_accum.device)
    a = N.CombineArgs()
    a.n_rows, a.s_q, a.h_q, a.n_splits = n_rows, 1, h_q, n_splits
    a.o_accum, a.lse_accum, a.attn_sink = o_accum.data_ptr(), lse_accum.data_ptr(), _ptr(attn_sink)
    a.out, a.lse = out.data_ptr(), lse.data_ptr()
    a.stride_o_b, a.stride_o_s, a.stride_o_h = out.stride(0), 0, out.stride(1)
    a.stride_lse_b, a.stride_lse_s, a.stride_lse_h = lse.stride(0), 0, 1
    with torch.cuda.device(o_accum.device):
        N.check(N.lib.dsv4_split_combine(C.byref(a), torch.cuda.current_stream(o_accum.device).cuda_stream),
                "dsv4_split_combine")
    return out, lse


def device_status(reset: bool = True) -> int:
    """Health word of the tensor-core kernels on the current device (synchronises)."""
    v = C.c_int32(0)
    N.check(N.lib.dsv4_device_status(C.byref(v), 1 if reset else 0), "dsv4_device_status")
    return v.value


def umma_selftest(mode: int, a: torch.Tensor, b: torch.Tensor) -> Tuple[torch.Tensor, int]:
    """Run the tensor-core self-test; see dsv4_umma_selftest in the C header."""
    if mode == 0:
        k, n = a.size(1), b.size(0)
    else:
        k, n = a.size(0), b.size(1)
    d = torch.zeros((128, n), dtype=torch.float32, device=a.device)
    status = torch.full((1,), -1, dtype=torch.int32, device=a.device)
    with torch.cuda.device(a.device):
        N.check(N.lib.dsv4_umma_selftest(mode, n, k, a.data_ptr(), b.data_ptr(), d.data_ptr(),
                                         status.data_ptr(),
                                         torch.cuda.current_stream(a.device).cuda_stream),
                "dsv4_umma_selftest")
    return d, int(status.item())


class DecodeCall:
    """A prepared decode launch over fixed buffers: the argument block is built
    once and re-queued with `decode()` / `combine()`, so the two kernels can be
    launched (and timed) separately and a serving loop or CUDA graph pays no
    per-step host work.  Tensors are borrowed; keep them alive."""

    def __init__(self, q, kv, indices, sm_scale, topk_length=None, attn_sink=None,
                 n_splits: Optional[int] = None, flags: int = 0):
        b, s_q, h_q, d_qk = q.shape
        self.q, self.kv, self.indices = q, kv, indices
        self.keep = (topk_length, attn_sink)
        dev = q.device
        self.n_splits = n_splits or plan_splits(b, s_q, h_q, indices.size(2), 0, num_sms(dev))
        self.out = torch.empty((b, s_q, h_q, 512), dtype=torch.bfloat16, device=dev)
        self.lse = torch.empty((b, h_q, s_q), dtype=torch.float32, device=dev)
        self.o_accum = self.lse_accum = None
        if self.n_splits > 1:
            self.o_accum = torch.empty((self.n_splits, b * s_q, h_q, 512), dtype=torch.float32, device=dev)
            self.lse_accum = torch.empty((self.n_splits, b * s_q, h_q), dtype=torch.float32, device=dev)
        a = N.DecodeArgs()
        a.b, a.s_q, a.h_q, a.d_qk, a.d_v, a.topk = b, s_q, h_q, d_qk, 512, indices.size(2)
        a.kv_format = _kv_format(d_qk, kv.size(3))
        a.num_blocks, a.page_block_size = kv.size(0), kv.size(1)
        a.n_splits, a.flags, a.sm_scale = self.n_splits, flags, float(sm_scale)
        a.q, a.kv, a.indices = q.data_ptr(), kv.data_ptr(), indices.data_ptr()
        a.topk_length, a.attn_sink = _ptr(topk_length), _ptr(attn_sink)
        a.out, a.lse = self.out.data_ptr(), self.lse.data_ptr()
        a.o_accum, a.lse_accum = _ptr(self.o_accum), _ptr(self.lse_accum)
        a.stride_q_b, a.stride_q_s, a.stride_q_h = q.stride(0), q.stride(1), q.stride(2)
        a.stride_kv_block = kv.stride(0)
        a.stride_indices_b, a.stride_indices_s = indices.stride(0), indices.stride(1)
        a.stride_o_b, a.stride_o_s, a.stride_o_h = self.out.stride(0), self.out.stride(1), self.out.stride(2)
        a.stride_lse_b, a.stride_lse_h, a.stride_lse_s = self.lse.stride(0), self.lse.stride(1), self.lse.stride(2)
        self.args = a
        # partial sets the decode kernel leaves behind (splits are merged in groups on chip)
        self.partial_sets = N.lib.dsv4_decode_partial_sets(C.byref(a))
        c = N.CombineArgs()
        c.n_rows, c.s_q, c.h_q, c.n_splits = b * s_q, s_q, h_q, self.partial_sets
        c.o_accum, c.lse_accum, c.attn_sink = a.o_accum, a.lse_accum, a.attn_sink
        c.out, c.lse = a.out, a.lse
        c.stride_o_b, c.stride_o_s, c.stride_o_h = a.stride_o_b, a.stride_o_s, a.stride_o_h
        c.stride_lse_b, c.stride_lse_s, c.stride_lse_h = a.stride_lse_b, a.stride_lse_s, a.stride_lse_h
        self.cargs = c
        self.base_flags = flags

    def set_indices(self, indices: torch.Tensor) -> None:
        self.indices = indices
        self.args.indices = indices.data_ptr()

    def decode(self, stream: int, with_combine: bool = True) -> None:
        self.args.flags = self.base_flags | (0 if with_combine else N.FLAG_NO_COMBINE)
        N.check(N.lib.dsv4_sparse_decode(C.byref(self.args), stream), "dsv4_sparse_decode")

    def combine(self, stream: int) -> None:
        if self.partial_sets > 1:
            N.check(N.lib.dsv4_split_combine(C.byref(self.cargs), stream), "dsv4_split_combine")

    @property
    def launches_per_call(self) -> int:
        return 2 if self.partial_sets > 1 else 1
