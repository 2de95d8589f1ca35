"""Runtime injection: route FlashMLA's sparse FP8 decode and sgl_kernel's sparse
prefill through this package's kernels.

Behaviour follows the reference's `deepseek_v4_kernel/_patch.py`:
  * `flash_mla.flash_mla_interface.flash_mla_with_kvcache` (and the top-level
    re-export) and `vllm.third_party.flashmla.flash_mla_interface.
    flash_mla_with_kvcache` are wrapped; the wrapper takes over only when
    `indices` is given, the cache is FP8, q is a 2-byte type and the device is
    supported, and otherwise calls the original (reference: _patch.py:46-156);
  * `sgl_kernel.flash_mla.flash_mla_sparse_fwd` is wrapped (reference: :201-257);
  * two SGLang indexer helpers get a squeeze of a trailing 1-dim of `seq_lens`
    (reference: :260-296);
  * on an exception the original is called unless DSV4_KERNEL_STRICT=1;
    DSV4_KERNEL_TRACE=1 logs every gating decision; `install()` is idempotent.
Differences: the device gate accepts compute capability 10.x (B200) as well as
12.x, and the decode wrapper tolerates keyword arguments newer FlashMLA
interfaces add (for example `out=`), passing them through to the original.
"""
from __future__ import annotations

import functools
import logging
import os
from typing import Any, Callable, Optional

import torch

from .ops import sparse_decode_fwd as _decode
from .ops import sparse_prefill_fwd as _prefill

_log = logging.getLogger("deepseek_v4_kernel.patch_flash_mla")
_INSTALLED = False
SUPPORTED_MAJORS = (10, 12)

_DECODE_ARGS = ("q", "k_cache", "block_table", "cache_seqlens", "head_dim_v",
                "tile_scheduler_metadata", "num_splits", "softmax_scale", "causal",
                "is_fp8_kvcache", "indices", "attn_sink", "extra_k_cache",
                "extra_indices_in_kvcache", "topk_length", "extra_topk_length")
_DECODE_DEFAULTS = dict(num_splits=None, softmax_scale=None, causal=False, is_fp8_kvcache=False,
                        indices=None, attn_sink=None, extra_k_cache=None,
                        extra_indices_in_kvcache=None, topk_length=None, extra_topk_length=None)


def _device_supported() -> bool:
    if not torch.cuda.is_available():
        return False
    return torch.cuda.get_device_capability(0)[0] in SUPPORTED_MAJORS


def _strict() -> bool:
    return os.environ.get("DSV4_KERNEL_STRICT", "0") == "1"


def _bind(args: tuple, kwargs: dict) -> dict:
    """Positional + keyword arguments of flash_mla_with_kvcache -> one dict."""
    if len(args) > len(_DECODE_ARGS):
        raise TypeError("too many positional arguments")
    bound = dict(_DECODE_DEFAULTS)
    bound.update(zip(_DECODE_ARGS, args))
    bound.update(kwargs)
    return bound


def _make_wrapper(original: Callable, schedmeta_cls: Any) -> Callable:
    """Drop-in replacement for ``flash_mla_with_kvcache``."""

    @functools.wraps(original)
    def flash_mla_with_kvcache(*args, **kwargs):
        a = _bind(args, kwargs)
        q, k_cache, indices = a.get("q"), a.get("k_cache"), a.get("indices")
        gate = (indices is not None, _device_supported(), bool(a["is_fp8_kvcache"]),
                int(q.element_size()) if isinstance(q, torch.Tensor) else None)
        if os.environ.get("DSV4_KERNEL_TRACE", "0") == "1":
            _log.warning("dsv4 gating: %s q=%s kcache=%s", gate,
                         tuple(q.shape) if isinstance(q, torch.Tensor) else q,
                         tuple(k_cache.shape) if isinstance(k_cache, torch.Tensor) else k_cache)
        if all(gate[:3]) and gate[3] == 2:
            try:
                out, lse = _run_decode(a, schedmeta_cls)
                if a.get("out") is not None:      # newer interfaces let the caller own `out`
                    a["out"].copy_(out)
                    out = a["out"]
                return out, lse
            except Exception as exc:  # noqa: BLE001
                if _strict():
                    raise
                _log.warning("deepseek_v4_kernel sparse decode failed (%s); falling back to "
                             "upstream flash_mla.", exc)
        return original(**a)

    flash_mla_with_kvcache.__wrapped__ = original
    flash_mla_with_kvcache.__dsv4_patched__ = True
    return flash_mla_with_kvcache


def _run_decode(a: dict, schedmeta_cls: Any):
    q, k_cache, indices = a["q"], a["k_cache"], a["indices"]
    meta = a["tile_scheduler_metadata"]
    scale = a["softmax_scale"]
    if scale is None:
        scale = q.shape[-1] ** (-0.5)
    is_meta_obj = schedmeta_cls is not None and isinstance(meta, schedmeta_cls)
    sched_t = splits_t = None
    if is_meta_obj:
        sched_t, splits_t = meta.tile_scheduler_metadata, meta.num_splits
    elif isinstance(meta, torch.Tensor):
        sched_t, splits_t = meta, a["num_splits"]
    extra_k, extra_idx = a["extra_k_cache"], a["extra_indices_in_kvcache"]
    out, lse, new_meta, new_splits = _decode(
        q, k_cache, indices, a["topk_length"], a["attn_sink"], sched_t, splits_t, extra_k,
        extra_idx, a["extra_topk_length"], a["head_dim_v"], float(scale))
    if is_meta_obj:
        meta.tile_scheduler_metadata, meta.num_splits = new_meta, new_splits
        if not meta.have_initialized:
            # Fill the config record so later calls pass the interface's own consistency check.
            meta.have_initialized = True
            meta.config = schedmeta_cls.Config(
                q.shape[0], q.shape[1], q.shape[2], k_cache.shape[1], k_cache.shape[2],
                a["causal"], a["is_fp8_kvcache"], indices.shape[-1],
                extra_k.shape[1] if extra_k is not None else None,
                extra_idx.shape[-1] if extra_idx is not None else None)
    return out, lse


def _patch_interface(module: Any, *reexports: Any) -> bool:
    original = getattr(module, "flash_mla_with_kvcache", None)
    if original is None:
        return False
    if getattr(original, "__dsv4_patched__", False):
        return True
    wrapped = _make_wrapper(original, getattr(module, "FlashMLASchedMeta", None))
    module.flash_mla_with_kvcache = wrapped
    for pkg in reexports:
        if pkg is not None and hasattr(pkg, "flash_mla_with_kvcache"):
            pkg.flash_mla_with_kvcache = wrapped
    return True


def _patch_flash_mla_pkg() -> bool:
    try:
        import flash_mla  # type: ignore
        from flash_mla import flash_mla_interface as fmi  # type: ignore
    except ImportError:
        return False
    if not _patch_interface(fmi):
        return False
    flash_mla.flash_mla_with_kvcache = fmi.flash_mla_with_kvcache   # re-export used by sglang
    return True


def _patch_vllm_pkg() -> bool:
    try:
        from vllm.third_party.flashmla import flash_mla_interface as vfmi  # type: ignore
    except Exception:  # noqa: BLE001  (ImportError, or a missing driver library)
        return False
    try:
        from vllm.third_party import flashmla as vpkg  # type: ignore
    except Exception:  # noqa: BLE001
        vpkg = None
    return _patch_interface(vfmi, vpkg)


def _patch_sgl_kernel_sparse_prefill() -> bool:
    """Replace ``sgl_kernel.flash_mla.flash_mla_sparse_fwd`` with this package's
    prefill, keeping its (out, max_logits, lse) contract."""
    if not _device_supported():
        return False
    try:
        from sgl_kernel import flash_mla as skf  # type: ignore
    except Exception:  # noqa: BLE001
        return False
    original = getattr(skf, "flash_mla_sparse_fwd", None)
    if original is None:
        return False
    if getattr(original, "__dsv4_patched__", False):
        return True

    def flash_mla_sparse_fwd(q, kv, indices, sm_scale, d_v=512, attn_sink=None, topk_length=None):
        try:
            return _prefill(q, kv, indices, float(sm_scale), int(d_v), attn_sink, topk_length)
        except Exception as exc:  # noqa: BLE001
            if _strict():
                raise
            _log.warning("deepseek_v4_kernel sparse prefill failed (%s); falling back to the "
                         "stock sgl_kernel prefill.", exc)
            return original(q=q, kv=kv, indices=indices, sm_scale=sm_scale, d_v=d_v,
                            attn_sink=attn_sink, topk_length=topk_length)

    flash_mla_sparse_fwd.__wrapped__ = original
    flash_mla_sparse_fwd.__dsv4_patched__ = True
    skf.flash_mla_sparse_fwd = flash_mla_sparse_fwd
    return True


def _squeeze_seq_lens(owner: Any, name: str) -> None:
    original = getattr(owner, name, None) if owner is not None else None
    if original is None or getattr(original, "__dsv4_patched__", False):
        return

    def wrapper(q_fp8, kvcache_fp8, weight, seq_lens, *args, **kwargs):
        if isinstance(seq_lens, torch.Tensor) and seq_lens.dim() == 2 and seq_lens.shape[-1] == 1:
            seq_lens = seq_lens.squeeze(-1).contiguous()
        return original(q_fp8, kvcache_fp8, weight, seq_lens, *args, **kwargs)

    wrapper.__wrapped__ = original
    wrapper.__dsv4_patched__ = True
    setattr(owner, name, wrapper)


def _patch_sglang_indexer_fallbacks() -> None:
    """SGLang's indexer fallbacks assert a 1-D ``seq_lens`` although their caller
    passes [n, 1]; squeezing the trailing dimension is harmless on every path."""
    try:
        from sglang.srt.layers.attention.nsa import tilelang_kernel as tk  # type: ignore
    except Exception:  # noqa: BLE001
        tk = None
    try:
        from sglang.srt.layers.attention.compressed import indexer as idx  # type: ignore
    except Exception:  # noqa: BLE001
        idx = None
    _squeeze_seq_lens(tk, "tilelang_fp8_paged_mqa_logits")
    _squeeze_seq_lens(idx, "fp8_paged_mqa_logits_torch")


def install() -> None:
    """Install the patch.  Idempotent."""
    global _INSTALLED
    if _INSTALLED:
        return
    results = [_patch_flash_mla_pkg(), _patch_vllm_pkg(), _patch_sgl_kernel_sparse_prefill()]
    _patch_sglang_indexer_fallbacks()
    if not any(results):
        _log.warning("deepseek_v4_kernel: neither flash_mla nor vllm.third_party.flashmla was "
                     "importable; nothing patched.")
        return
    _INSTALLED = True
    cap = torch.cuda.get_device_capability(0) if torch.cuda.is_available() else (-1, -1)
    _log.info("deepseek_v4_kernel.patch_flash_mla installed (device SM %d.%d).", *cap)
