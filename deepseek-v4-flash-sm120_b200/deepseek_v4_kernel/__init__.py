"""DeepSeek-V4-Flash sparse MLA attention kernels for B200 (sm_100a), behind the
reference project's operator names (reference: deepseek_v4_kernel/__init__.py)."""
from __future__ import annotations

from .ops import sparse_decode_fwd, sparse_prefill_fwd  # noqa: F401
from ._patch import install as patch_flash_mla  # noqa: F401

__all__ = ["sparse_decode_fwd", "sparse_prefill_fwd", "patch_flash_mla"]
