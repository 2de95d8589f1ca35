"""Shared helpers for the test-suite."""
from __future__ import annotations

import os

import numpy as np
import torch

from oracle import sparse_mla as O

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
BF16_KEYS = {"q", "out", "kv", "dense_head"}


def load_golden(name: str) -> dict:
    """Golden file -> dict of torch tensors (BF16 restored from its bit pattern)."""
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    out = {}
    for k in z.files:
        a = z[k]
        if k in BF16_KEYS:
            out[k] = torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)
        elif a.ndim == 0:
            out[k] = a.item()
        else:
            out[k] = torch.from_numpy(a.copy())
    return out


def cpu_quantize(k_nope, k_rope, slots, kv):
    """`quantize` callable for the workload generators, backed by the oracle."""
    layout = O.V32 if kv.size(3) == 644 else O.MODEL1
    body, scales = O.quantize_rows(k_nope.cpu(), k_rope.cpu(), layout)
    arena = kv.view(kv.size(0), -1)
    O.store_rows(arena, kv.size(1), layout, slots.cpu(), body, scales)


def arena2d(kv4: torch.Tensor) -> torch.Tensor:
    """[num_blocks, P, 1, bytes] cache view -> uint8 [num_blocks, page_bytes] on CPU."""
    nb = kv4.size(0)
    flat = torch.as_strided(kv4, (nb, kv4.size(1) * kv4.size(3)), (kv4.stride(0), 1))
    return flat.cpu().view(torch.uint8) if flat.dtype != torch.uint8 else flat.cpu()


def max_rel_err(got: torch.Tensor, ref: torch.Tensor) -> float:
    """max |got - ref| / max |ref| — the 'max relative error' of the acceptance bar."""
    ref = ref.float()
    return float((got.float() - ref).abs().max() / ref.abs().max().clamp_min(1e-30))
