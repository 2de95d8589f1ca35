"""The injection layer, exercised against stub modules standing in for
flash_mla / sgl_kernel (neither is installed here)."""
import importlib
import sys
import types

import pytest
import torch


@pytest.fixture()
def patch_env(monkeypatch):
    import deepseek_v4_kernel._patch as P
    importlib.reload(P)
    calls = {"orig_decode": 0, "orig_prefill": 0, "ours_decode": [], "ours_prefill": 0}

    class Meta:
        class Config(tuple):
            def __new__(cls, *a):
                return super().__new__(cls, a)

        def __init__(self):
            self.tile_scheduler_metadata = None
            self.num_splits = None
            self.have_initialized = False
            self.config = None

    def original(q, k_cache, block_table, cache_seqlens, head_dim_v, tile_scheduler_metadata,
                 num_splits=None, softmax_scale=None, causal=False, is_fp8_kvcache=False,
                 indices=None, attn_sink=None, extra_k_cache=None, extra_indices_in_kvcache=None,
                 topk_length=None, extra_topk_length=None, out=None):
        calls["orig_decode"] += 1
        return "orig_out", "orig_lse"

    fmi = types.ModuleType("flash_mla.flash_mla_interface")
    fmi.flash_mla_with_kvcache = original
    fmi.FlashMLASchedMeta = Meta
    pkg = types.ModuleType("flash_mla")
    pkg.flash_mla_interface = fmi
    pkg.flash_mla_with_kvcache = original
    monkeypatch.setitem(sys.modules, "flash_mla", pkg)
    monkeypatch.setitem(sys.modules, "flash_mla.flash_mla_interface", fmi)

    def orig_prefill(q, kv, indices, sm_scale, d_v=512, attn_sink=None, topk_length=None):
        calls["orig_prefill"] += 1
        return "po", "pm", "pl"

    skf = types.ModuleType("sgl_kernel.flash_mla")
    skf.flash_mla_sparse_fwd = orig_prefill
    sk = types.ModuleType("sgl_kernel")
    sk.flash_mla = skf
    monkeypatch.setitem(sys.modules, "sgl_kernel", sk)
    monkeypatch.setitem(sys.modules, "sgl_kernel.flash_mla", skf)

    def ours_decode(*a):
        calls["ours_decode"].append(a)
        return torch.ones(2), "lse", "meta_t", "splits_t"

    def ours_prefill(*a):
        calls["ours_prefill"] += 1
        return "o", "m", "l"

    monkeypatch.setattr(P, "_decode", ours_decode)
    monkeypatch.setattr(P, "_prefill", ours_prefill)
    monkeypatch.setattr(P, "_device_supported", lambda: True)
    return P, pkg, fmi, skf, Meta, calls


def test_install_wraps_both_entry_points_and_is_idempotent(patch_env):
    P, pkg, fmi, skf, Meta, calls = patch_env
    P.install()
    w = fmi.flash_mla_with_kvcache
    assert getattr(w, "__dsv4_patched__", False) and pkg.flash_mla_with_kvcache is w
    assert getattr(skf.flash_mla_sparse_fwd, "__dsv4_patched__", False)
    P.install()
    assert fmi.flash_mla_with_kvcache is w                    # not wrapped twice


def test_gating_and_schedmeta_update(patch_env):
    P, pkg, fmi, skf, Meta, calls = patch_env
    P.install()
    q = torch.zeros(2, 1, 16, 512, dtype=torch.bfloat16)
    kc = torch.zeros(4, 64, 1, 584, dtype=torch.uint8)
    idx = torch.zeros(2, 1, 64, dtype=torch.int32)
    meta = Meta()
    out, lse = fmi.flash_mla_with_kvcache(q, kc, None, None, 512, meta, is_fp8_kvcache=True,
                                          indices=idx)
    assert lse == "lse" and calls["orig_decode"] == 0
    args = calls["ours_decode"][-1]
    assert args[10] == 512 and abs(args[11] - 512 ** -0.5) < 1e-12     # default scale d_qk^-0.5
    assert meta.tile_scheduler_metadata == "meta_t" and meta.num_splits == "splits_t"
    assert meta.have_initialized and meta.config[0] == 2 and meta.config[7] == 64
    # dense call (no indices), non-fp8 cache, or 4-byte q: the original runs
    assert fmi.flash_mla_with_kvcache(q, kc, None, None, 512, meta, is_fp8_kvcache=True)[0] == "orig_out"
    assert fmi.flash_mla_with_kvcache(q, kc, None, None, 512, meta, indices=idx)[0] == "orig_out"
    assert fmi.flash_mla_with_kvcache(q.float(), kc, None, None, 512, meta, is_fp8_kvcache=True,
                                      indices=idx)[0] == "orig_out"
    assert calls["orig_decode"] == 3


def test_out_keyword_of_newer_interfaces(patch_env):
    P, pkg, fmi, skf, Meta, calls = patch_env
    P.install()
    q = torch.zeros(2, 1, 16, 512, dtype=torch.bfloat16)
    kc = torch.zeros(4, 64, 1, 584, dtype=torch.uint8)
    idx = torch.zeros(2, 1, 64, dtype=torch.int32)
    buf = torch.zeros(2)
    out, _ = fmi.flash_mla_with_kvcache(q, kc, None, None, 512, torch.zeros(1, 8, dtype=torch.int32),
                                        is_fp8_kvcache=True, indices=idx, out=buf)
    assert out is buf and bool((buf == 1).all())


def test_failure_falls_back_unless_strict(patch_env, monkeypatch):
    P, pkg, fmi, skf, Meta, calls = patch_env
    P.install()

    def boom(*a):
        raise RuntimeError("kernel failed")

    monkeypatch.setattr(P, "_decode", boom)
    monkeypatch.setattr(P, "_prefill", boom)
    q = torch.zeros(2, 1, 16, 512, dtype=torch.bfloat16)
    kc = torch.zeros(4, 64, 1, 584, dtype=torch.uint8)
    idx = torch.zeros(2, 1, 64, dtype=torch.int32)
    assert fmi.flash_mla_with_kvcache(q, kc, None, None, 512, None, is_fp8_kvcache=True,
                                      indices=idx)[0] == "orig_out"
    assert skf.flash_mla_sparse_fwd(q, kc, idx, 0.1)[0] == "po"
    monkeypatch.setenv("DSV4_KERNEL_STRICT", "1")
    with pytest.raises(RuntimeError):
        fmi.flash_mla_with_kvcache(q, kc, None, None, 512, None, is_fp8_kvcache=True, indices=idx)
    with pytest.raises(RuntimeError):
        skf.flash_mla_sparse_fwd(q, kc, idx, 0.1)


def test_unsupported_device_defers_to_original(patch_env, monkeypatch):
    P, pkg, fmi, skf, Meta, calls = patch_env
    monkeypatch.setattr(P, "_device_supported", lambda: False)
    P.install()
    assert not getattr(skf.flash_mla_sparse_fwd, "__dsv4_patched__", False)
    q = torch.zeros(2, 1, 16, 512, dtype=torch.bfloat16)
    idx = torch.zeros(2, 1, 64, dtype=torch.int32)
    assert fmi.flash_mla_with_kvcache(q, None, None, None, 512, None, is_fp8_kvcache=True,
                                      indices=idx)[0] == "orig_out"


def test_sitecustomize_hook_honours_disable(monkeypatch, capsys):
    monkeypatch.setenv("DSV4_KERNEL_DISABLE", "1")
    sys.modules.pop("deepseek_v4_kernel.sitecustomize_hook", None)
    importlib.import_module("deepseek_v4_kernel.sitecustomize_hook")
    assert "patch skipped" not in capsys.readouterr().err


def test_host_checks_raise_runtime_error_like_the_reference():
    from deepseek_v4_kernel import ops
    q = torch.zeros(2, 1, 16, 512, dtype=torch.bfloat16)
    kc = torch.zeros(4, 64, 1, 584, dtype=torch.uint8)
    idx = torch.zeros(2, 1, 64, dtype=torch.int32)
    with pytest.raises(RuntimeError, match="CUDA"):
        ops.sparse_decode_fwd(q, kc, idx, None, None, None, None, None, None, None, 512, 0.1)
    with pytest.raises(RuntimeError):
        ops.sparse_prefill_fwd(q[0], kc, idx[:, 0], 0.1)
