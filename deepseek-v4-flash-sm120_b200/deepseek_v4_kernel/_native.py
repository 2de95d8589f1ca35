"""ctypes binding of the C-ABI library `libdsv4_b200.so` (see include/dsv4_b200.h).

The library is built in-tree next to this file.  There is no fallback: if it is
missing, importing this module raises.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# DSV4_B200_LIB names another build of the same library (e.g. one compiled with debug defines).
LIB_PATH = os.environ.get("DSV4_B200_LIB") or os.path.join(_HERE, "libdsv4_b200.so")

KV_BF16, KV_MODEL1, KV_V32 = 0, 1, 2
FLAG_MASK_INVALID, FLAG_IMPL_SIMPLE, FLAG_NO_COMBINE, FLAG_ZERO_LENGTH_EMPTY = 1, 2, 4, 8
ABI_VERSION = 1

i32, i64, f32, vp = C.c_int32, C.c_int64, C.c_float, C.c_void_p


class DecodeArgs(C.Structure):
    _fields_ = [(n, i32) for n in (
        "b", "s_q", "h_q", "d_qk", "d_v", "topk", "kv_format", "num_blocks", "page_block_size",
        "extra_num_blocks", "extra_page_block_size", "extra_topk", "n_splits", "flags")] + [
        ("sm_scale", f32), ("_pad0", i32)] + [(n, vp) for n in (
            "q", "kv", "indices", "topk_length", "attn_sink", "extra_kv", "extra_indices",
            "extra_topk_length", "out", "lse", "o_accum", "lse_accum")] + [(n, i64) for n in (
                "stride_q_b", "stride_q_s", "stride_q_h", "stride_kv_block",
                "stride_extra_kv_block", "stride_indices_b", "stride_indices_s",
                "stride_extra_indices_b", "stride_extra_indices_s", "stride_o_b", "stride_o_s",
                "stride_o_h", "stride_lse_b", "stride_lse_s", "stride_lse_h")]


MAX_PEERS = 8


class GatherArgs(C.Structure):
    _fields_ = [(n, i32) for n in ("world", "rank", "b", "s_q", "h_local", "step")] + [
        ("out_local", vp), ("lse_local", vp), ("peer_out", vp * MAX_PEERS),
        ("peer_lse", vp * MAX_PEERS), ("peer_flags", vp * MAX_PEERS), ("counter", vp),
        ("status", vp)]


class CombineArgs(C.Structure):
    _fields_ = [(n, i32) for n in ("n_rows", "s_q", "h_q", "n_splits")] + [(n, vp) for n in (
        "o_accum", "lse_accum", "attn_sink", "out", "lse")] + [(n, i64) for n in (
            "stride_o_b", "stride_o_s", "stride_o_h", "stride_lse_b", "stride_lse_s",
            "stride_lse_h")]


class PrefillArgs(C.Structure):
    _fields_ = [(n, i32) for n in (
        "s_q", "s_kv", "h_q", "d_qk", "d_v", "topk", "kv_format", "num_blocks",
        "page_block_size", "flags")] + [("sm_scale", f32), ("_pad0", i32)] + [(n, vp) for n in (
            "q", "kv", "indices", "attn_sink", "topk_length", "out", "max_logits", "lse")] + [
        (n, i64) for n in ("stride_q_s", "stride_q_h", "stride_kv_row", "stride_indices_s",
                           "stride_o_s", "stride_o_h", "stride_ml_s", "stride_lse_s")]


class StoreArgs(C.Structure):
    _fields_ = [(n, i32) for n in ("n_tokens", "kv_format", "num_blocks", "page_block_size")] + [
        (n, vp) for n in ("k_nope", "k_rope", "slots", "kv")] + [
        (n, i64) for n in ("stride_nope", "stride_rope", "stride_kv_block")]


class StoreRowsArgs(C.Structure):
    _fields_ = [(n, i32) for n in ("n_tokens", "kv_format", "num_blocks", "page_block_size")] + [
        (n, vp) for n in ("k", "loc", "kv")] + [
        (n, i64) for n in ("stride_k", "stride_kv_block")] + [
        (n, i32) for n in ("loc_is_int64", "reserved")]


# name -> (restype, argtypes); every symbol include/dsv4_b200.h declares.
SYMBOLS = {
    "dsv4_abi_version": (C.c_int, []),
    "dsv4_strerror": (C.c_char_p, [C.c_int]),
    "dsv4_last_cuda_error": (C.c_char_p, []),
    "dsv4_device_info": (C.c_int, [C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int),
                                   C.POINTER(C.c_int)]),
    "dsv4_plan_splits": (C.c_int, [C.c_int] * 6),
    "dsv4_gather_heads": (C.c_int, [C.POINTER(GatherArgs), C.c_void_p]),
    "dsv4_sparse_decode_gather": (C.c_int, [C.POINTER(DecodeArgs), C.POINTER(GatherArgs), C.c_void_p]),
    "dsv4_decode_partial_sets": (C.c_int, [C.POINTER(DecodeArgs)]),
    "dsv4_sparse_decode": (C.c_int, [C.POINTER(DecodeArgs), vp]),
    "dsv4_sparse_decode_noalloc": (C.c_int, [C.POINTER(DecodeArgs), vp]),
    "dsv4_split_combine": (C.c_int, [C.POINTER(CombineArgs), vp]),
    "dsv4_sparse_prefill": (C.c_int, [C.POINTER(PrefillArgs), vp]),
    "dsv4_kv_store": (C.c_int, [C.POINTER(StoreArgs), vp]),
    "dsv4_kv_store_rows": (C.c_int, [C.POINTER(StoreRowsArgs), vp]),
    "dsv4_gather_dequant": (C.c_int, [vp, i64, i32, i32, i32, vp, i32, vp, i32, vp]),
    "dsv4_device_status": (C.c_int, [C.POINTER(C.c_int32), C.c_int]),
    "dsv4_debug_set_timeline": (C.c_int, [vp]),
    "dsv4_umma_selftest": (C.c_int, [C.c_int, C.c_int, C.c_int, vp, vp, vp, vp, vp]),
}


def _load() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} not built. Run `python -c 'import __graft_entry__ as g; g.build()'` "
            "at the repository root (or build_native.py next to this package).")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SYMBOLS.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    if lib.dsv4_abi_version() != ABI_VERSION:
        raise ImportError("libdsv4_b200.so ABI version does not match this binding; rebuild")
    return lib


lib = _load()


def check(rc: int, what: str) -> None:
    """Raise RuntimeError for a non-zero status (mirrors TORCH_CHECK -> RuntimeError
    in the reference's host code)."""
    if rc != 0:
        msg = lib.dsv4_strerror(rc).decode()
        if rc == 6:
            msg += ": " + lib.dsv4_last_cuda_error().decode()
        raise RuntimeError(f"{what}: {msg} (status {rc})")
