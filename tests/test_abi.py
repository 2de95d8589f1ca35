"""The C-ABI library loads on a machine without a GPU, exports every symbol the
header declares, and rejects bad arguments with status codes (no kernel runs)."""
import ctypes as C
import os
import re

from deepseek_v4_kernel import _native as N

HEADER = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include",
                      "dsv4_b200.h")


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(dsv4_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound():
    names = declared_symbols()
    assert len(names) >= 10
    raw = C.CDLL(N.LIB_PATH)
    for n in names:
        assert hasattr(raw, n), f"{n} declared in the header but not exported"
        assert n in N.SYMBOLS, f"{n} has no ctypes prototype"
    assert sorted(N.SYMBOLS) == names


def test_abi_version_and_error_text():
    assert N.lib.dsv4_abi_version() == N.ABI_VERSION
    for code in range(0, 9):
        assert N.lib.dsv4_strerror(code).decode()
    assert b"unknown" in N.lib.dsv4_strerror(99)


def test_struct_layout_matches_the_header():
    # 16 x 4-byte scalars, 12 pointers, 15 x int64
    assert C.sizeof(N.DecodeArgs) == 16 * 4 + 12 * 8 + 15 * 8
    assert C.sizeof(N.CombineArgs) == 4 * 4 + 5 * 8 + 6 * 8
    assert C.sizeof(N.PrefillArgs) == 12 * 4 + 8 * 8 + 8 * 8
    assert C.sizeof(N.StoreArgs) == 4 * 4 + 4 * 8 + 3 * 8
    assert C.sizeof(N.StoreRowsArgs) == 4 * 4 + 3 * 8 + 2 * 8 + 2 * 4
    assert N.DecodeArgs.q.offset == 64 and N.PrefillArgs.q.offset == 48


def test_null_and_shape_errors_without_a_gpu():
    lib = N.lib
    assert lib.dsv4_sparse_decode(None, None) == 1
    a = N.DecodeArgs()
    assert lib.dsv4_sparse_decode(C.byref(a), None) == 1          # null tensors
    buf = (C.c_char * 4096)()
    p = C.addressof(buf)
    p16 = (p + 15) & ~15
    a.q = a.kv = a.indices = a.out = a.lse = p16
    a.b, a.s_q, a.h_q, a.d_qk, a.d_v, a.topk = 1, 1, 16, 512, 512, 0
    a.num_blocks, a.page_block_size, a.n_splits = 1, 64, 1
    assert lib.dsv4_sparse_decode(C.byref(a), None) == 2          # topk < 1
    a.topk, a.kv_format, a.stride_kv_block = 64, N.KV_MODEL1, 64 * 584
    a.d_qk = 576
    assert lib.dsv4_sparse_decode(C.byref(a), None) == 3          # layout mismatch
    a.d_qk, a.stride_kv_block = 512, 64 * 584 - 16
    assert lib.dsv4_sparse_decode(C.byref(a), None) == 3          # page too short
    a.stride_kv_block = 64 * 584 + 8
    assert lib.dsv4_sparse_decode(C.byref(a), None) == 4          # stride not 16-byte multiple
    a.stride_kv_block = 64 * 584
    a.q = p16 + 2
    assert lib.dsv4_sparse_decode(C.byref(a), None) == 4          # misaligned q
    a.q, a.n_splits = p16, 3                                        # (2 and 4 are merged on chip: no scratch)
    assert lib.dsv4_sparse_decode(C.byref(a), None) == 7          # scratch missing
    c = N.CombineArgs()
    assert lib.dsv4_split_combine(C.byref(c), None) == 1
    s = N.StoreArgs()
    assert lib.dsv4_kv_store(C.byref(s), None) == 1
    assert lib.dsv4_kv_store_rows(C.byref(N.StoreRowsArgs()), None) == 1
    assert lib.dsv4_gather_dequant(None, 0, 1, 1, 64, None, 0, None, 0, None) == 1
    assert lib.dsv4_umma_selftest(0, 64, 64, None, None, None, None, None) == 1


def test_split_plan_is_a_pure_function_of_shapes():
    plan = N.lib.dsv4_plan_splits
    assert plan(16, 1, 64, 2048, 0, 148) == 8          # 128 CTAs x 2 tiles
    assert plan(64, 1, 64, 2048, 0, 148) == 2          # 128 CTAs x 8 tiles
    assert plan(1, 1, 64, 2048, 0, 148) == 16          # never finer than one tile per split
    assert plan(256, 1, 64, 2048, 0, 148) == 1         # the batch alone fills the GPU
    assert plan(2, 1, 64, 64, 0, 148) == 1             # a single tile cannot be split
    assert plan(16, 1, 128, 2048, 0, 148) == plan(32, 1, 64, 2048, 0, 148)
    for args in [(3, 1, 16, 512, 0, 148), (5, 2, 64, 1024, 128, 132)]:
        s = plan(*args)
        assert 1 <= s <= 128 and s == plan(*args)
    assert plan(0, 1, 64, 2048, 0, 148) == 1           # degenerate shapes never fail
