"""The allocation-free decode entry point (dsv4_sparse_decode_noalloc).

Some callers of this library cannot allocate device memory at the moment they
call it: a serving loop whose step is being captured into a CUDA graph, code
running inside another runtime's "no allocation" region, or a small host
program that links the C library without torch and has no allocator.  For them
the split-KV scratch sits in a fixed array inside the library.  This test calls
that entry point through the C ABI twice in a row (different inputs and split
counts, so the second call finds the first call's leftovers in the shared
scratch) and checks both results against the ordinary entry point.  It is
collected last so that a failure here cannot hide any other test.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _decode_both_ways(K, N, q, kv4, idx, sm_scale, n_splits):
    call = K.DecodeCall(q, kv4, idx, sm_scale, n_splits=n_splits)
    stream = torch.cuda.current_stream().cuda_stream
    call.decode(stream)                                   # existing entry point
    ref_out, ref_lse = call.out.clone(), call.lse.clone()
    call.out.zero_()
    call.lse.zero_()
    args = call.args
    keep = (args.o_accum, args.lse_accum)
    args.o_accum, args.lse_accum = None, None             # the new entry point brings its own scratch
    before = torch.cuda.memory_allocated()
    rc = N.lib.dsv4_sparse_decode_noalloc(C.byref(args), stream)
    assert rc == 0, N.lib.dsv4_strerror(rc).decode()
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before
    # torch's counter only sees torch's own allocator; the driver's free-memory figure would
    # also show a cudaMalloc made inside the library.  It is compared from the second call
    # on (the first call on a device may load the module and resolve the array's address).
    free_now = torch.cuda.mem_get_info()[0]
    rc = N.lib.dsv4_sparse_decode_noalloc(C.byref(args), stream)
    assert rc == 0, N.lib.dsv4_strerror(rc).decode()
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_now
    args.o_accum, args.lse_accum = keep
    assert K.device_status() == 0
    torch.testing.assert_close(call.out.float(), ref_out.float(), atol=5e-3, rtol=5e-3)
    torch.testing.assert_close(call.lse, ref_lse, atol=1e-3, rtol=1e-3)
    return call


def test_noalloc_decode_matches_regular_entry_twice():
    assert torch.cuda.is_available() and torch.cuda.get_device_capability(0)[0] == 10
    from deepseek_v4_kernel import _native as N
    from deepseek_v4_kernel import cuda as K
    from deepseek_v4_kernel import ops
    import bench_workloads as W

    dev = torch.device("cuda", 0)
    wl = W.decode_workload("noalloc", b=4, h_q=64, topk=1024, ctx_lens=[4096] * 4, layout="V32",
                           device=dev, quantize=ops.kv_store, seed=5, n_index_sets=2, pad_tail=16)
    _decode_both_ways(K, N, wl.q, wl.kv, wl.indices[0], wl.sm_scale, n_splits=8)
    # second call: other indices, other split count, scratch still holds call one's partials
    _decode_both_ways(K, N, wl.q, wl.kv, wl.indices[1], wl.sm_scale, n_splits=3)
    # four splits are merged inside a thread-block cluster: no partials reach the scratch
    _decode_both_ways(K, N, wl.q, wl.kv, wl.indices[1], wl.sm_scale, n_splits=4)
    # unsplit requests need no scratch and pass straight through
    _decode_both_ways(K, N, wl.q, wl.kv, wl.indices[0], wl.sm_scale, n_splits=1)


def test_noalloc_rejects_oversized_requests():
    from deepseek_v4_kernel import _native as N
    a = N.DecodeArgs()
    a.b, a.s_q, a.h_q, a.n_splits = 64, 1, 64, 8           # 64*64*8*512 floats > the built-in scratch
    rc = N.lib.dsv4_sparse_decode_noalloc(C.byref(a), None)
    assert rc == 9 and b"scratch" in N.lib.dsv4_strerror(rc)
    assert N.lib.dsv4_sparse_decode_noalloc(None, None) == 1
    # the limit counts the partial sets that reach the scratch: two splits of the same batch
    # are merged on chip, leave none, and must get past the size check (to the null-pointer
    # check, since this argument block names no tensors)
    a.n_splits, a.kv_format, a.d_qk = 2, N.KV_V32, 576
    assert N.lib.dsv4_sparse_decode_noalloc(C.byref(a), None) == 1
