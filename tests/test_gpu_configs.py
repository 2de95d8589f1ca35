"""Parity at the shapes the benchmark numbers are quoted on, and on the attention
kernel's own conversion path.

Every case runs the CUDA path through the C ABI at the full size of the
configuration and compares with the CPU oracle on the gathered rows only
(`whole_arena=False`: the same arithmetic without dequantising the whole cache).
The caches are filled on the GPU by the store kernel, which is checked bit for
bit against the oracle's quantiser in test_gpu_parts.py.  Tolerances: lse 1e-3
(decode), 1e-2 (prefill max_logits / lse) as in the reference's own tests; out
max relative error <= 2e-2 and element-wise atol 5e-3 with rtol 2^-7.  The
reference's tests use rtol 5e-3 on inputs scaled down so that outputs stay well
below 1; the configurations here draw latents from N(0, 1), outputs reach 2..4,
where one BF16 unit in the last place is 0.0156 = 2^-7 relative, and two correct
fp32 results that straddle a rounding boundary differ by exactly that.
"""
import math

import pytest
import torch

import bench_workloads as W
from oracle import sparse_mla as O
from util import arena2d, max_rel_err

pytestmark = pytest.mark.gpu
DEV = "cuda"
OUT_RTOL = 2.0 ** -7          # one BF16 unit in the last place


@pytest.fixture(scope="module")
def K():
    assert torch.cuda.is_available() and torch.cuda.get_device_capability(0)[0] == 10
    from deepseek_v4_kernel import cuda as K
    return K


def check_decode(K, out, lse, out_ref, lse_ref):
    assert K.device_status() == 0, "a bounded wait inside the kernel gave up"
    out, lse = out.cpu(), lse.cpu().transpose(1, 2)
    torch.testing.assert_close(lse, lse_ref, atol=1e-3, rtol=1e-3)
    torch.testing.assert_close(out.float(), out_ref.float(), atol=5e-3, rtol=OUT_RTOL)
    assert max_rel_err(out, out_ref) <= 2e-2


def oracle_on_requests(wl, which, layout, reqs):
    """CPU oracle for the requests `reqs` of index set `which` (rows gathered, not the arena)."""
    pages = arena2d(wl.kv)
    idx = wl.indices[which].cpu()
    q = wl.q.cpu()
    r = torch.tensor(reqs)
    return O.sparse_decode(q[r], pages, idx[r], None, None, wl.sm_scale, W.PAGE, layout,
                           whole_arena=False)


def test_config2_as_written(K):
    """b 16, h_q 64, 32 768-token contexts behind a permuted page table, top-k 2048 without
    padding, the planned split count; every request is compared."""
    from deepseek_v4_kernel import ops
    wl = W.config2(torch.device(DEV), ops.kv_store, n_index_sets=2)
    assert wl.kv.numel() == 16 * 32768 * 644
    for which in (0, 1):
        out, lse, _, _ = ops.sparse_decode_fwd(wl.q, wl.kv, wl.indices[which], None, None, None,
                                               None, None, None, None, 512, wl.sm_scale)
        out_ref, lse_ref = oracle_on_requests(wl, which, O.V32, list(range(16)))
        check_decode(K, out, lse, out_ref, lse_ref)


def test_config2_properties_that_do_not_depend_on_size(K):
    """configs[1] at full size, checked through properties rather than against the oracle:
    (i) two runs return the same bits (no result depends on timing: the split combine and the
    cluster merge sum in a fixed order); (ii) an index list in another order names the same
    set, so the result moves by rounding only; (iii) every split plan (one split, clusters of
    two and four, eight partial sets through the combine kernel) gives the same result
    within the same bars."""
    from deepseek_v4_kernel import ops
    wl = W.config2(torch.device(DEV), ops.kv_store, n_index_sets=1)
    idx = wl.indices[0]

    def run(indices, n_splits=None):
        call = K.DecodeCall(wl.q, wl.kv, indices, wl.sm_scale, n_splits=n_splits)
        call.decode(torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        assert K.device_status() == 0
        return call.out.clone(), call.lse.clone()

    out0, lse0 = run(idx)
    out1, lse1 = run(idx)
    assert torch.equal(out0, out1) and torch.equal(lse0, lse1)
    gen = torch.Generator(device=DEV).manual_seed(5)
    perm = torch.randperm(idx.size(-1), device=DEV, generator=gen)
    out2, lse2 = run(idx[..., perm].contiguous())
    torch.testing.assert_close(lse2, lse0, atol=1e-3, rtol=1e-3)
    torch.testing.assert_close(out2.float(), out0.float(), atol=5e-3, rtol=OUT_RTOL)
    for n_splits in (1, 2, 4, 8):
        out3, lse3 = run(idx, n_splits)
        torch.testing.assert_close(lse3, lse0, atol=1e-3, rtol=1e-3)
        torch.testing.assert_close(out3.float(), out0.float(), atol=5e-3, rtol=OUT_RTOL)


@pytest.mark.parametrize("h_q", [16, 32])
def test_config2_as_one_tensor_parallel_shard(K, h_q):
    """configs[1] with the heads of one shard (16 of 64, and 32)."""
    from deepseek_v4_kernel import ops
    wl = W.config2(torch.device(DEV), ops.kv_store, b=16, h_q=h_q, ctx=8192, n_index_sets=1)
    out, lse, _, _ = ops.sparse_decode_fwd(wl.q, wl.kv, wl.indices[0], None, None, None, None,
                                           None, None, None, 512, wl.sm_scale)
    out_ref, lse_ref = oracle_on_requests(wl, 0, O.V32, list(range(16)))
    check_decode(K, out, lse, out_ref, lse_ref)


def test_target_shape_batch_64(K):
    """The north-star shape (b 64, 1.35 GB cache); six requests spread over the batch."""
    from deepseek_v4_kernel import ops
    wl = W.config2(torch.device(DEV), ops.kv_store, b=64, n_index_sets=1)
    out, lse, _, _ = ops.sparse_decode_fwd(wl.q, wl.kv, wl.indices[0], None, None, None, None,
                                           None, None, None, 512, wl.sm_scale)
    reqs = [0, 1, 17, 31, 46, 63]
    out_ref, lse_ref = oracle_on_requests(wl, 0, O.V32, reqs)
    check_decode(K, out[reqs], lse[reqs], out_ref, lse_ref)


def test_config3_rows_beyond_4_gib(K):
    """configs[2]: 128 requests, context lengths 4096..65536, half of every list in runs of 64
    consecutive positions, in a 4.6 GB cache: the pages of the compared requests lie below
    2^31, between 2^31 and 2^32, and beyond 2^32 bytes from the cache base.  Only the
    gathered rows are written (the rest of the cache is never read)."""
    from deepseek_v4_kernel import ops
    dev = torch.device(DEV)
    b, topk, h_q = 128, 2048, 64
    gen = W.generator(dev, 3)
    g_cpu = torch.Generator().manual_seed(1003)
    ctx = torch.randint(4096, 65537, (b,), generator=g_cpu).tolist()
    pages_needed = sum((c + W.PAGE - 1) // W.PAGE for c in ctx)
    num_blocks = 112000                                    # x 41 216 B = 4.62 GB
    assert pages_needed <= num_blocks
    kv = torch.empty((num_blocks, W.PAGE, 1, 644), dtype=torch.uint8, device=dev)
    table = torch.randperm(num_blocks, device=dev, generator=gen)
    idx = W._paged_indices(ctx, topk, table, gen, dev, clustered_frac=0.5)
    slots = idx.view(-1).long()
    n = slots.numel()
    k_nope = torch.randn((n, 512), device=dev, generator=gen).to(torch.bfloat16)
    k_rope = torch.randn((n, 64), device=dev, generator=gen).to(torch.bfloat16)
    ops.kv_store(k_nope, k_rope, slots, kv)
    q = torch.randn((b, 1, h_q, 576), device=dev, generator=gen).to(torch.bfloat16)
    sm = 576 ** -0.5
    out, lse, _, _ = ops.sparse_decode_fwd(q, kv, idx, None, None, None, None, None, None, None,
                                           512, sm)
    # pick requests by where their rows live
    page_bytes = W.PAGE * 644
    far = (idx.view(b, -1).long() // W.PAGE * page_bytes)
    lo, hi = far.min(dim=1).values.cpu(), far.max(dim=1).values.cpu()
    assert int(hi.max()) > 2 ** 32 and int(lo.min()) < 2 ** 31
    reqs = sorted({0, b - 1, int(hi.argmax()), int(lo.argmin()),
                   int(((hi > 2 ** 31) & (hi < 2 ** 32)).int().argmax())})
    # oracle input: the gathered rows copied (by torch indexing) into a small cache of their own
    for r in reqs:
        s = idx[r, 0].long()
        flat = kv.view(num_blocks, -1)
        pg, rw = s // W.PAGE, s % W.PAGE
        ar = torch.arange(640, device=dev)
        body = flat[pg.unsqueeze(1), (rw * 640).unsqueeze(1) + ar]
        sc = flat[pg.unsqueeze(1), (W.PAGE * 640 + rw * 4).unsqueeze(1) + torch.arange(4, device=dev)]
        small = torch.cat([body.view(topk // W.PAGE, W.PAGE * 640),
                           sc.view(topk // W.PAGE, W.PAGE * 4)], 1).cpu().contiguous()
        ridx = torch.arange(topk, dtype=torch.int32).view(1, 1, topk)
        out_ref, lse_ref = O.sparse_decode(q[r:r + 1].cpu(), small, ridx, None, None, sm, W.PAGE,
                                           O.V32, whole_arena=False)
        check_decode(K, out[r:r + 1], lse[r:r + 1], out_ref, lse_ref)


def test_config4_exactly(K):
    """b 1, h_q 64, 131 072-token context, top-k 2048 with 256 trailing -1, 128 forced splits
    of 16 entries merged by the combine kernel."""
    from deepseek_v4_kernel import ops
    wl = W.config4(torch.device(DEV), ops.kv_store)
    assert wl.force_splits == 128 and int((wl.indices[0] < 0).sum()) == 256
    out, lse, _, _ = K.sparse_decode_fwd(wl.q, wl.kv, wl.indices[0], None, None, None, None, None,
                                         None, None, 512, wl.sm_scale, n_splits=128)
    out_ref, lse_ref = oracle_on_requests(wl, 0, O.V32, [0])
    check_decode(K, out, lse, out_ref, lse_ref)


def check_prefill(K, got, ref):
    assert K.device_status() == 0
    out, mx, lse = (t.cpu() for t in got)
    out_ref, mx_ref, lse_ref = ref
    cos = torch.nn.functional.cosine_similarity(out.float().flatten(), out_ref.float().flatten(), dim=0)
    assert cos >= 0.999
    torch.testing.assert_close(out.float(), out_ref.float(), atol=5e-3, rtol=OUT_RTOL)
    assert max_rel_err(out, out_ref) <= 2e-2
    for a, b in ((mx, mx_ref), (lse, lse_ref)):
        assert torch.equal(torch.isfinite(a), torch.isfinite(b))
        fin = torch.isfinite(b)
        torch.testing.assert_close(a[fin], b[fin], atol=1e-2, rtol=1e-2)


@pytest.mark.parametrize("entry", ["fp8_pages", "bf16_workspace"])
def test_config5_sampled_rows(K, entry):
    """configs[4] at full size (8192 causal queries, h_q 64, top-k 2048, V32); the first rows,
    rows around the point where the lists fill up, and the last rows are compared."""
    from deepseek_v4_kernel import ops
    pw = W.config5(torch.device(DEV), ops.kv_store)
    if entry == "fp8_pages":
        got = ops.sparse_prefill_fwd_fp8(pw.q, pw.kv_pages, pw.indices, pw.sm_scale, 512)
        dense = O.pages_to_bf16(arena2d(pw.kv_pages), W.PAGE, O.V32)
    else:
        got = ops.sparse_prefill_fwd(pw.q, pw.kv_bf16, pw.indices, pw.sm_scale, 512)
        dense = pw.kv_bf16.cpu()
    rows = torch.tensor([0, 1, 2, 63, 127, 128, 1000, 2046, 2047, 2048, 2049, 5000, 8190, 8191])
    ref = O.sparse_prefill(pw.q.cpu()[rows], dense, pw.indices.cpu()[rows], pw.sm_scale)
    check_prefill(K, tuple(t[rows.to(DEV)] for t in got), ref)


@pytest.mark.parametrize("h_q,topk", [(64, 2048), (128, 256)])
def test_prefill_16384_queries(K, h_q, topk):
    """s_q = 16384, the size at which the serving framework switches to this kernel; 1024 rows
    are compared, as the reference's own test does (tests/test_sparse_prefill.py:44-82)."""
    s_kv = max(4096, topk * 4)
    gen = torch.Generator(device=DEV).manual_seed(0)
    q = (torch.randn(16384, h_q, 512, device=DEV, generator=gen) * 0.1).bfloat16()
    kv = (torch.randn(s_kv, 512, device=DEV, generator=gen) * 0.5).bfloat16()
    idx = torch.randint(-1, s_kv, (16384, topk), device=DEV, generator=gen, dtype=torch.int32)
    sm = 1 / math.sqrt(512)
    got = K.sparse_prefill_fwd(q, kv, idx.unsqueeze(1), sm, 512, None, None)
    ref = O.sparse_prefill(q[:1024].cpu(), kv.cpu(), idx[:1024].cpu(), sm)
    check_prefill(K, tuple(t[:1024] for t in got), ref)


@pytest.mark.parametrize("layout", [O.MODEL1, O.V32], ids=["model1", "v32"])
@pytest.mark.parametrize("page_block", [256, 48])
def test_other_page_sizes(K, layout, page_block):
    """Pages of 256 tokens (the size the reference's launch recipe uses) and a page size that
    is not a power of two (division instead of shift in the row address)."""
    gen = torch.Generator().manual_seed(page_block)
    nb = 6
    n = nb * page_block
    pages = O.build_pages(torch.randn(n, layout.d_nope, generator=gen).bfloat16(),
                          torch.randn(n, 64, generator=gen).bfloat16(), page_block, layout)
    q = torch.randn(3, 1, 64, layout.d_qk, generator=gen).bfloat16()
    idx = torch.randint(-1, n, (3, 1, 700), generator=gen, dtype=torch.int32)
    tk = torch.tensor([700, 129, 5], dtype=torch.int32)
    sm = layout.d_qk ** -0.5
    kv4 = pages.cuda().view(nb, page_block, 1, layout.bytes_per_token)
    for n_splits in (1, 2, 5):
        out, lse, _, _ = K.sparse_decode_fwd(q.cuda(), kv4, idx.cuda(), tk.cuda(), None, None,
                                             None, None, None, None, 512, sm, n_splits=n_splits)
        out_ref, lse_ref = O.sparse_decode(q, pages, idx, tk, None, sm, page_block, layout)
        check_decode(K, out, lse, out_ref, lse_ref)
    dense = O.pages_to_bf16(pages, page_block, layout)
    pidx = idx[:, 0]
    got = K.sparse_prefill_fwd_fp8(q[:, 0].cuda(), kv4, pidx.cuda(), sm)
    check_prefill(K, got, O.sparse_prefill(q[:, 0], dense, pidx, sm))


# 240 is the largest scale byte kept: beyond it 448 * 2^(s-127) overflows BF16 and 0 * inf would
# turn the logit into NaN.
SCALE_BYTES = [0, 1, 2, 100, 118, 125, 126, 127, 128, 133, 134, 135, 140, 200, 240]


@pytest.mark.parametrize("layout", [O.MODEL1, O.V32], ids=["model1", "v32"])
@pytest.mark.parametrize("h_q", [16, 64])
def test_single_entry_lists_return_the_value_row_exactly(K, layout, h_q):
    """With a one-entry list the softmax weight is exactly 1, so `out` must equal the BF16 V
    row (first 512 dequantised columns) exactly (as values: a sum of products cannot keep the
    sign of a zero, so -0 comes back as +0): this checks the attention kernel's own
    gather, FP8 x UE8M0 -> BF16 conversion and swizzled shared-memory staging, for every
    e4m3 code under scale bytes that include 0 and values above 134 (where one packed
    multiply does not cover the range).  Scales are kept where the product stays finite and
    normal in fp32 accumulation of a single term."""
    vals = torch.arange(256, dtype=torch.int16)
    vals = vals[(vals & 0x7f) != 0x7f].to(torch.uint8)                  # no NaN codes
    gen = torch.Generator().manual_seed(11)
    n = 64 * len(SCALE_BYTES)
    body = torch.zeros(n, layout.nope_rope_bytes, dtype=torch.uint8)
    for r in range(n):
        body[r, :layout.d_nope] = vals[torch.randint(0, vals.numel(), (layout.d_nope,), generator=gen)]
        off = (r * 37) % (layout.d_nope - 254)
        body[r, off:off + 254] = vals                                    # every code in every row
    rope = (torch.randn(n, 64, generator=gen)).bfloat16()
    body[:, layout.d_nope:] = rope.view(torch.uint8).view(n, 128)
    scales = torch.zeros(n, layout.scale_slots, dtype=torch.uint8)
    sb = torch.tensor(SCALE_BYTES, dtype=torch.uint8)
    for i in range(len(SCALE_BYTES)):
        scales[i * 64:(i + 1) * 64, 0] = sb[i]
    scales[:, 1:layout.scale_active] = sb[torch.randint(0, len(SCALE_BYTES),
                                                       (n, layout.scale_active - 1), generator=gen)]
    nb = n // 64
    nrb = layout.nope_rope_bytes
    pages = torch.cat([body.view(nb, 64 * nrb), scales.view(nb, 64 * layout.scale_slots)], 1).contiguous()
    dense = O.pages_to_bf16(pages, 64, layout)
    order = torch.randperm(n, generator=gen)
    idx = torch.full((n, 1, 64), -1, dtype=torch.int32)
    idx[:, 0, 0] = order.int()
    tk = torch.ones(n, dtype=torch.int32)
    # q = 0: every logit is 0 whatever the row holds, so no overflow can occur in Q.K^T
    q = torch.zeros(n, 1, h_q, layout.d_qk, dtype=torch.bfloat16)
    kv4 = pages.cuda().view(nb, 64, 1, layout.bytes_per_token)
    out, lse, _, _ = K.sparse_decode_fwd(q.cuda(), kv4, idx.cuda(), tk.cuda(), None, None, None,
                                         None, None, None, 512, 1.0)
    assert K.device_status() == 0
    want = dense[order][:, :512]
    got = out.cpu()[:, 0]                                                # [n, h_q, 512]
    first_scale = sb[order // 64]                                        # scale byte of tile 0 per request
    for h in (0, h_q // 2, h_q - 1):
        bad = (got[:, h].float() != want.float()).any(dim=1)
        assert not bad.any(), (f"head {h}: {int(bad.sum())} rows differ; first-tile scale bytes "
                               f"of those rows: {sorted(set(first_scale[bad].tolist()))}")
    assert torch.equal(lse.cpu(), torch.zeros_like(lse.cpu()))
