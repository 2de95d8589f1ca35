"""Parity of the CUDA prefill path with the CPU oracle and golden vectors.
Tolerances are the reference's own (tests/test_sparse_prefill.py:68-82):
cosine >= 0.999, out 5e-3, max_logits and lse 1e-2 on finite entries."""
import math

import pytest
import torch

from oracle import sparse_mla as O
from util import load_golden, max_rel_err

pytestmark = pytest.mark.gpu
IMPLS = [pytest.param(0, id="tcgen05"), pytest.param(2, id="simple")]


@pytest.fixture(scope="module")
def K():
    assert torch.cuda.is_available() and torch.cuda.get_device_capability(0)[0] == 10
    from deepseek_v4_kernel import cuda as K
    return K


def check(got, ref):
    from deepseek_v4_kernel import cuda as K
    assert K.device_status() == 0, "a bounded wait inside the kernel gave up"
    out, mx, lse = (t.cpu() for t in got)
    out_ref, mx_ref, lse_ref = ref
    cos = torch.nn.functional.cosine_similarity(out.float().flatten(), out_ref.float().flatten(), dim=0)
    assert cos >= 0.999
    torch.testing.assert_close(out.float(), out_ref.float(), atol=5e-3, rtol=5e-3)
    assert max_rel_err(out, out_ref) <= 2e-2
    for a, b in ((mx, mx_ref), (lse, lse_ref)):
        assert torch.equal(torch.isfinite(a), torch.isfinite(b))
        assert torch.equal(torch.isposinf(a), torch.isposinf(b))
        fin = torch.isfinite(b)
        torch.testing.assert_close(a[fin], b[fin], atol=1e-2, rtol=1e-2)


def batch(s_q, h_q, s_kv, topk, seed, d_qk=512, with_len=False, with_sink=False):
    gen = torch.Generator().manual_seed(seed)
    q = (torch.randn(s_q, h_q, d_qk, generator=gen) * 0.1).bfloat16()
    kv = (torch.randn(s_kv, d_qk, generator=gen) * 0.5).bfloat16()
    idx = torch.randint(-1, s_kv, (s_q, topk), generator=gen, dtype=torch.int32)
    sink = torch.randn(h_q, generator=gen) if with_sink else None
    tl = torch.randint(1, topk + 1, (s_q,), generator=gen, dtype=torch.int32) if with_len else None
    return q, kv, idx, sink, tl


@pytest.mark.parametrize("flags", IMPLS)
@pytest.mark.parametrize("name", ["prefill_h16_topk128", "prefill_h16_topk256_len_sink"])
def test_golden_vectors(K, name, flags):
    g = load_golden(name)
    c = lambda t: None if t is None else t.cuda()
    got = K.sparse_prefill_fwd(g["q"].cuda(), g["kv"].cuda(), g["indices"].cuda(), g["sm_scale"], 512,
                               c(g.get("attn_sink")), c(g.get("topk_length")), flags=flags)
    check(got, (g["out"], g["max_logits"], g["lse"]))


@pytest.mark.parametrize("flags", IMPLS)
@pytest.mark.parametrize("s_q", [1, 64, 1024])
@pytest.mark.parametrize("h_q", [64, 128])
@pytest.mark.parametrize("topk", [64, 256, 2048])
def test_reference_test_grid(K, s_q, h_q, topk, flags):
    """The reference's parametrisation (tests/test_sparse_prefill.py:44-82); the
    oracle is compared on the first <= 128 rows to bound its dense gather."""
    if flags == 2 and s_q * h_q * topk > 64 * 128 * 2048:
        pytest.skip("CUDA-core cross-check kernel: large shapes covered by the tensor-core path")
    s_kv = max(4096, topk * 4)
    q, kv, idx, _, _ = batch(s_q, h_q, s_kv, topk, seed=0)
    sm = 1 / math.sqrt(512)
    got = K.sparse_prefill_fwd(q.cuda(), kv.cuda(), idx.cuda().unsqueeze(1), sm, 512, None, None,
                               flags=flags)
    rows = min(s_q, 128)
    ref = O.sparse_prefill(q[:rows], kv, idx[:rows], sm)
    check(tuple(t[:rows] for t in got), ref)


@pytest.mark.parametrize("flags", IMPLS)
def test_topk_length_sink_and_lonely_rows(K, flags):
    q, kv, idx, sink, tl = batch(128, 64, 4096, 512, seed=1, with_len=True, with_sink=True)
    idx[5] = -1
    idx[6] = 4096 + 7                      # out of range is masked too
    tl[9] = 0
    sm = 1 / math.sqrt(512)
    ref = O.sparse_prefill(q, kv, idx, sm, 512, sink, tl)
    got = K.sparse_prefill_fwd(q.cuda(), kv.cuda().unsqueeze(1), idx.cuda(), sm, 512, sink.cuda(),
                               tl.cuda(), flags=flags)
    check(got, ref)
    out = got[0].cpu()
    assert (out[5] == 0).all() and (out[6] == 0).all() and (out[9] == 0).all()


@pytest.mark.parametrize("flags", IMPLS)
@pytest.mark.parametrize("layout", [O.MODEL1, O.V32], ids=["model1", "v32"])
def test_prefill_from_fp8_pages(K, layout, flags):
    gen = torch.Generator().manual_seed(8)
    s_kv, s_q, h_q, topk = 512, 96, 16, 160
    pages = O.build_pages(torch.randn(s_kv, layout.d_nope, generator=gen).bfloat16(),
                          torch.randn(s_kv, 64, generator=gen).bfloat16(), 64, layout)
    q = torch.randn(s_q, h_q, layout.d_qk, generator=gen).bfloat16()
    idx = torch.randint(-1, s_kv, (s_q, topk), generator=gen, dtype=torch.int32)
    sm = layout.d_qk ** -0.5
    ref = O.sparse_prefill_paged(q, pages, idx, sm, 64, layout)
    kv4 = pages.cuda().view(s_kv // 64, 64, 1, layout.bytes_per_token)
    got = K.sparse_prefill_fwd_fp8(q.cuda(), kv4, idx.cuda(), sm, flags=flags)
    check(got, ref)
    # and the flat BF16 entry on the dequantised rows gives the same answer (d_qk 512 or 576)
    dense = O.pages_to_bf16(pages, 64, layout)
    got2 = K.sparse_prefill_fwd(q.cuda(), dense.cuda(), idx.cuda(), sm, flags=flags)
    check(got2, ref)
