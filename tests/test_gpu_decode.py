"""Parity of the CUDA decode path (through the C ABI) with the CPU oracle and
the reference's golden vectors.  Tolerances: out atol = rtol = 5e-3 and lse
1e-3 absolute (the reference's own test bars, tests/test_sparse_decode.py:47-49),
which are tighter than the acceptance bar of 2e-2 max relative error."""
import math

import pytest
import torch

from oracle import sparse_mla as O
from util import arena2d, load_golden, max_rel_err

pytestmark = pytest.mark.gpu

SIMPLE = 2          # DSV4_FLAG_IMPL_SIMPLE
MASK_INVALID = 1
IMPLS = [pytest.param(0, id="tcgen05"), pytest.param(SIMPLE, id="simple")]


@pytest.fixture(scope="module")
def cuda_mod():
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    assert torch.cuda.get_device_capability(0)[0] == 10, "sm_100 required"
    from deepseek_v4_kernel import cuda as K
    return K


def check(out, lse, out_ref, lse_ref):
    """lse arrives as [b, h_q, s_q]; the oracle returns [b, s_q, h_q]."""
    from deepseek_v4_kernel import cuda as K
    assert K.device_status() == 0, "a bounded wait inside the kernel gave up"
    out, lse = out.cpu(), lse.cpu().transpose(1, 2)
    torch.testing.assert_close(lse, lse_ref, atol=1e-3, rtol=1e-3)
    torch.testing.assert_close(out.float(), out_ref.float(), atol=5e-3, rtol=5e-3)
    assert max_rel_err(out, out_ref) <= 2e-2


def run(K, q, pages2d, idx, sm, tk=None, sink=None, flags=0, n_splits=None, layout=O.MODEL1,
        page_block=64, **extra):
    dev = "cuda"
    kv4 = pages2d.to(dev).view(pages2d.size(0), page_block, 1, layout.bytes_per_token)
    g = lambda t: None if t is None else t.to(dev)
    out, lse, _, _ = K.sparse_decode_fwd(g(q), kv4, g(idx), g(tk), g(sink), None, None,
                                         extra.get("extra_kv"), g(extra.get("extra_indices")),
                                         g(extra.get("extra_topk_length")), 512, sm,
                                         n_splits=n_splits, flags=flags)
    return out, lse


@pytest.mark.parametrize("flags", IMPLS)
@pytest.mark.parametrize("name", ["decode_h64_topk64", "decode_h16_topk256", "decode_h16_topk2048",
                                  "decode_h16_topk512_len", "decode_h16_topk128_sink_len0"])
def test_golden_vectors(cuda_mod, name, flags):
    g = load_golden(name)
    out, lse = run(cuda_mod, g["q"], g["kv_pages"], g["indices"], g["sm_scale"],
                   g.get("topk_length"), g.get("attn_sink"), flags)
    check(out, lse, g["out"], g["lse"])


def fake_batch(b, h_q, num_blocks, topk, seed, layout=O.MODEL1, q_std=0.1, with_neg=True):
    """Seeded batch with the value distributions of the reference's fake batch
    (q ~ 0.1 N, latent ~ 0.5 N cast straight to e4m3 with random scale exponents
    125..128, RoPE ~ 0.05 N, indices uniform with replacement including -1)."""
    gen = torch.Generator().manual_seed(seed)
    n = num_blocks * 64
    q = (torch.randn(b, 1, h_q, layout.d_qk, generator=gen) * q_std).bfloat16()
    fp8 = (torch.randn(n, layout.d_nope, generator=gen) * 0.5).to(torch.float8_e4m3fn).view(torch.uint8)
    rope = (torch.randn(n, 64, generator=gen) * 0.05).bfloat16().view(torch.uint8).view(n, 128)
    scales = torch.zeros(n, layout.scale_slots, dtype=torch.uint8)
    scales[:, :layout.scale_active] = (125 + torch.randint(0, 4, (n, layout.scale_active), generator=gen)).to(torch.uint8)
    nrb = layout.nope_rope_bytes
    pages = torch.cat([torch.cat([fp8, rope], 1).view(num_blocks, 64 * nrb),
                       scales.view(num_blocks, 64 * layout.scale_slots)], 1).contiguous()
    lo = -1 if with_neg else 0
    idx = torch.randint(lo, n, (b, 1, topk), generator=gen, dtype=torch.int32)
    return q, pages, idx


@pytest.mark.parametrize("flags", IMPLS)
@pytest.mark.parametrize("h_q", [64, 128])
@pytest.mark.parametrize("topk", [64, 256, 2048])
def test_reference_test_grid(cuda_mod, h_q, topk, flags):
    """The reference's own parametrisation (tests/test_sparse_decode.py:27-49)."""
    q, pages, idx = fake_batch(2, h_q, 8, topk, seed=0)
    sm = 1 / math.sqrt(512)
    out_ref, lse_ref = O.sparse_decode(q, pages, idx, None, None, sm, 64)
    out, lse = run(cuda_mod, q, pages, idx, sm, flags=flags)
    check(out, lse, out_ref, lse_ref)


@pytest.mark.parametrize("flags", IMPLS)
@pytest.mark.parametrize("layout", [O.MODEL1, O.V32], ids=["model1", "v32"])
@pytest.mark.parametrize("n_splits", [1, 2, 3, 7, 16, 128])
def test_forced_split_counts_agree(cuda_mod, layout, n_splits, flags):
    q, pages, idx = fake_batch(2, 16, 8, 1000, seed=3, layout=layout)
    tk = torch.tensor([1000, 333], dtype=torch.int32)
    sink = torch.randn(16, generator=torch.Generator().manual_seed(1))
    sm = layout.d_qk ** -0.5
    out_ref, lse_ref = O.sparse_decode(q, pages, idx, tk, sink, sm, 64, layout)
    out, lse = run(cuda_mod, q, pages, idx, sm, tk, sink, flags, n_splits=n_splits, layout=layout)
    check(out, lse, out_ref, lse_ref)


@pytest.mark.parametrize("flags", IMPLS)
def test_config1_shape_v32(cuda_mod, flags):
    """b=1, h_q=16, 4096 tokens, top-k 128 with 8 trailing -1, quantised N(0,1) latents."""
    gen = torch.Generator().manual_seed(0)
    pages = O.build_pages(torch.randn(4096, 512, generator=gen).bfloat16(),
                          torch.randn(4096, 64, generator=gen).bfloat16(), 64, O.V32)
    q = torch.randn(1, 1, 16, 576, generator=gen).bfloat16()
    idx = torch.randperm(4096, generator=gen)[:128].int().view(1, 1, 128)
    idx[..., -8:] = -1
    sm = 576 ** -0.5
    out_ref, lse_ref = O.sparse_decode(q, pages, idx, None, None, sm, 64, O.V32)
    out, lse = run(cuda_mod, q, pages, idx, sm, flags=flags, layout=O.V32)
    check(out, lse, out_ref, lse_ref)


@pytest.mark.parametrize("flags", IMPLS)
def test_edge_cases(cuda_mod, flags):
    q, pages, idx = fake_batch(3, 16, 4, 200, seed=9)
    sm = 1 / math.sqrt(512)
    idx[0] = -1                                  # a request of only -1: all zero rows
    idx[1, 0, 100:] = 10 ** 6                    # out of range behaves like -1
    tk = torch.tensor([200, 150, 0], dtype=torch.int32)     # length 0 is raised to 1
    out_ref, lse_ref = O.sparse_decode(q, pages, idx, tk, None, sm, 64)
    out, lse = run(cuda_mod, q, pages, idx, sm, tk, None, flags)
    check(out, lse, out_ref, lse_ref)
    assert (out[0] == 0).all()
    # FlashMLA semantics on request: -1 masked; an all-masked request gives out 0, lse -inf
    out_ref, lse_ref = O.sparse_decode(q, pages, idx, tk, None, sm, 64, mask_invalid=True)
    out, lse = run(cuda_mod, q, pages, idx, sm, tk, None, flags | MASK_INVALID)
    assert torch.isneginf(lse[0]).all() and torch.isneginf(lse_ref[0]).all()
    check(out[1:], lse[1:], out_ref[1:], lse_ref[1:])
    assert (out[0] == 0).all()


@pytest.mark.parametrize("flags", IMPLS)
@pytest.mark.parametrize("with_sink", [False, True])
def test_zero_length_attends_to_nothing_on_request(cuda_mod, flags, with_sink):
    """DSV4_FLAG_ZERO_LENGTH_EMPTY: a topk_length below one gives out 0 and lse = sink or
    -inf, as the reference's CUDA kernel does (csrc/sm120/decode/sparse_decode_kernel.cuh:
    373-375, 527-529); the other requests of the batch are unaffected."""
    ZERO_LENGTH_EMPTY = 8
    q, pages, idx = fake_batch(3, 16, 4, 200, seed=12)
    sm = 1 / math.sqrt(512)
    tk = torch.tensor([0, 150, -3], dtype=torch.int32)
    sink = torch.randn(16, generator=torch.Generator().manual_seed(3)) if with_sink else None
    out_ref, lse_ref = O.sparse_decode(q, pages, idx, tk, sink, sm, 64)
    for n_splits in (1, 2, 3):
        out, lse = run(cuda_mod, q, pages, idx, sm, tk, sink, flags | ZERO_LENGTH_EMPTY,
                       n_splits=n_splits)
        check(out[1:2], lse[1:2], out_ref[1:2], lse_ref[1:2])
        out, lse = out.cpu(), lse.cpu()
        for r in (0, 2):
            assert (out[r] == 0).all()
            if with_sink:
                torch.testing.assert_close(lse[r, :, 0], sink)
            else:
                assert torch.isneginf(lse[r]).all()


@pytest.mark.parametrize("flags", IMPLS)
def test_multi_query_tokens_and_padded_page_stride(cuda_mod, flags):
    """s_q = 3 (the reference rejects s_q > 1) and a cache whose pages are padded."""
    K = cuda_mod
    gen = torch.Generator().manual_seed(4)
    q, pages, _ = fake_batch(2, 16, 6, 64, seed=4)
    q = (torch.randn(2, 3, 16, 512, generator=gen) * 0.1).bfloat16()
    idx = torch.randint(-1, 6 * 64, (2, 3, 320), generator=gen, dtype=torch.int32)
    tk = torch.tensor([320, 77], dtype=torch.int32)
    sm = 1 / math.sqrt(512)
    out_ref, lse_ref = O.sparse_decode(q, pages, idx, tk, None, sm, 64)
    stride = 64 * 584 + 256
    arena = torch.zeros(6, stride, dtype=torch.uint8, device="cuda")
    arena[:, : 64 * 584] = pages.cuda()
    kv4 = torch.as_strided(arena, (6, 64, 1, 584), (stride, 584, 584, 1))
    out, lse, _, _ = K.sparse_decode_fwd(q.cuda(), kv4, idx.cuda(), tk.cuda(), None, None, None,
                                         None, None, None, 512, sm, flags=flags)
    check(out, lse, out_ref, lse_ref)


@pytest.mark.parametrize("flags", IMPLS)
@pytest.mark.parametrize("n_splits", [1, 4])
def test_extra_kv(cuda_mod, flags, n_splits):
    q, pages, idx = fake_batch(2, 16, 4, 300, seed=6)
    _, xpages, xidx = fake_batch(2, 16, 2, 70, seed=7)
    tk = torch.tensor([300, 128], dtype=torch.int32)
    xtk = torch.tensor([70, 5], dtype=torch.int32)
    sm = 1 / math.sqrt(512)
    out_ref, lse_ref = O.sparse_decode(q, pages, idx, tk, None, sm, 64, extra_kv_pages=xpages,
                                       extra_indices=xidx, extra_topk_length=xtk)
    xkv4 = xpages.cuda().view(2, 64, 1, 584)
    out, lse = run(cuda_mod, q, pages, idx, sm, tk, None, flags, n_splits=n_splits,
                   extra_kv=xkv4, extra_indices=xidx, extra_topk_length=xtk)
    check(out, lse, out_ref, lse_ref)


def test_plan_is_used_and_outputs_have_reference_shapes(cuda_mod):
    q, pages, idx = fake_batch(2, 64, 8, 2048, seed=0)
    kv4 = pages.cuda().view(8, 64, 1, 584)
    out, lse, meta, splits = cuda_mod.sparse_decode_fwd(q.cuda(), kv4, idx.cuda(), None, None, None,
                                                        None, None, None, None, 512, 0.044)
    assert out.shape == (2, 1, 64, 512) and out.dtype == torch.bfloat16
    assert lse.shape == (2, 64, 1) and lse.dtype == torch.float32 and lse.is_contiguous()
    assert meta.dtype == torch.int32 and meta.shape == (1, 8) and splits.shape == (3,)
    with pytest.raises(RuntimeError):
        cuda_mod.sparse_decode_fwd(q.cuda(), kv4.view(8, 64, 1, 584)[..., :580], idx.cuda(), None, None,
                                   None, None, None, None, None, 512, 0.044)


@pytest.mark.parametrize("layout", [O.MODEL1, O.V32], ids=["model1", "v32"])
@pytest.mark.parametrize("n_splits", [2, 4])
def test_cluster_merge_with_empty_and_ragged_splits(cuda_mod, layout, n_splits):
    """Two and four splits are merged inside one thread-block cluster (no combine
    launch).  Lengths are chosen so that some CTAs of a cluster own no tile at all
    (they still take part in the merge), some a ragged one; with a sink."""
    q, pages, idx = fake_batch(5, 64, 8, 600, seed=77, layout=layout)
    tk = torch.tensor([1, 17, 40, 333, 600], dtype=torch.int32)
    sink = torch.randn(64, generator=torch.Generator().manual_seed(5))
    sm = 1.0 / math.sqrt(layout.d_qk)
    out, lse = run(cuda_mod, q, pages, idx, sm, tk, sink, 0, n_splits, layout)
    out_ref, lse_ref = O.sparse_decode(q, pages, idx, tk, sink, sm, 64, layout)
    check(out, lse, out_ref, lse_ref)


def test_grouped_cluster_merge_feeds_the_combine():
    """DSV4_CLUSTER=group merges the splits in groups of 4 and combines the groups
    (a measurement configuration; the variable is read once per process, hence the
    child process).  8 and 16 splits, one request shorter than a group."""
    import os
    import subprocess
    import sys
    code = r'''
import math, sys, torch
sys.path[:0] = [%r, %r]
from oracle import sparse_mla as O
import test_gpu_decode as T
from deepseek_v4_kernel import cuda as K
q, pages, idx = T.fake_batch(3, 64, 16, 1024, seed=91, layout=O.V32)
tk = torch.tensor([1024, 700, 30], dtype=torch.int32)
sm = 1.0 / math.sqrt(576)
ref = O.sparse_decode(q, pages, idx, tk, None, sm, 64, O.V32)
for n in (8, 16):
    out, lse = T.run(K, q, pages, idx, sm, tk, None, 0, n, O.V32)
    T.check(out, lse, *ref)
print("ok")
''' % (os.path.dirname(os.path.abspath(__file__)),
       os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))),
                    "deepseek-v4-flash-sm120_b200"))
    env = dict(os.environ, DSV4_CLUSTER="group")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env["PYTHONPATH"] = root + os.pathsep + env.get("PYTHONPATH", "")
    res = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True,
                         timeout=240)
    assert res.returncode == 0 and "ok" in res.stdout, res.stdout + res.stderr
