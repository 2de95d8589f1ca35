"""GPU checks of the pieces around the attention kernel: FP8 gather/dequantise
(bit-exact), the KV store/quantise kernel (bit-exact), the split-KV combine and
the tensor-core descriptor self-test."""
import pytest
import torch

from oracle import sparse_mla as O
from util import max_rel_err

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    assert torch.cuda.is_available() and torch.cuda.get_device_capability(0)[0] == 10
    from deepseek_v4_kernel import cuda as K
    return K


@pytest.mark.parametrize("layout", [O.MODEL1, O.V32], ids=["model1", "v32"])
@pytest.mark.parametrize("method", [0, 1], ids=["packed_bf16", "via_fp32"])
def test_gather_dequant_bit_exact_all_bytes(K, layout, method):
    """Every e4m3 byte (NaN codes excepted) under a spread of scale bytes, and
    row selection through the page table arithmetic."""
    scale_bytes = [0, 1, 2, 100, 118, 125, 126, 127, 128, 133, 134, 135, 140, 200, 254]
    n = 64 * len(scale_bytes)
    body = torch.zeros(n, layout.nope_rope_bytes, dtype=torch.uint8)
    vals = torch.arange(256, dtype=torch.int16)
    vals = vals[(vals & 0x7f) != 0x7f].to(torch.uint8)                  # drop the two NaN codes
    gen = torch.Generator().manual_seed(0)
    for r in range(n):
        body[r, :layout.d_nope] = vals[torch.randint(0, vals.numel(), (layout.d_nope,), generator=gen)]
        body[r, :254] = vals                                             # every code in every row
    body[:, layout.d_nope:] = torch.randint(0, 256, (n, 128), generator=gen, dtype=torch.uint8)
    scales = torch.zeros(n, layout.scale_slots, dtype=torch.uint8)
    for i, s in enumerate(scale_bytes):
        scales[i * 64:(i + 1) * 64, :layout.scale_active] = s
    scales[:, 1:layout.scale_active] = torch.tensor(scale_bytes)[torch.randint(
        0, len(scale_bytes), (n, layout.scale_active - 1), generator=gen)].to(torch.uint8)
    nb = n // 64
    nrb = layout.nope_rope_bytes
    pages = torch.cat([body.view(nb, 64 * nrb), scales.view(nb, 64 * layout.scale_slots)], 1).contiguous()
    dense = O.pages_to_bf16(pages, 64, layout)
    idx = torch.cat([torch.randperm(n, generator=gen), torch.tensor([-1, n, n + 5])]).int()
    want = torch.zeros(idx.numel(), layout.d_qk, dtype=torch.bfloat16)
    ok = (idx >= 0) & (idx < n)
    want[ok] = dense[idx[ok].long()]
    kv4 = pages.cuda().view(nb, 64, 1, layout.bytes_per_token)
    got = K.gather_dequant(kv4, idx.cuda(), method).cpu()
    # RoPE bytes are arbitrary bit patterns (may be NaN): compare as integers
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))


@pytest.mark.parametrize("layout", [O.MODEL1, O.V32], ids=["model1", "v32"])
def test_kv_store_bit_exact(K, layout):
    gen = torch.Generator().manual_seed(2)
    n, nb = 300, 6
    mag = torch.logspace(-5, 3, n).unsqueeze(1)
    k_nope = (torch.randn(n, layout.d_nope, generator=gen) * mag).bfloat16()
    k_nope[5] = 0
    k_nope[6, :layout.quant_tile] = 448.0                     # amax exactly on a power-of-two edge
    k_nope[7, :layout.quant_tile] = 224.0
    k_rope = torch.randn(n, 64, generator=gen).bfloat16()
    slots = torch.randperm(nb * 64, generator=gen)[:n].long()
    slots[11] = -1
    want = torch.full((nb, layout.page_bytes(64)), 0xAB, dtype=torch.uint8)
    body, scales = O.quantize_rows(k_nope, k_rope, layout)
    O.store_rows(want, 64, layout, slots, body, scales)
    kv = torch.full((nb, layout.page_bytes(64)), 0xAB, dtype=torch.uint8, device="cuda")
    kv4 = kv.view(nb, 64, 1, layout.bytes_per_token)
    K.kv_store(k_nope.cuda(), k_rope.cuda(), slots.cuda(), kv4)
    assert torch.equal(kv.cpu(), want)
    # store -> gather returns the input rounded through FP8 with the tile scale
    back = K.gather_dequant(kv4, slots.clamp(min=0).int().cuda()).cpu()
    assert torch.equal(back[:, layout.d_nope:][slots >= 0], k_rope[slots >= 0])


@pytest.mark.parametrize("layout", [O.MODEL1, O.V32], ids=["model1", "v32"])
@pytest.mark.parametrize("loc_dtype", [torch.int32, torch.int64], ids=["loc32", "loc64"])
def test_kv_store_rows_writes_the_same_bytes(K, layout, loc_dtype):
    """The cache-writer form (one strided row per token, int32 / int64 slot mapping) must
    leave exactly the bytes of the oracle quantiser; a row that does not start on a 16-byte
    boundary is refused."""
    gen = torch.Generator().manual_seed(9)
    n, nb, page = 333, 3, 256
    d_qk = layout.d_nope + 64
    wide = (torch.randn(n, 1, d_qk + 40, generator=gen) * torch.logspace(-3, 2, n).view(n, 1, 1)).bfloat16()
    k = wide[:, :, 8:8 + d_qk]                                  # a view: row stride d_qk + 40, offset 16 B
    loc = torch.randperm(nb * page, generator=gen)[:n].to(loc_dtype)
    loc[17] = -1
    want = torch.full((nb, layout.page_bytes(page)), 0x5C, dtype=torch.uint8)
    body, scales = O.quantize_rows(k[:, 0, :layout.d_nope].contiguous(), k[:, 0, layout.d_nope:].contiguous(), layout)
    O.store_rows(want, page, layout, loc.long(), body, scales)
    kv = torch.full((nb, layout.page_bytes(page)), 0x5C, dtype=torch.uint8, device="cuda")
    kv4 = kv.view(nb, page, 1, layout.bytes_per_token)
    wide_d = wide.cuda()
    K.kv_store_rows(wide_d[:, :, 8:8 + d_qk], loc.cuda(), kv4)
    assert torch.equal(kv.cpu(), want)
    with pytest.raises(RuntimeError):
        K.kv_store_rows(wide_d[:, :, 4:4 + d_qk], loc.cuda(), kv4)      # rows start 8 bytes off a 16-byte line


@pytest.mark.parametrize("n_splits,h_q", [(2, 16), (5, 64), (128, 64), (256, 8)])
@pytest.mark.parametrize("with_sink", [False, True])
def test_combine_matches_oracle(K, n_splits, h_q, with_sink):
    gen = torch.Generator().manual_seed(n_splits)
    rows = 3
    o = torch.randn(n_splits, rows, h_q, 512, generator=gen)
    l = torch.randn(n_splits, rows, h_q, generator=gen) * 3
    l[torch.rand(n_splits, rows, h_q, generator=gen) < 0.2] = float("-inf")
    l[:, 1, 2] = float("-inf")                                 # a fully empty row/head
    sink = torch.randn(h_q, generator=gen) if with_sink else None
    out_ref, lse_ref = O.combine_splits(o, l, sink)
    out, lse = K.split_combine(o.cuda(), l.cuda(), None if sink is None else sink.cuda())
    torch.testing.assert_close(lse.cpu(), lse_ref, atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(out.cpu().float(), out_ref.float(), atol=1e-2, rtol=1e-2)
    assert (out.cpu()[1, 2] == 0).all()


@pytest.mark.parametrize("mode,n,k", [(0, 64, 64), (0, 64, 256), (0, 16, 128), (0, 32, 192),
                                      (1, 64, 64), (1, 64, 256), (1, 32, 128), (1, 16, 128)])
def test_umma_descriptor_selftest(K, mode, n, k):
    gen = torch.Generator().manual_seed(mode * 100 + n + k)
    a = torch.randn(128, k, generator=gen).bfloat16()
    b = torch.randn(n, k, generator=gen).bfloat16()
    want = a.float() @ b.float().t()
    if mode == 0:
        d, status = K.umma_selftest(0, a.cuda(), b.cuda())
    else:
        d, status = K.umma_selftest(1, a.t().contiguous().cuda(), b.t().contiguous().cuda())
    assert status == 0, "the MMA never signalled its barrier"
    torch.testing.assert_close(d.cpu(), want, atol=1e-3, rtol=1e-3)


def test_head_gather_gives_up_on_a_missing_peer(K):
    """The peer-memory all-gather waits for every rank's flag with a bound.  Here rank 0
    of a pretended two-rank group runs alone (the "peer" buffers are local memory and
    nobody ever sets the peer's flag): the kernel must copy its own shard, give up after
    its bounded wait, report that through the status word and leave the context usable."""
    import ctypes as C
    from deepseek_v4_kernel import _native as N
    dev = torch.device("cuda", 0)
    b, h_local, world = 2, 8, 2
    h_q = h_local * world
    out_local = torch.randn(b, 1, h_local, 512, device=dev).bfloat16()
    lse_local = torch.randn(b, h_local, 1, device=dev)
    gathered = [torch.zeros(b, 1, h_q, 512, dtype=torch.bfloat16, device=dev) for _ in range(world)]
    lse_g = [torch.zeros(b, h_q, 1, device=dev) for _ in range(world)]
    flags = [torch.zeros(world, dtype=torch.int32, device=dev) for _ in range(world)]
    counter = torch.zeros(1, dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    a = N.GatherArgs()
    a.world, a.rank, a.b, a.s_q, a.h_local, a.step = world, 0, b, 1, h_local, 1
    a.out_local, a.lse_local = out_local.data_ptr(), lse_local.data_ptr()
    for r in range(world):
        a.peer_out[r], a.peer_lse[r], a.peer_flags[r] = (gathered[r].data_ptr(), lse_g[r].data_ptr(),
                                                         flags[r].data_ptr())
    a.counter, a.status = counter.data_ptr(), status.data_ptr()
    N.check(N.lib.dsv4_gather_heads(C.byref(a), torch.cuda.current_stream().cuda_stream), "gather")
    torch.cuda.synchronize()
    assert status.item() == 2                      # 1 + the rank that never arrived
    assert flags[0][0].item() == 1 and flags[1][0].item() == 1 and flags[0][1].item() == 0
    for r in range(world):                         # the shard itself did land everywhere
        assert torch.equal(gathered[r][:, :, :h_local], out_local)
        assert torch.equal(lse_g[r][:, :h_local], lse_local)
    # the context is intact: a normal kernel still runs
    assert torch.equal(out_local + 0, out_local)


def test_head_gather_counter_survives_a_change_of_grid(K):
    """Two calls that share one counter but differ in batch size (hence in grid): the last
    CTA of each call must be recognised as such, so every call publishes its flag exactly
    once, after all of its stores.  One rank, its "peers" being local buffers."""
    import ctypes as C
    from deepseek_v4_kernel import _native as N
    dev = torch.device("cuda", 0)
    counter = torch.zeros(1, dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    flags = torch.zeros(1, dtype=torch.int32, device=dev)
    step = 0
    for b in (1, 12, 3, 64, 2):                      # 4, 48, 12, 64 (capped), 8 CTAs
        step += 1
        out_local = torch.randn(b, 1, 8, 512, device=dev).bfloat16()
        lse_local = torch.randn(b, 8, 1, device=dev)
        gathered = torch.zeros(b, 1, 8, 512, dtype=torch.bfloat16, device=dev)
        lse_g = torch.zeros(b, 8, 1, device=dev)
        a = N.GatherArgs()
        a.world, a.rank, a.b, a.s_q, a.h_local, a.step = 1, 0, b, 1, 8, step
        a.out_local, a.lse_local = out_local.data_ptr(), lse_local.data_ptr()
        a.peer_out[0], a.peer_lse[0], a.peer_flags[0] = (gathered.data_ptr(), lse_g.data_ptr(),
                                                         flags.data_ptr())
        a.counter, a.status = counter.data_ptr(), status.data_ptr()
        N.check(N.lib.dsv4_gather_heads(C.byref(a), torch.cuda.current_stream().cuda_stream), "gather")
        torch.cuda.synchronize()
        assert status.item() == 0 and flags.item() == step and counter.item() == 0
        assert torch.equal(gathered, out_local) and torch.equal(lse_g, lse_local)


@pytest.mark.parametrize("n_splits", [1, 2, 5, 16])
def test_decode_and_exchange_in_one_call_on_one_rank(K, n_splits):
    """dsv4_sparse_decode_gather with a group of one rank (its "peer" buffers are local):
    whatever the split plan, the gathered buffers must hold what the plain decode returns,
    the step flag must be published once, and the shared counter must be back at zero."""
    import ctypes as C
    import math
    import test_gpu_decode as T
    from deepseek_v4_kernel import _native as N
    dev = torch.device("cuda", 0)
    b, h = 5, 16
    q, pages, idx = T.fake_batch(b, h, 16, 700, seed=31, layout=O.V32)
    sm = 1.0 / math.sqrt(576)
    kv4 = pages.to(dev).view(pages.size(0), 64, 1, O.V32.bytes_per_token)
    sink = torch.randn(h, generator=torch.Generator().manual_seed(2)).to(dev)
    call = K.DecodeCall(q.to(dev), kv4, idx.to(dev), sm, attn_sink=sink, n_splits=n_splits)
    stream = torch.cuda.current_stream().cuda_stream
    call.decode(stream)
    want_out, want_lse = call.out.clone(), call.lse.clone()
    gathered = torch.zeros(b, 1, h, 512, dtype=torch.bfloat16, device=dev)
    lse_g = torch.zeros(b, h, 1, device=dev)
    flags = torch.zeros(1, dtype=torch.int32, device=dev)
    counter = torch.zeros(1, dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    a = N.GatherArgs()
    a.world, a.rank, a.b, a.s_q, a.h_local, a.step = 1, 0, b, 1, h, 7
    a.peer_out[0], a.peer_lse[0], a.peer_flags[0] = gathered.data_ptr(), lse_g.data_ptr(), flags.data_ptr()
    a.counter, a.status = counter.data_ptr(), status.data_ptr()
    N.check(N.lib.dsv4_sparse_decode_gather(C.byref(call.args), C.byref(a), stream), "decode_gather")
    torch.cuda.synchronize()
    assert K.device_status() == 0 and status.item() == 0
    assert flags.item() == 7 and counter.item() == 0
    assert torch.equal(gathered, want_out) and torch.equal(lse_g, want_lse)
