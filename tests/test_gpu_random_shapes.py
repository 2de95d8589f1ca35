"""Seeded random shapes: the tensor-core kernels against the CUDA-core cross-check kernels on
the same GPU (both through the C ABI).  The fixed-shape tests compare with the CPU oracle;
this one walks the corners between them: head counts that fill 16 / 32 / 64-head instantiations
only partly, list lengths around the 128-entry tile, forced split counts (cluster merges with
empty and ragged splits, combine kernel), lengths, sinks and the masking flags, both layouts.
Bars as in the other tests: lse 1e-3 (decode) / 1e-2 (prefill), out atol 5e-3 with rtol 2^-7."""
import math
import random

import pytest
import torch

from oracle import sparse_mla as O
import test_gpu_decode as D
import test_gpu_prefill as P

pytestmark = pytest.mark.gpu
SIMPLE = 2                     # DSV4_FLAG_IMPL_SIMPLE


@pytest.fixture(scope="module")
def K():
    assert torch.cuda.is_available() and torch.cuda.get_device_capability(0)[0] == 10
    from deepseek_v4_kernel import cuda as K
    return K


@pytest.mark.parametrize("seed", [11, 12, 13])
def test_random_decode_shapes(K, seed):
    rng = random.Random(seed)
    for _ in range(150):
        layout = rng.choice([O.MODEL1, O.V32])
        b, h_q = rng.choice([1, 2, 3, 5, 16]), rng.choice([8, 16, 32, 48, 64, 128])
        topk, nb = rng.choice([16, 48, 128, 130, 256, 700, 1024, 2048]), rng.choice([2, 8, 33])
        n_splits = rng.choice([None, 1, 2, 3, 4, 5, 8, 16])
        s = rng.randrange(1 << 30)
        q, pages, idx = D.fake_batch(b, h_q, nb, topk, seed=s, layout=layout)
        gen = torch.Generator().manual_seed(s)
        tk = torch.randint(0, topk + 1, (b,), generator=gen, dtype=torch.int32) if rng.random() < 0.5 else None
        sink = torch.randn(h_q, generator=gen) if rng.random() < 0.5 else None
        flags = rng.choice([0, 1, 8, 9])               # masking of invalid entries, empty zero-length lists
        sm = 1 / math.sqrt(layout.d_qk)
        case = (layout is O.V32, b, h_q, topk, nb, n_splits, s, flags, tk is not None, sink is not None)
        o1, l1 = D.run(K, q, pages, idx, sm, tk, sink, flags, n_splits, layout)
        o2, l2 = D.run(K, q, pages, idx, sm, tk, sink, flags | SIMPLE, n_splits, layout)
        assert K.device_status() == 0, case
        fin = torch.isfinite(l2)
        assert torch.equal(torch.isfinite(l1), fin), case
        assert torch.allclose(l1[fin], l2[fin], atol=1e-3, rtol=1e-3), case
        assert torch.allclose(o1.float(), o2.float(), atol=5e-3, rtol=2 ** -7), case


@pytest.mark.parametrize("seed", [21, 22])
def test_random_prefill_shapes(K, seed):
    rng = random.Random(seed)
    c = lambda t: None if t is None else t.cuda()
    for _ in range(100):
        s_q, h_q = rng.choice([1, 3, 17, 64, 200]), rng.choice([8, 16, 32, 64, 128])
        s_kv, topk = rng.choice([1, 40, 129, 1000, 5000]), rng.choice([16, 100, 128, 129, 512, 1500, 2048])
        d_qk, s = rng.choice([512, 576]), rng.randrange(1 << 30)
        q, kv, idx, sink, tl = P.batch(s_q, h_q, s_kv, topk, s, d_qk=d_qk, with_len=rng.random() < 0.5,
                                       with_sink=rng.random() < 0.5)
        sm = 1 / math.sqrt(d_qk)
        case = (s_q, h_q, s_kv, topk, d_qk, s, tl is not None, sink is not None)
        a = K.sparse_prefill_fwd(q.cuda(), kv.cuda(), idx.cuda(), sm, 512, c(sink), c(tl), flags=0)
        b = K.sparse_prefill_fwd(q.cuda(), kv.cuda(), idx.cuda(), sm, 512, c(sink), c(tl), flags=SIMPLE)
        assert K.device_status() == 0, case
        assert torch.allclose(a[0].float(), b[0].float(), atol=5e-3, rtol=2 ** -7), case
        for x, y in ((a[1], b[1]), (a[2], b[2])):
            fin = torch.isfinite(y)
            assert torch.equal(torch.isfinite(x), fin) and torch.equal(torch.isposinf(x), torch.isposinf(y)), case
            assert torch.allclose(x[fin], y[fin], atol=1e-2, rtol=1e-2), case
