"""GPU tests of the cache that reserves device addresses once and maps memory behind them as it fills
(shainet_attn_kv_create_reserved; no counterpart in the reference, whose cache is reallocated and uploaded again when it
grows).  To the kernels it is an ordinary cache, so the parity bars are the usual ones (decode 1e-5, TF32 prefill 2e-3)."""
import numpy as np
import pytest

from helpers import DECODE_TOL, make_pair, qkv, rel_err

pytestmark = pytest.mark.gpu
PREFILL_TOL = 2e-3


@pytest.fixture(scope="module")
def ctx():
    import shainet_b200 as S
    from shainet_b200 import build
    build.build()
    c = S.AttnContext(0)
    yield c
    c.close()


def test_growth_maps_pages_and_moves_nothing(ctx):
    """head_dim 64 fp32: a 2 MB page holds 8192 rows of one kv head.  The cache is filled to just below a page boundary,
    decoded across it, extended by a tensor-core chunk; addresses and capacity never change, device memory in use follows
    the pages mapped, and every output matches the oracle."""
    import torch
    import shainet_b200 as S
    from shainet_b200 import _lib
    rng = np.random.default_rng(9001)
    shape = dict(H=8, KV=2, hd=64, theta=500000.0)
    free0 = torch.cuda.mem_get_info()[0]
    o, g = make_pair(ctx, shape, rng, reserve_capacity=20000)
    cap = g.cache.capacity
    assert cap >= 20000 and cap % 8192 == 0
    ptrs = g.cache.device_ptrs()
    assert free0 - torch.cuda.mem_get_info()[0] < (4 << 20)          # addresses only, no memory yet
    kc = rng.standard_normal((2, 8190, 64), dtype=np.float32)
    vc = rng.standard_normal((2, 8190, 64), dtype=np.float32)
    o.import_cache(kc, vc); g.cache.import_(kc, vc)
    used1 = free0 - torch.cuda.mem_get_info()[0]
    assert (8 << 20) <= used1 <= (16 << 20)                            # one 2 MB page behind each of 2 heads x 2 tensors
    for step in range(5):                                              # rows 8190 .. 8194: across the page boundary
        q, k, v = qkv(rng, shape, 1)
        assert rel_err(g.forward_cached(q, k, v), o.attend_cached(q, k, v, threads=8)) <= DECODE_TOL, step
    used2 = free0 - torch.cuda.mem_get_info()[0]
    assert used2 - used1 >= (8 << 20)                                  # a second page each
    q, k, v = qkv(rng, shape, 300)                                     # tensor-core prefill chunk on top
    ref = o.attend_cached(q, k, v, threads=8)
    got = g.forward_cached(q, k, v)
    assert rel_err(got, ref) <= PREFILL_TOL, rel_err(got, ref)
    assert g.cache.device_ptrs() == ptrs and g.cache.capacity == cap and g.cache_len == 8495
    ko, vo = o.export_cache(); kg, vg = g.cache.export()
    assert np.array_equal(vo, vg) and np.abs(ko - kg).max() <= 4e-7 * np.abs(ko).max()
    # clear and reuse: pages stay mapped
    o.clear_cache(); g.clear_cache()
    q, k, v = qkv(rng, shape, 3)
    assert rel_err(g.forward_cached(q, k, v), o.attend_cached(q, k, v)) <= DECODE_TOL
    # past the reservation
    with pytest.raises(S.ShainetAttnError) as e:
        g.cache.reserve(cap + 1)
    assert e.value.code == _lib.E_INVALID
    used3 = free0 - torch.cuda.mem_get_info()[0]
    g.close()
    torch.cuda.synchronize()
    # the 8 pages are unmapped and released (what remains is the context's own scratch)
    assert used3 - (free0 - torch.cuda.mem_get_info()[0]) >= (16 << 20)


def test_reserved_bf16_cache_and_batched_decode(ctx):
    """The element format and the address reservation are independent: bfloat16 rows in reserved ranges, two such caches
    and an ordinary one decoded in one batched launch."""
    import torch
    import shainet_b200 as S
    rng = np.random.default_rng(9002)
    shape = dict(H=32, KV=8, hd=128, theta=1e6, qk_norm=True)
    qn = (1.0 + 0.02 * rng.standard_normal(128)).astype(np.float32)
    pairs = [make_pair(ctx, shape, rng, q_norm=qn, k_norm=qn, kv_format="bf16", reserve_capacity=r) for r in (5000, 9000, 0)]
    lens = [4090, 70, 900]
    for (o, g), L in zip(pairs, lens):
        kc = rng.standard_normal((8, L, 128), dtype=np.float32)
        vc = rng.standard_normal((8, L, 128), dtype=np.float32)
        o.import_cache(kc, vc); g.cache.import_(kc, vc)
    dev = torch.device("cuda:0")
    stream = torch.cuda.current_stream().cuda_stream
    for step in range(8):                                              # the first cache crosses 4096 rows = its first page
        q, k, v = qkv(rng, shape, 3)
        tq, tk, tv = (torch.from_numpy(x).to(dev) for x in (q, k, v))
        out = torch.empty_like(tq)
        S.forward_batched_dev(ctx, [g.cache for _, g in pairs], tq.data_ptr(), tk.data_ptr(), tv.data_ptr(), out.data_ptr(),
                              pairs[0][1].scale, stream)
        torch.cuda.synchronize()
        got = out.cpu().numpy()
        for b, (o, g) in enumerate(pairs):
            ref = o.attend_cached(q[b:b + 1], k[b:b + 1], v[b:b + 1], threads=8)
            assert rel_err(got[b:b + 1], ref) <= 5e-3 if not np.array_equal(o.export_cache()[0], g.cache.export()[0]) \
                else rel_err(got[b:b + 1], ref) <= DECODE_TOL, (step, b)
    for _, g in pairs:
        g.close()
