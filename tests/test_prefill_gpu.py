"""Tensor-core (tcgen05, TF32) causal prefill against the CPU oracle.
Tolerance: max|y-ref|/max|ref| <= 2e-3 (TF32 rounds the inputs of both
contractions to 10 mantissa bits); decode steps that follow stay at 1e-5
because the cache itself is fp32 and identical."""
import numpy as np
import pytest

from helpers import DECODE_TOL, L1B, Q30, Q8B, make_pair, qkv, rel_err

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


@pytest.mark.parametrize("shape,T", [(L1B, 512), (Q8B, 256), (Q30, 130), (Q8B, 64), (L1B, 1000)],
                         ids=["llama1b_512", "qwen3_8b_256", "qwen3_30b_130", "qwen3_8b_64", "llama1b_1000"])
def test_prefill_from_empty_cache(ctx, shape, T):
    import shainet_b200 as S
    rng = np.random.default_rng(3001)
    o, g = make_pair(ctx, shape, rng)
    q, k, v = qkv(rng, shape, T)
    ref = o.attend_cached(q, k, v, threads=8)
    got = g.forward_cached(q, k, v, S.F_TENSOR)
    e = rel_err(got, ref)
    assert e <= PREFILL_TOL, e
    # every row, not only the largest: per-row error against the row's own scale
    per_row = np.abs(got - ref).max(axis=1) / np.abs(ref).max(axis=1)
    assert per_row.max() <= 4 * PREFILL_TOL, per_row.max()
    # the cache is exact fp32 work, and decode after the prefill is at decode tolerance
    ko, vo = o.export_cache(); kg, vg = g.cache.export()
    assert np.array_equal(vo, vg) and np.abs(ko - kg).max() <= 4e-7 * np.abs(ko).max()
    q, k, v = qkv(rng, shape, 1)
    assert rel_err(g.forward_cached(q, k, v), o.attend_cached(q, k, v)) <= DECODE_TOL
    g.close()


def test_chunked_prefill_over_existing_cache(ctx):
    """A second chunk attends to the rows of the first (start_pos > 0) and to
    its own rows causally; chunk sizes are not multiples of the tiles."""
    import shainet_b200 as S
    rng = np.random.default_rng(3002)
    o, g = make_pair(ctx, Q8B, rng)
    for T in (300, 200, 77):
        q, k, v = qkv(rng, Q8B, T)
        ref = o.attend_cached(q, k, v, threads=8)
        got = g.forward_cached(q, k, v, S.F_TENSOR)
        assert rel_err(got, ref) <= PREFILL_TOL, (T, rel_err(got, ref))
    assert g.cache_len == 577
    g.close()


def test_default_dispatch_uses_tensor_kernel_for_long_chunks(ctx):
    """No flags: >= 64 rows go to the tensor-core kernel (TF32-level agreement
    with the fp32 kernel, not bit equality), short chunks stay on fp32 kernels."""
    import shainet_b200 as S
    rng = np.random.default_rng(3003)
    shape = Q30
    o, g = make_pair(ctx, shape, rng)
    _, g2 = make_pair(ctx, shape, np.random.default_rng(3003))
    q, k, v = qkv(rng, shape, 192)
    ref = o.attend_cached(q, k, v, threads=8)
    a = g.forward_cached(q, k, v)                 # default: tensor cores
    b = g2.forward_cached(q, k, v, S.F_GENERIC)   # forced fp32
    assert rel_err(b, ref) <= DECODE_TOL
    assert rel_err(a, ref) <= PREFILL_TOL
    assert not np.array_equal(a, b)
    g.close(); g2.close()


@pytest.mark.parametrize("H,KV,hd,T", [(8, 8, 64, 300), (6, 2, 128, 520), (4, 4, 128, 128)],
                         ids=["mha_3_row_tiles", "group3_5_row_tiles", "mha_one_row_tile"])
def test_prefill_pairs_row_tiles_when_the_group_size_is_odd(ctx, H, KV, hd, T):
    """With an odd group size a CTA takes two consecutive row tiles of one head instead of
    two heads of a kv group; the tiles then see different numbers of K/V tiles, and with an
    odd number of row tiles the last CTA has one empty tile."""
    import shainet_b200 as S
    rng = np.random.default_rng(3003)
    shape = dict(H=H, KV=KV, hd=hd, theta=10000.0, qk_norm=False)
    o, g = make_pair(ctx, shape, rng)
    q, k, v = qkv(rng, shape, T)
    ref = o.attend_cached(q, k, v, threads=8)
    got = g.forward_cached(q, k, v, S.F_TENSOR)
    assert rel_err(got, ref) <= PREFILL_TOL, rel_err(got, ref)
    q, k, v = qkv(rng, shape, 70)      # a second chunk over the first
    ref = o.attend_cached(q, k, v, threads=8)
    got = g.forward_cached(q, k, v, S.F_TENSOR)
    assert rel_err(got, ref) <= PREFILL_TOL, rel_err(got, ref)
    g.close()


@pytest.mark.parametrize("shape,T", [(Q8B, 700), (L1B, 384), (Q30, 257)], ids=["qwen3_8b_700", "llama1b_384", "qwen3_30b_257"])
def test_cluster_pair_kernel_and_single_cta_kernel_against_the_oracle(ctx, shape, T):
    """Even group sizes at head_dim 128 run on a cluster of two CTAs (two query heads of one kv head, one tensor-core tile
    of 256 rows, 128-position steps); SHAINET_ATTN_F_TENSOR_1CTA keeps the one-CTA kernel (two tiles per CTA, 64-position steps).
    Both against the oracle, a first chunk and a second one over it; the two kernels also agree with each other
    far inside the tolerance (same TF32 products, different summation order)."""
    import shainet_b200 as S
    rng = np.random.default_rng(3010)
    o, g = make_pair(ctx, shape, rng)
    _, g1 = make_pair(ctx, shape, np.random.default_rng(3010))
    for n in (T, 130):
        q, k, v = qkv(rng, shape, n)
        ref = o.attend_cached(q, k, v, threads=8)
        pair = g.forward_cached(q, k, v, S.F_TENSOR)
        single = g1.forward_cached(q, k, v, S.F_TENSOR | S.F_TENSOR_1CTA)
        assert rel_err(pair, ref) <= PREFILL_TOL, (n, rel_err(pair, ref))
        assert rel_err(single, ref) <= PREFILL_TOL, (n, rel_err(single, ref))
        assert rel_err(pair, single) <= PREFILL_TOL / 2
        # head_dim 128: two different kernels did run; head_dim 64 runs the one-CTA kernel either way
        assert np.array_equal(pair, single) == (shape["hd"] == 64)
    g.close(); g1.close()


@pytest.mark.parametrize("H,KV,hd,T,pre", [(4, 2, 128, 130, 0), (16, 1, 64, 300, 45), (8, 4, 64, 129, 128), (16, 2, 128, 257, 3)],
                         ids=["g2_hd128", "g16_hd64_over_45", "g2_hd64_over_128", "g8_hd128_over_3"])
def test_cluster_pair_kernel_group_sizes_and_ragged_edges(ctx, H, KV, hd, T, pre):
    """Group sizes 2, 8 and 16 at both head dims (the pair kernel at 128, the one-CTA kernel at 64), row counts one past
    a tile, and existing cache lengths that leave the first step ragged."""
    import shainet_b200 as S
    rng = np.random.default_rng(3011)
    shape = dict(H=H, KV=KV, hd=hd, theta=10000.0, qk_norm=(hd == 128))
    o, g = make_pair(ctx, shape, rng)
    if pre:
        q, k, v = qkv(rng, shape, pre)
        o.attend_cached(q, k, v); g.forward_cached(q, k, v, S.F_GENERIC)
    q, k, v = qkv(rng, shape, T)
    ref = o.attend_cached(q, k, v, threads=8)
    got = g.forward_cached(q, k, v, S.F_TENSOR)
    assert rel_err(got, ref) <= PREFILL_TOL, rel_err(got, ref)
    per_row = np.abs(got - ref).max(axis=1) / np.abs(ref).max(axis=1)
    assert per_row.max() <= 4 * PREFILL_TOL, (float(per_row.max()), int(per_row.argmax()))
    g.close()
