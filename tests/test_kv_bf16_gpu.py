"""GPU parity of the opt-in bfloat16 KV cache.  The reference keeps fp32 rows only; this
format is defined as "the reference's arithmetic over rows rounded to bfloat16 (nearest
even) as they are appended", which is what the oracle computes with kv_rounding="bf16".
Tolerances are those of the fp32 cache: decode max|y-ref|/max|ref| <= 1e-5, TF32
tensor-core prefill <= 2e-3.  V rows are compared bit for bit; rotated K rows may differ
from the oracle's by one bfloat16 step where the device's and libm's cosf/sinf (an fp32
ulp apart) fall on the two sides of a rounding boundary."""
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


def _k_rows_agree(kg, ko):
    """Equal, except for rare elements one bfloat16 step apart."""
    diff = kg != ko
    if diff.any():
        assert diff.mean() < 2e-3, diff.mean()
        step = np.abs(ko[diff]) * 2.0 ** -7 + 1e-30     # one bfloat16 step is at most 2^-7 of the value
        assert (np.abs(kg[diff] - ko[diff]) <= step).all()


def _checked_step(o, g, q, k, v):
    """One token through both sides.  With bit-identical rows the outputs agree to the decode
    tolerance.  Where a rotated K element of the new row landed one bfloat16 step away from the
    oracle's (see the module text), the step is held to that element's worst effect instead and
    the oracle continues from the library's rows.  Returns True for such a step."""
    ref = o.attend_cached(q, k, v)
    got = g.forward_cached(q, k, v)
    ko, vo = o.export_cache(); kg, vg = g.cache.export()
    assert np.array_equal(vo, vg)
    if np.array_equal(ko, kg):
        assert rel_err(got, ref) <= DECODE_TOL, rel_err(got, ref)
        return False
    assert np.array_equal(ko[:, :-1], kg[:, :-1])       # only the row appended by this step can differ
    _k_rows_agree(kg, ko)
    assert rel_err(got, ref) <= 5e-3, rel_err(got, ref)
    o.clear_cache()
    o.import_cache(kg, vg)
    return True


def test_import_export_and_fill_round_to_nearest_even(ctx):
    import shainet_b200 as S
    from oracle import oracle as O
    rng = np.random.default_rng(11)
    c = S.KVCache(ctx, 8, 2, 64, kv_format="bf16")
    assert c.kv_format == "bf16"
    k = (rng.standard_normal((2, 300, 64)) * 3).astype(np.float32)
    v = rng.standard_normal((2, 300, 64)).astype(np.float32)
    k[0, 0, :4] = [1.00390625, 1.01171875, -1.00390625, 0.0]     # ties: to even
    c.import_(k, v)
    kg, vg = c.export()
    assert np.array_equal(kg, O.round_bf16(k)) and np.array_equal(vg, O.round_bf16(v))
    assert kg[0, 0, 0] == 1.0 and kg[0, 0, 1] == 1.015625 and kg[0, 0, 2] == -1.0
    # the device generator's values, rounded
    f = S.KVCache(ctx, 8, 2, 64)
    assert f.kv_format == "f32"
    f.fill_normal(1000, 77)
    c.fill_normal(1000, 77)
    for a, b in zip(c.export(), f.export()):
        assert np.array_equal(a, O.round_bf16(b))
    with pytest.raises(S.ShainetAttnError) as e:
        c.device_ptrs()
    from shainet_b200 import _lib
    assert e.value.code == _lib.E_UNSUPPORTED
    c.close(); f.close()


@pytest.mark.parametrize("shape,ctx_len", [(L1B, 4096), (Q8B, 3000), (Q30, 9000)],
                         ids=["llama1b_4k", "qwen3_8b_3k", "qwen3_30b_9k"])
def test_decode_over_a_bf16_cache(ctx, shape, ctx_len):
    """Fused decode kernel streaming bfloat16 rows: several steps over an imported long cache
    (many splits, merged through the epoch words), every output against the oracle."""
    rng = np.random.default_rng(5101)
    o, g = make_pair(ctx, shape, rng, kv_format="bf16")
    kc = rng.standard_normal((shape["KV"], ctx_len, shape["hd"]), dtype=np.float32)
    vc = rng.standard_normal((shape["KV"], ctx_len, shape["hd"]), dtype=np.float32)
    o.import_cache(kc, vc); g.cache.import_(kc, vc)
    for step in range(4):
        q, k, v = qkv(rng, shape, 1)
        ref = o.attend_cached(q, k, v, threads=8)
        got = g.forward_cached(q, k, v)
        assert rel_err(got, ref) <= DECODE_TOL, (step, rel_err(got, ref))
    ko, vo = o.export_cache(); kg, vg = g.cache.export()
    assert np.array_equal(vo, vg)
    _k_rows_agree(kg, ko)
    assert np.array_equal(kg[:, :ctx_len], ko[:, :ctx_len])
    g.close()


@pytest.mark.parametrize("G", [1, 2, 4, 8, 16])
@pytest.mark.parametrize("hd", [64, 128])
def test_every_group_size_from_an_empty_cache(ctx, G, hd):
    """Token by token from length 0 (single tile, ragged tiles, first split boundary), every
    template instance of the bfloat16 kernel."""
    rng = np.random.default_rng(100 * G + hd)
    shape = dict(H=16, KV=16 // G, hd=hd, theta=10000.0, qk_norm=(G % 4 == 0))
    o, g = make_pair(ctx, shape, rng, kv_format="bf16")
    moved = sum(_checked_step(o, g, *qkv(rng, shape, 1)) for _ in range(70))
    assert moved <= 4, moved
    g.close()


def test_prefill_chunks_growth_truncate_and_forced_kernels(ctx):
    """Chunks of several tokens (generic kernel, tensor-core kernel), growth of the 16-bit
    buffers, roll-back, and the unfused decode path: all read the fp32 image of the rows."""
    import shainet_b200 as S
    rng = np.random.default_rng(5202)
    shape = Q8B
    o, g = make_pair(ctx, shape, rng, initial_capacity=256, kv_format="bf16")
    q, k, v = qkv(rng, shape, 7)                       # short chunk: fp32 kernels
    assert rel_err(g.forward_cached(q, k, v), o.attend_cached(q, k, v)) <= DECODE_TOL
    q, k, v = qkv(rng, shape, 600)                     # long chunk: TF32 tensor cores, capacity 256 -> 1024
    ref = o.attend_cached(q, k, v, threads=8)
    got = g.forward_cached(q, k, v)
    assert rel_err(got, ref) <= PREFILL_TOL, rel_err(got, ref)
    assert g.cache.capacity >= 607 and g.cache_len == 607
    ko, vo = o.export_cache(); kg, vg = g.cache.export()
    assert np.array_equal(vo, vg)
    _k_rows_agree(kg, ko)
    for flags in (0, S.F_UNFUSED, S.F_GENERIC, S.F_SPLITK | S.F_UNFUSED):
        q, k, v = qkv(rng, shape, 1)
        ref = o.attend_cached(q, k, v, threads=8)
        got = g.forward_cached(q, k, v, flags)
        assert rel_err(got, ref) <= DECODE_TOL, (flags, rel_err(got, ref))
    # roll three positions back and replay different tokens (the oracle replays from its exported rows)
    n = g.cache_len - 3
    g.cache.truncate(n)
    ko, vo = o.export_cache()
    o.clear_cache()
    o.import_cache(ko[:, :n], vo[:, :n])
    for _ in range(3):
        q, k, v = qkv(rng, shape, 1)
        assert rel_err(g.forward_cached(q, k, v), o.attend_cached(q, k, v, threads=8)) <= DECODE_TOL
    g.close()


def test_batched_ragged_decode_over_bf16_caches(ctx):
    import torch
    import shainet_b200 as S
    from shainet_b200 import _lib
    rng = np.random.default_rng(4101)
    shape = Q8B
    lens = [1, 17, 64, 100, 1000, 3000]
    qn = (1.0 + 0.02 * rng.standard_normal(shape["hd"])).astype(np.float32)
    kn = (1.0 + 0.02 * rng.standard_normal(shape["hd"])).astype(np.float32)
    pairs = [make_pair(ctx, shape, rng, q_norm=qn, k_norm=kn, kv_format="bf16") for _ in lens]
    dev = torch.device("cuda:0")
    stream = torch.cuda.current_stream().cuda_stream
    for (o, g), L in zip(pairs, lens):
        kc = rng.standard_normal((shape["KV"], L, shape["hd"]), dtype=np.float32)
        vc = rng.standard_normal((shape["KV"], L, shape["hd"]), dtype=np.float32)
        o.import_cache(kc, vc); g.cache.import_(kc, vc)
    B = len(lens)
    for step in range(3):
        q, k, v = qkv(rng, shape, B)
        tq, tk, tv = (torch.from_numpy(x).to(dev) for x in (q, k, v))
        out = torch.empty_like(tq)
        S.forward_batched_dev(ctx, [g.cache for _, g in pairs], tq.data_ptr(), tk.data_ptr(), tv.data_ptr(),
                              out.data_ptr(), pairs[0][1].scale, stream)
        torch.cuda.synchronize()
        got = out.cpu().numpy()
        for b, (o, g) in enumerate(pairs):
            ref = o.attend_cached(q[b:b + 1], k[b:b + 1], v[b:b + 1])
            assert rel_err(got[b:b + 1], ref) <= DECODE_TOL, (step, b)
            assert g.cache_len == lens[b] + step + 1
    # formats cannot be mixed in one batch, and a forced kernel has no 16-bit batched form
    plain = S.LlamaAttention(ctx, shape["H"], shape["KV"], shape["hd"], shape["theta"], q_norm=qn, k_norm=kn)
    tq, tk, tv = (torch.zeros(2, n, device=dev) for n in (plain.q_dim, plain.kv_dim, plain.kv_dim))
    out = torch.empty_like(tq)
    with pytest.raises(S.ShainetAttnError) as e:
        S.forward_batched_dev(ctx, [pairs[0][1].cache, plain.cache], tq.data_ptr(), tk.data_ptr(), tv.data_ptr(),
                              out.data_ptr(), plain.scale, stream)
    assert e.value.code == _lib.E_INVALID
    with pytest.raises(S.ShainetAttnError) as e:
        S.forward_batched_dev(ctx, [pairs[0][1].cache, pairs[1][1].cache], tq.data_ptr(), tk.data_ptr(), tv.data_ptr(),
                              out.data_ptr(), plain.scale, stream, S.F_UNFUSED)
    assert e.value.code == _lib.E_UNSUPPORTED
    assert pairs[0][1].cache_len == lens[0] + 3
    plain.close()
    for _, g in pairs:
        g.close()


def test_bf16_result_is_the_reference_arithmetic_on_the_stored_rows(ctx):
    """The definition, without the oracle's rounding mode: after a step, the rows the 16-bit cache holds
    (exported, the new token's included) go into a plain fp32 oracle; its attention over them, for the
    same q, is the step's output."""
    import shainet_b200 as S
    from oracle import oracle as O
    rng = np.random.default_rng(77)
    shape = dict(H=32, KV=8, hd=64, theta=500000.0)
    a = S.LlamaAttention(ctx, 32, 8, 64, 500000.0, kv_format="bf16")
    kc = rng.standard_normal((8, 5000, 64), dtype=np.float32)
    vc = rng.standard_normal((8, 5000, 64), dtype=np.float32)
    a.cache.import_(kc, vc)
    q, k, v = qkv(rng, shape, 1)
    got = a.forward_cached(q, k, v)
    ka, va = a.cache.export()
    assert ka.shape[1] == 5001 and np.array_equal(ka, O.round_bf16(ka)) and np.array_equal(va[:, 5000], O.round_bf16(v).reshape(8, 64))
    o = O.OracleAttention(32, 8, 64, 500000.0)
    o.import_cache(ka, va)
    ref = o.attend_only(q, 5000, threads=8)       # q is rotated inside, at position 5000
    assert rel_err(got, ref) <= DECODE_TOL, rel_err(got, ref)
    a.close()
