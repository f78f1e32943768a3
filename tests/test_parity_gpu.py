"""GPU parity: libshainet_attn (through its C ABI) against the CPU oracle on the
same seeded inputs.  Tolerances: decode max|y-ref|/max|ref| <= 1e-5; the
reference's own spec bound (max-abs < 1e-3, cosine > 0.9999) is asserted too
where the case replays one of its specs."""
import numpy as np
import pytest

from helpers import DECODE_TOL, L1B, Q30, Q8B, SPEC_ABS_TOL, cosine, make_pair, qkv, rel_err

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    import shainet_b200 as S
    from shainet_b200 import build
    build.build()
    c = S.AttnContext(0)
    yield c
    c.close()


def _run_both(o, g, seq, flags=0):
    outs = []
    for (q, k, v) in seq:
        outs.append((o.attend_cached(q, k, v), g.forward_cached(q, k, v, flags)))
    return outs


def test_spec_gqa_prefill_then_decode(ctx):
    # spec/llama_attention_gpu_spec.cr:17-66 — 8 heads / 4 KV heads, head_dim 8,
    # inputs U(-1,1), prefill of 6 then 3 single-token steps.
    rng = np.random.default_rng(42)
    shape = dict(H=8, KV=4, hd=8, theta=10000.0)
    o, g = make_pair(ctx, shape, rng)
    seq = [qkv(rng, shape, 6, "uniform")] + [qkv(rng, shape, 1, "uniform") for _ in range(3)]
    for ref, got in _run_both(o, g, seq):
        assert np.abs(ref - got).max() < SPEC_ABS_TOL
        assert cosine(got, ref) > 0.9999
        assert rel_err(got, ref) <= DECODE_TOL
    assert g.cache_len == 9 == o.cache_len
    g.close()


def test_spec_growth_and_clear_cache(ctx):
    # spec/llama_attention_gpu_spec.cr:68-104 — 4/2 heads, head_dim 8, 290-token
    # prefill (past the initial capacity of 256) + 10 steps, replayed after clear.
    rng = np.random.default_rng(7)
    shape = dict(H=4, KV=2, hd=8, theta=10000.0)
    o, g = make_pair(ctx, shape, rng, initial_capacity=256)
    assert g.cache.capacity == 256
    seq = [qkv(rng, shape, 290, "uniform")] + [qkv(rng, shape, 1, "uniform") for _ in range(10)]
    first = _run_both(o, g, seq)
    assert g.cache.capacity >= 300 and g.cache_len == 300
    cap = g.cache.capacity
    o.clear_cache(); g.clear_cache()
    assert g.cache_len == 0 and g.cache.capacity == cap      # buffers are kept (llama_block.cr:120-121)
    second = _run_both(o, g, seq)
    for ref, got in first + second:
        assert np.abs(ref - got).max() < SPEC_ABS_TOL
        assert rel_err(got, ref) <= DECODE_TOL
    g.close()


def test_growth_moves_rows_device_to_device(ctx):
    rng = np.random.default_rng(9)
    shape = dict(H=4, KV=2, hd=16, theta=10000.0)
    o, g = make_pair(ctx, shape, rng)
    for n in (3, 250, 4, 300, 1):     # 0 -> 256 -> 512 -> 1024
        q, k, v = qkv(rng, shape, n)
        assert rel_err(g.forward_cached(q, k, v), o.attend_cached(q, k, v)) <= DECODE_TOL
    assert g.cache.capacity == 1024
    ko, vo = o.export_cache(); kg, vg = g.cache.export()
    assert np.array_equal(vo, vg)
    assert np.abs(ko - kg).max() <= 2e-6
    g.close()


@pytest.mark.parametrize("shape", [L1B, Q8B, Q30], ids=["llama1b", "qwen3_8b", "qwen3_30b"])
def test_cache_contents_match_oracle(ctx, shape):
    """Fused bias/QK-norm/RoPE/append: V rows bit-exact, rotated K rows equal up
    to the ulp-level difference between device and libm cosf/sinf."""
    rng = np.random.default_rng(100)
    o, g = make_pair(ctx, shape, rng)
    for n in (37, 1, 1):
        q, k, v = qkv(rng, shape, n)
        o.attend_cached(q, k, v); g.forward_cached(q, k, v)
    ko, vo = o.export_cache(); kg, vg = g.cache.export()
    assert np.array_equal(vo, vg)
    assert np.abs(ko - kg).max() <= 4 * np.finfo(np.float32).eps * np.abs(ko).max()
    assert (ko != kg).mean() < 0.2     # most rotated elements are bit-identical
    g.close()


@pytest.mark.parametrize("shape,ctx_len", [(L1B, 4096), (Q8B, 3000), (Q30, 32768)],
                         ids=["llama1b_4k", "qwen3_8b_3k", "qwen3_30b_32k"])
def test_decode_long_context(ctx, shape, ctx_len):
    """Split-K decode over a pre-filled N(0,1) cache at the benchmark contexts."""
    import shainet_b200 as S
    rng = np.random.default_rng(5001)
    o, g = make_pair(ctx, shape, rng)
    kc = rng.standard_normal((shape["KV"], ctx_len, shape["hd"]), dtype=np.float32)
    vc = rng.standard_normal((shape["KV"], ctx_len, shape["hd"]), dtype=np.float32)
    o.import_cache(kc, vc); g.cache.import_(kc, vc)
    for step in range(2):
        q, k, v = qkv(rng, shape, 1)
        ref = o.attend_cached(q, k, v, threads=8)
        got = g.forward_cached(q, k, v)
        assert rel_err(got, ref) <= DECODE_TOL, (step, rel_err(got, ref))
    # the forced generic kernel agrees too, and both sit at the f64 truth's distance
    q, k, v = qkv(rng, shape, 1)
    ref = o.attend_cached(q, k, v, threads=8)
    got = g.forward_cached(q, k, v, S.F_GENERIC)
    assert rel_err(got, ref) <= DECODE_TOL
    assert g.cache_len == ctx_len + 3
    g.close()


def test_decode_error_against_f64_truth(ctx):
    """The kernel is no further from an f64-accumulated truth than the reference's
    sequential fp32 arithmetic is (or within the tolerance floor)."""
    rng = np.random.default_rng(77)
    shape = Q30
    o, g = make_pair(ctx, shape, rng)
    L = 8192
    kc = rng.standard_normal((shape["KV"], L, shape["hd"]), dtype=np.float32)
    vc = rng.standard_normal((shape["KV"], L, shape["hd"]), dtype=np.float32)
    g.cache.import_(kc, vc)
    q, k, v = qkv(rng, shape, 1)
    got = g.forward_cached(q, k, v)
    o.import_cache(kc, vc)
    ref32 = o.attend_cached(q, k, v, threads=8, mode=0)
    o.import_cache(kc, vc)
    ref64 = o.attend_cached(q, k, v, threads=8, mode=1)
    e_kernel, e_oracle = rel_err(got, ref64), rel_err(ref32, ref64)
    assert e_kernel <= max(DECODE_TOL, e_oracle), (e_kernel, e_oracle)
    g.close()


@pytest.mark.parametrize("fused", ["fused", "fused_tickets", "three_launches"])
@pytest.mark.parametrize("hd", [64, 128])
@pytest.mark.parametrize("G", [1, 2, 4, 8, 16])
def test_splitk_every_group_size_and_ragged_lengths(ctx, hd, G, fused):
    """Split-K decode, one fused launch or RoPE/append + split-K + merge: every
    template instance, lengths around the tile and split boundaries (empty cache,
    1 row, partial tiles, exact multiples)."""
    import shainet_b200 as S
    flags = S.F_SPLITK | {"fused": 0, "fused_tickets": S.F_TICKET_MERGE, "three_launches": S.F_UNFUSED}[fused]
    rng = np.random.default_rng(hd * 100 + G)
    KV = 2
    shape = dict(H=KV * G, KV=KV, hd=hd, theta=10000.0)
    for L in (0, 1, 7, 8, 63, 64, 65, 255, 1031, 2500):
        o, g = make_pair(ctx, shape, rng)
        if L:
            q, k, v = qkv(rng, shape, L)
            o.attend_cached(q, k, v)
            kc, vc = o.export_cache()
            g.cache.import_(kc, vc)
        for _ in range(2):
            q, k, v = qkv(rng, shape, 1)
            e = rel_err(g.forward_cached(q, k, v, flags), o.attend_cached(q, k, v))
            assert e <= DECODE_TOL, (L, fused, e)
        g.close()


@pytest.mark.parametrize("inputs_ready", [False, True], ids=["dependent", "inputs_ready"])
def test_back_to_back_decode_without_sync(ctx, inputs_ready):
    """Asynchronous device-pointer calls queued back to back: a fused kernel may
    start while its predecessor is still appending the previous row of the same
    cache; two caches are also interleaved on one stream.  With F_INPUTS_READY
    (the inputs here were uploaded long before) it also computes while the
    predecessor drains."""
    import torch
    import shainet_b200 as S
    flags = S.F_INPUTS_READY if inputs_ready else 0
    rng = np.random.default_rng(808)
    dev = torch.device("cuda:0")
    stream = torch.cuda.current_stream().cuda_stream
    pairs = [make_pair(ctx, Q30, rng), make_pair(ctx, Q30, rng)]
    for o, g in pairs:
        q, k, v = qkv(rng, Q30, 4500)
        o.attend_cached(q, k, v, threads=8)
        kc, vc = o.export_cache()
        g.cache.import_(kc, vc)
        g.cache.reserve(4600)
    steps = 24
    ins = [[qkv(rng, Q30, 1) for _ in pairs] for _ in range(steps)]
    dins = [[tuple(torch.from_numpy(x).to(dev) for x in trip) for trip in row] for row in ins]
    outs = [[torch.empty(1, Q30["H"] * Q30["hd"], device=dev) for _ in pairs] for _ in range(steps)]
    torch.cuda.synchronize()
    for t in range(steps):
        for i, (_, g) in enumerate(pairs):
            reps = 2 if (t % 5 == 0 and i == 0) else 1     # sometimes the same cache twice in a row
            for _ in range(reps):
                tq, tk, tv = dins[t][i]
                g.forward_cached_dev(tq.data_ptr(), tk.data_ptr(), tv.data_ptr(), outs[t][i].data_ptr(), 1, stream, flags)
    torch.cuda.synchronize()
    ctx.sync()
    for t in range(steps):
        for i, (o, _) in enumerate(pairs):
            reps = 2 if (t % 5 == 0 and i == 0) else 1
            for _ in range(reps):
                ref = o.attend_cached(*ins[t][i])
            assert rel_err(outs[t][i].cpu().numpy(), ref) <= DECODE_TOL, (t, i)
    for o, g in pairs:
        ko, vo = o.export_cache(); kg, vg = g.cache.export()
        assert np.array_equal(vo, vg) and np.abs(ko - kg).max() <= 4e-7 * np.abs(ko).max()
        g.close()


def test_splitk_several_new_tokens(ctx):
    """2..16 new tokens go through the decode kernel, one row per CTA column."""
    rng = np.random.default_rng(31)
    o, g = make_pair(ctx, Q30, rng)
    q, k, v = qkv(rng, Q30, 700)
    o.attend_cached(q, k, v); kc, vc = o.export_cache(); g.cache.import_(kc, vc)
    for T in (5, 16, 2):
        q, k, v = qkv(rng, Q30, T)
        assert rel_err(g.forward_cached(q, k, v), o.attend_cached(q, k, v)) <= DECODE_TOL
    g.close()


def test_prefill_then_decode_qwen_shape(ctx):
    rng = np.random.default_rng(3001)
    o, g = make_pair(ctx, Q8B, rng)
    import shainet_b200 as S
    q, k, v = qkv(rng, Q8B, 96)
    # fp32 prefill kernel (the default for 96 rows would be the TF32 tensor-core kernel, tested elsewhere)
    assert rel_err(g.forward_cached(q, k, v, S.F_GENERIC), o.attend_cached(q, k, v, threads=8)) <= DECODE_TOL
    for _ in range(4):
        q, k, v = qkv(rng, Q8B, 1)
        assert rel_err(g.forward_cached(q, k, v), o.attend_cached(q, k, v)) <= DECODE_TOL
    g.close()


def test_bias_and_scaled_rope_table(ctx):
    # nil bias == zero bias (spec/llama_qkv_bias_spec.cr:8-40), real bias vs oracle,
    # LLaMA-3 scaled frequencies (hf_loader.cr:235-265) as an explicit table.
    from oracle import oracle as O
    rng = np.random.default_rng(17)
    shape = dict(H=8, KV=2, hd=64, theta=500000.0)
    freqs = O.llama3_rope_freqs(500000.0, 64, 32.0, 1.0, 4.0, 8192.0)
    bq = rng.standard_normal(8 * 64).astype(np.float32) * 0.1
    bk = rng.standard_normal(2 * 64).astype(np.float32) * 0.1
    bv = rng.standard_normal(2 * 64).astype(np.float32) * 0.1
    o, g = make_pair(ctx, shape, rng, rope_freqs=freqs, b_q=bq, b_k=bk, b_v=bv)
    o0, g0 = make_pair(ctx, shape, rng, rope_freqs=freqs)
    _, gz = make_pair(ctx, shape, rng, rope_freqs=freqs, b_q=0 * bq, b_k=0 * bk, b_v=0 * bv)
    for T in (20, 1, 1):
        q, k, v = qkv(rng, shape, T)
        got = g.forward_cached(q, k, v)
        assert rel_err(got, o.attend_cached(q, k, v)) <= DECODE_TOL
        a, z = g0.forward_cached(q, k, v), gz.forward_cached(q, k, v)
        assert np.abs(a - z).max() <= 1e-6
        assert np.abs(a - got).sum() > 0.01
    for x in (g, g0, gz):
        x.close()


def test_device_pointer_entry_and_batched_ragged_decode(ctx):
    """forward_dev on torch's stream, then lock-step batched decode of ragged
    sequences (lengths 1..3000) against one oracle per sequence."""
    import torch
    import shainet_b200 as S
    rng = np.random.default_rng(4001)
    shape = Q8B
    lens = [1, 17, 64, 100, 1000, 3000]
    qn = (1.0 + 0.02 * rng.standard_normal(shape["hd"])).astype(np.float32)
    kn = (1.0 + 0.02 * rng.standard_normal(shape["hd"])).astype(np.float32)
    pairs = [make_pair(ctx, shape, rng, q_norm=qn, k_norm=kn) for _ in lens]
    dev = torch.device("cuda:0")
    stream = torch.cuda.current_stream().cuda_stream
    for (o, g), L in zip(pairs, lens):
        q, k, v = qkv(rng, shape, L)
        ref = o.attend_cached(q, k, v, threads=8)
        tq, tk, tv = (torch.from_numpy(x).to(dev) for x in (q, k, v))
        out = torch.empty_like(tq)
        # fp32 kernels only (long chunks would otherwise go to the TF32 tensor-core kernel)
        g.forward_cached_dev(tq.data_ptr(), tk.data_ptr(), tv.data_ptr(), out.data_ptr(), L, stream, S.F_GENERIC if L > 16 else 0)
        torch.cuda.synchronize()
        assert rel_err(out.cpu().numpy(), ref) <= DECODE_TOL
    B = len(lens)
    for step in range(3):
        q, k, v = qkv(rng, shape, B)
        tq, tk, tv = (torch.from_numpy(x).to(dev) for x in (q, k, v))
        out = torch.empty_like(tq)
        S.forward_batched_dev(ctx, [g.cache for _, g in pairs], tq.data_ptr(), tk.data_ptr(), tv.data_ptr(),
                              out.data_ptr(), pairs[0][1].scale, stream)
        torch.cuda.synchronize()
        ctx.sync()
        got = out.cpu().numpy()
        for b, (o, g) in enumerate(pairs):
            ref = o.attend_cached(q[b:b + 1], k[b:b + 1], v[b:b + 1])
            assert rel_err(got[b:b + 1], ref) <= DECODE_TOL, (step, b)
            assert g.cache_len == lens[b] + step + 1
    for _, g in pairs:
        g.close()


def test_fill_normal_statistics(ctx):
    import shainet_b200 as S
    c = S.KVCache(ctx, 8, 2, 128)
    c.fill_normal(4096, 5001)
    k, v = c.export()
    for a in (k, v):
        assert abs(a.mean()) < 5e-3 and abs(a.std() - 1.0) < 5e-3
        assert np.isfinite(a).all() and np.abs(a).max() < 7
    assert abs(np.corrcoef(k.ravel()[:100000], v.ravel()[:100000])[0, 1]) < 0.02
    c2 = S.KVCache(ctx, 8, 2, 128)
    c2.fill_normal(4096, 5001)
    assert np.array_equal(c2.export()[0], k)
    c.close(); c2.close()


def test_error_paths(ctx):
    import shainet_b200 as S
    from shainet_b200 import _lib
    with pytest.raises(S.ShainetAttnError) as e:
        S.KVCache(ctx, 6, 4, 8)                      # llama_block.cr:80
    assert e.value.code == _lib.E_INVALID
    with pytest.raises(S.ShainetAttnError) as e:
        S.KVCache(ctx, 4, 4, 7)
    assert e.value.code == _lib.E_UNSUPPORTED
    a = S.LlamaAttention(ctx, 4, 2, 8)
    z = np.zeros((1, 32), np.float32), np.zeros((1, 16), np.float32), np.zeros((1, 16), np.float32)
    with pytest.raises(S.ShainetAttnError) as e:
        a.forward_cached(*z, flags=S.F_SPLITK)       # head_dim 8 has no split-K instance
    assert e.value.code == _lib.E_UNSUPPORTED and a.cache_len == 0
    with pytest.raises(S.ShainetAttnError):
        a.cache.set_rope(np.ones(3, np.float32))     # wrong table size
    with pytest.raises(S.ShainetAttnError):
        a.cache.export(5)                            # more rows than the cache holds
    out = a.forward_cached(np.zeros((0, 32), np.float32), np.zeros((0, 16), np.float32), np.zeros((0, 16), np.float32))
    assert out.shape == (0, 32) and a.cache_len == 0
    with pytest.raises(S.ShainetAttnError) as e:
        ctx.close()                                  # a cache is still alive
    assert e.value.code == _lib.E_STATE
    a.close()


def test_sequence_split_over_two_parts(ctx):
    """One sequence whose positions alternate between two caches (what two ranks
    of one head group hold): each part attends over its own rows with the token's
    true RoPE position, only the owner appends, and the library's merge of the
    two (output, log-sum-exp) pairs equals the unsplit oracle."""
    import torch
    import shainet_b200 as S
    from shainet_b200.sharding import plan
    rng = np.random.default_rng(5005)
    shape = Q30
    H, KV, hd = shape["H"], shape["KV"], shape["hd"]
    qn = (1 + 0.02 * rng.standard_normal(hd)).astype(np.float32)
    kn = (1 + 0.02 * rng.standard_normal(hd)).astype(np.float32)
    from oracle import oracle as O
    o = O.OracleAttention(H, KV, hd, shape["theta"], 1e-6, q_norm=qn, k_norm=kn)
    parts = [S.LlamaAttention(ctx, H, KV, hd, shape["theta"], 1e-6, q_norm=qn, k_norm=kn) for _ in range(2)]
    L0 = 3001
    q, k, v = qkv(rng, shape, L0)
    o.attend_cached(q, k, v, threads=8)
    kc, vc = o.export_cache()
    for p, part in enumerate(parts):
        part.cache.import_(kc[:, p::2], vc[:, p::2])
        assert len(part.cache) == plan(2 * KV, p, H, KV).local_rows(L0)
    dev = torch.device("cuda:0")
    stream = torch.cuda.current_stream().cuda_stream
    gathered = torch.zeros(2, H * hd + H, device=dev)
    merged = torch.empty(H * hd, device=dev)
    for step in range(5):
        pos = L0 + step
        q, k, v = qkv(rng, shape, 1)
        ref = o.attend_cached(q, k, v, threads=8)[0]
        tq, tk, tv = (torch.from_numpy(x).to(dev) for x in (q, k, v))
        for p, part in enumerate(parts):
            ctx.set_lse_out(gathered[p, H * hd:].data_ptr())
            part.forward_cached_dev_at(tq.data_ptr(), tk.data_ptr(), tv.data_ptr(), gathered[p].data_ptr(), pos,
                                       append=(pos % 2 == p), stream=stream)
        ctx.set_lse_out(None)
        ctx.merge_parts(gathered.data_ptr(), 2, 2, H, hd, merged.data_ptr(), stream)
        torch.cuda.synchronize()
        ctx.sync()
        assert rel_err(merged.cpu().numpy(), ref) <= DECODE_TOL, step
    assert len(parts[0].cache) + len(parts[1].cache) == L0 + 5
    for part in parts:
        part.close()


def test_uncached_full_sequence_relation(ctx):
    """spec/rope_kv_cache_spec.cr:30-59 on the GPU: the reference's uncached forward
    (attention_full_cpu + causal_attention!, llama_block.cr:209-243, 696-716: dense S x S
    scores through f64-accumulating matmuls) and its cached path agree within 1e-3.  Here
    the cached side is the library on an empty cache with T = S (exact-fp32 kernel), the
    uncached side is the oracle's restatement of attention_full_cpu."""
    import shainet_b200 as S
    rng = np.random.default_rng(59)
    for shape, T, dist in ((dict(H=4, KV=4, hd=4, theta=10000.0), 4, "uniform"),      # the tiny-llama fixture's heads
                           (dict(H=8, KV=4, hd=8, theta=10000.0), 9, "uniform"),      # the GQA spec shape
                           (dict(H=8, KV=2, hd=64, theta=500000.0), 150, "normal")):
        o, g = make_pair(ctx, shape, rng)
        q, k, v = qkv(rng, shape, T, dist)
        full = o.attend_full(q, k, v)
        got = g.forward_cached(q, k, v, S.F_GENERIC)
        assert np.abs(got - full).max() < SPEC_ABS_TOL
        assert rel_err(got, full) < SPEC_ABS_TOL
        # prefill of T-1 rows, then one decode row: the last row equals the uncached last row (the spec's assertion)
        g.clear_cache()
        g.forward_cached(q[:-1], k[:-1], v[:-1], S.F_GENERIC)
        last = g.forward_cached(q[-1:], k[-1:], v[-1:])
        assert np.abs(last[0] - full[-1]).max() < SPEC_ABS_TOL
        g.close()


def test_rope_known_answers_in_the_appended_rows(ctx):
    """spec/rope_kv_cache_spec.cr:5-26 against the rows the norm/RoPE/append kernel writes:
    position 0 is the identity (1e-5); the unit vector (1,0,0,0) at position 1 with head_dim 4
    becomes (cos 1, 0, sin 1, 0) (1e-4, half-split pairing).  RoPE.apply itself
    (rope.cr:7-33, all-f64) agrees with the stored fp32 rows to 1e-5 on random rows."""
    from oracle import oracle as O
    import shainet_b200 as S
    rng = np.random.default_rng(26)
    # identity at position 0, 8-wide row
    g = S.LlamaAttention(ctx, 1, 1, 8, 10000.0)
    row = np.arange(1, 9, dtype=np.float32).reshape(1, 8)
    g.forward_cached(row, row, row)
    kc, _ = g.cache.export()
    assert np.abs(kc[0, 0] - row[0]).max() < 1e-5
    g.close()
    # unit vector at position 1, head_dim 4
    g = S.LlamaAttention(ctx, 1, 1, 4, 10000.0)
    x = np.zeros((2, 4), np.float32)
    x[:, 0] = 1.0
    g.forward_cached(x, x, x)
    kc, _ = g.cache.export()
    assert np.abs(kc[0, 1] - np.array([np.cos(1.0), 0.0, np.sin(1.0), 0.0])).max() < 1e-4
    g.close()
    # random rows, both append kernels (T > 1, and the fused decode prologue at T = 1), against RoPE.apply
    for hd, theta in ((64, 10000.0), (128, 1e6)):
        g = S.LlamaAttention(ctx, 2, 1, hd, theta)
        x = rng.standard_normal((40, hd)).astype(np.float32)
        qd = np.concatenate([x, x], axis=1)
        g.forward_cached(qd[:39], x[:39], x[:39])
        g.forward_cached(qd[39:], x[39:], x[39:])
        kc, _ = g.cache.export()
        ref = O.rope_apply(x, 0, theta)
        assert np.abs(kc[0] - ref).max() <= 1e-5 * max(1.0, np.abs(ref).max())
        g.close()


def test_truncate_then_inputs_ready_does_not_race_with_the_previous_launch(ctx):
    """Roll-back of speculative rows (kv_truncate) followed at once by a launch that declares its inputs
    ready: the new launch rewrites a row the still-running previous launch reads, so the library drops the
    declaration for that one launch.  Queued back to back on one stream, checked against the oracle."""
    import torch
    import shainet_b200 as S
    rng = np.random.default_rng(909)
    o, g = make_pair(ctx, Q30, rng)
    q, k, v = qkv(rng, Q30, 4500)
    o.attend_cached(q, k, v, threads=8)
    kc, vc = o.export_cache()
    g.cache.import_(kc, vc)
    g.cache.reserve(4700)
    dev = torch.device("cuda:0")
    stream = torch.cuda.current_stream().cuda_stream
    ins = [qkv(rng, Q30, 1) for _ in range(12)]
    dins = [tuple(torch.from_numpy(x).to(dev) for x in trip) for trip in ins]
    outs = [torch.empty(1, Q30["H"] * Q30["hd"], device=dev) for _ in ins]
    torch.cuda.synchronize()
    plan = [0, 1, 2, 3, "back2", 4, 5, "back1", 6, 7, 8, "back3", 9, 10, 11]
    for step in plan:
        if isinstance(step, str):
            g.cache.truncate(g.cache_len - int(step[-1]))
            continue
        tq, tk, tv = dins[step]
        g.forward_cached_dev(tq.data_ptr(), tk.data_ptr(), tv.data_ptr(), outs[step].data_ptr(), 1, stream, S.F_INPUTS_READY)
    torch.cuda.synchronize()
    ctx.sync()
    for step in plan:
        if isinstance(step, str):
            kc, vc = o.export_cache()
            n = o.cache_len - int(step[-1])
            o.import_cache(kc[:, :n], vc[:, :n])
            continue
        ref = o.attend_cached(*ins[step])
        assert rel_err(outs[step].cpu().numpy(), ref) <= DECODE_TOL, step
    assert g.cache_len == o.cache_len
    g.close()
