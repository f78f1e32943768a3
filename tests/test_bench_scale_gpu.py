"""Parity at the sizes the benchmark times, on ONE kv-head group so that the CPU
oracle finishes in about a minute: the 8192-token causal prefill of the
Qwen3-8B attention shape (128 K/V tiles per row tile, every accumulator-rescale
and barrier phase the full configuration goes through), the same prefill as two
4096-token chunks (second chunk over an existing cache), and lock-step batched
decode of 64 ragged sequences with context lengths log-uniform in [1k, 32k].
A kv-head group (one K/V head and its G query heads) is independent of every
other group in all kernels, so one group exercises the per-CTA work of the
full shape.

Tolerances: TF32 prefill max|y-ref|/max|ref| <= 2e-3 and <= 8e-3 per row against
the row's own scale; fp32 decode <= 1e-5."""
import numpy as np
import pytest

from helpers import DECODE_TOL, make_pair, norm_weights, qkv, rel_err

pytestmark = pytest.mark.gpu

PREFILL_TOL = 2e-3
Q8B_GROUP = dict(H=4, KV=1, hd=128, theta=1e6, qk_norm=True)   # one kv group of Qwen3-8B attention


@pytest.fixture(scope="module")
def ctx():
    import shainet_b200 as S
    from shainet_b200 import build
    build.build()
    c = S.AttnContext(0)
    yield c
    c.close()


def _threads():
    from oracle import oracle as O
    return max(1, O.max_threads())


@pytest.mark.parametrize("chunks", [(8192,), (4096, 4096)], ids=["one_call_8192", "two_chunks_4096"])
def test_prefill_at_the_benchmarked_length(ctx, chunks):
    """attention_heads_cpu (llama_block.cr:302-401) over 8192 positions against the
    tcgen05 kernel, default dispatch (what the bench's prefill block runs)."""
    rng = np.random.default_rng(3001)
    o, g = make_pair(ctx, Q8B_GROUP, rng)
    for T in chunks:
        q, k, v = qkv(rng, Q8B_GROUP, T)
        ref = o.attend_cached(q, k, v, threads=_threads())
        got = g.forward_cached(q, k, v)
        e = rel_err(got, ref)
        assert e <= PREFILL_TOL, (T, e)
        per_row = np.abs(got - ref).max(axis=1) / np.abs(ref).max(axis=1)
        assert per_row.max() <= 4 * PREFILL_TOL, (T, float(per_row.max()), int(per_row.argmax()))
    assert g.cache_len == 8192 == o.cache_len
    # the cache the prefill left is fp32 work: V exact, K within a sincosf ulp
    ko, vo = o.export_cache(); kg, vg = g.cache.export()
    assert np.array_equal(vo, vg) and np.abs(ko - kg).max() <= 4e-7 * np.abs(ko).max()
    q, k, v = qkv(rng, Q8B_GROUP, 1)
    assert rel_err(g.forward_cached(q, k, v), o.attend_cached(q, k, v, threads=_threads())) <= DECODE_TOL
    g.close()


@pytest.mark.parametrize("kv_format", ["f32", "bf16"])
def test_batched_ragged_decode_at_the_benchmarked_batch(ctx, kv_format):
    """64 sequences, lengths floor(exp(U(ln 1024, ln 32768))) from seed 4001 (the
    benchmark's draw), caches N(0,1), two lock-step steps against 64 oracles; also with the
    opt-in bfloat16 rows (24-row warp tiles in the batched launch) against oracles that round
    their rows the same way."""
    import torch
    import shainet_b200 as S
    from oracle import oracle as O
    shape = Q8B_GROUP
    H, KV, hd = shape["H"], shape["KV"], shape["hd"]
    rng = np.random.default_rng(4001)
    B = 64
    lens = np.exp(rng.uniform(np.log(1024), np.log(32768), B)).astype(np.int64)
    assert lens.min() >= 1024 and lens.max() < 32768
    qn, kn = norm_weights(rng, hd), norm_weights(rng, hd)
    oracles, caches = [], []
    for b in range(B):
        L = int(lens[b])
        kc = rng.standard_normal((KV, L, hd), dtype=np.float32)
        vc = rng.standard_normal((KV, L, hd), dtype=np.float32)
        o = O.OracleAttention(H, KV, hd, shape["theta"], 1e-6, q_norm=qn, k_norm=kn,
                              kv_rounding="bf16" if kv_format == "bf16" else None)
        o.import_cache(kc, vc)
        g = S.LlamaAttention(ctx, H, KV, hd, shape["theta"], 1e-6, q_norm=qn, k_norm=kn, kv_format=kv_format)
        g.cache.import_(kc, vc)
        g.cache.reserve(L + 4)
        oracles.append(o); caches.append(g)
    dev = torch.device("cuda:0")
    stream = torch.cuda.current_stream().cuda_stream
    worst = 0.0
    for step in range(2):
        q, k, v = qkv(rng, shape, B)
        tq, tk, tv = (torch.from_numpy(x).to(dev) for x in (q, k, v))
        out = torch.full_like(tq, float("nan"))
        S.forward_batched_dev(ctx, [g.cache for g in caches], tq.data_ptr(), tk.data_ptr(), tv.data_ptr(), out.data_ptr(),
                              caches[0].scale, stream)
        torch.cuda.synchronize()
        ctx.sync()
        got = out.cpu().numpy()
        for b, o in enumerate(oracles):
            ref = o.attend_cached(q[b:b + 1], k[b:b + 1], v[b:b + 1], threads=_threads())
            e = rel_err(got[b:b + 1], ref)
            worst = max(worst, e)
            assert e <= DECODE_TOL, (step, b, int(lens[b]), e)
    for b, g in enumerate(caches):
        assert g.cache_len == int(lens[b]) + 2
        g.close()
    assert worst > 0.0   # the two sides are different arithmetic, not the same code
