"""Pins the CPU oracle to what the reference's own specs assert for this path."""
import math
import os

import numpy as np
import pytest

from oracle import oracle as O

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def test_rope_identity_at_position_zero():
    # spec/rope_kv_cache_spec.cr:5-10
    m = np.arange(1, 9, dtype=np.float32)[None, :]
    out = O.rope_apply(m, 0, 10000.0)
    assert np.allclose(out, m, atol=1e-5)


def test_rope_half_split_pairing():
    # spec/rope_kv_cache_spec.cr:12-26 — head_dim 4, position 1, unit vector
    m = np.array([[1.0, 0.0, 0.0, 0.0]], np.float32)
    out = O.rope_apply(m, 1, 10000.0)
    assert abs(out[0, 0] - math.cos(1.0)) < 1e-4
    assert abs(out[0, 2] - math.sin(1.0)) < 1e-4
    assert out[0, 1] == 0.0 and out[0, 3] == 0.0


def test_block_rope_matches_module_rope():
    # LlamaBlock's private fp32 rotation (llama_block.cr:678-693) and the f64
    # RoPE module (rope.cr:7-33) describe the same rotation.
    rng = np.random.default_rng(0)
    hd, S = 8, 5
    a = O.OracleAttention(1, 1, hd, 10000.0)
    k = rng.standard_normal((S, hd)).astype(np.float32)
    a.attend_cached(np.zeros((S, hd), np.float32), k, k)
    kc, _ = a.export_cache()
    assert np.allclose(kc[0], O.rope_apply(k, 0, 10000.0), atol=2e-6)


def _tiny_llama():
    z = np.load(os.path.join(GOLDEN, "tiny_llama_slice.npz"))
    d, H, KV = int(z["hidden_size"]), int(z["num_heads"]), int(z["num_kv_heads"])
    blocks = []
    for l in range(int(z["num_layers"])):
        w = {k: z[f"l{l}.{k}"] for k in ("w_q", "w_k", "w_v", "w_o", "gate", "up", "down", "norm1", "norm2")}
        blocks.append(O.OracleLlamaBlock(d, H, KV, d // H, float(z["eps"]), float(z["rope_theta"]), w))
    return z["embed_rows"], blocks


def test_tiny_llama_cache_consistency():
    # spec/rope_kv_cache_spec.cr:30-59: uncached forward of tokens [1,42,100,7]
    # vs prefill of 3 + one cached step; last rows agree within 1e-3.
    emb, blocks = _tiny_llama()
    full = emb.copy()
    for b in blocks:
        full = b.forward(full)
    for b in blocks:
        b.clear_cache()
    pre = emb[:3].copy()
    for b in blocks:
        pre = b.forward_cached(pre)
    inc = emb[3:4].copy()
    for b in blocks:
        inc = b.forward_cached(inc)
    assert np.all(np.isfinite(inc)) and np.abs(inc).max() > 0
    assert np.abs(inc[0] - full[-1]).max() < 1e-3
    # the oracle is far inside the spec's tolerance
    assert np.abs(inc[0] - full[-1]).max() < 1e-5


def test_cached_equals_uncached_gqa():
    # Shapes of spec/llama_attention_gpu_spec.cr:17-66: 8 heads / 4 KV heads, head_dim 8
    rng = np.random.default_rng(42)
    H, KV, hd = 8, 4, 8
    q = rng.uniform(-1, 1, (9, H * hd)).astype(np.float32)
    k = rng.uniform(-1, 1, (9, KV * hd)).astype(np.float32)
    v = rng.uniform(-1, 1, (9, KV * hd)).astype(np.float32)
    a = O.OracleAttention(H, KV, hd)
    full = a.attend_full(q, k, v)
    outs = [a.attend_cached(q[:6], k[:6], v[:6])]
    for t in range(6, 9):
        outs.append(a.attend_cached(q[t:t + 1], k[t:t + 1], v[t:t + 1]))
    assert np.abs(np.concatenate(outs) - full).max() < 1e-5
    assert a.cache_len == 9


def test_nil_bias_equals_zero_bias():
    # spec/llama_qkv_bias_spec.cr:8-40 (1e-6) and :42-72 (a real bias moves the output)
    rng = np.random.default_rng(3)
    H, KV, hd, T = 4, 2, 8, 5
    q = rng.standard_normal((T, H * hd)).astype(np.float32)
    k = rng.standard_normal((T, KV * hd)).astype(np.float32)
    v = rng.standard_normal((T, KV * hd)).astype(np.float32)
    a = O.OracleAttention(H, KV, hd).attend_cached(q, k, v)
    z = O.OracleAttention(H, KV, hd, b_q=np.zeros(H * hd), b_k=np.zeros(KV * hd), b_v=np.zeros(KV * hd)).attend_cached(q, k, v)
    assert np.abs(a - z).max() <= 1e-6
    nz = O.OracleAttention(H, KV, hd, b_q=np.full(H * hd, 0.5), b_k=np.full(KV * hd, -0.3),
                           b_v=np.full(KV * hd, 0.2)).attend_cached(q, k, v)
    assert np.abs(a - nz).sum() > 0.01


def test_clear_cache_and_growth_replay():
    # spec/llama_attention_gpu_spec.cr:68-104: 290-token prefill + 10 steps, twice after clear
    rng = np.random.default_rng(7)
    H, KV, hd = 4, 2, 8
    a = O.OracleAttention(H, KV, hd)
    seq = [(rng.uniform(-1, 1, (n, H * hd)), rng.uniform(-1, 1, (n, KV * hd)), rng.uniform(-1, 1, (n, KV * hd)))
           for n in [290] + [1] * 10]
    first = [a.attend_cached(*s) for s in seq]
    assert a.cache_len == 300
    a.clear_cache()
    assert a.cache_len == 0
    second = [a.attend_cached(*s) for s in seq]
    for x, y in zip(first, second):
        assert np.array_equal(x, y)


def test_threads_do_not_change_results():
    rng = np.random.default_rng(5)
    H, KV, hd, T = 8, 2, 16, 33
    q = rng.standard_normal((T, H * hd)); k = rng.standard_normal((T, KV * hd)); v = rng.standard_normal((T, KV * hd))
    x = O.OracleAttention(H, KV, hd).attend_cached(q, k, v, threads=1)
    y = O.OracleAttention(H, KV, hd).attend_cached(q, k, v, threads=4)
    assert np.array_equal(x, y)


def test_f64_truth_close_to_fp32_path():
    rng = np.random.default_rng(11)
    H, KV, hd, L = 8, 2, 64, 2048
    kc = rng.standard_normal((KV, L, hd)).astype(np.float32)
    vc = rng.standard_normal((KV, L, hd)).astype(np.float32)
    a = O.OracleAttention(H, KV, hd, 500000.0)
    a.import_cache(kc, vc)
    q = rng.standard_normal((1, H * hd)).astype(np.float32)
    x = a.attend_only(q, L - 1, mode=0)
    y = a.attend_only(q, L - 1, mode=1)
    assert np.abs(x - y).max() / np.abs(y).max() < 1e-5


def test_qk_norm_formula():
    # llama_block.cr:615-641: v * f32(1/sqrt(f64(ss/hd)+eps)) * w, before RoPE
    rng = np.random.default_rng(13)
    hd = 16
    w = (1 + 0.02 * rng.standard_normal(hd)).astype(np.float32)
    k = rng.standard_normal((1, hd)).astype(np.float32)
    a = O.OracleAttention(1, 1, hd, 1e6, 1e-6, q_norm=w, k_norm=w)
    a.attend_cached(k, k, k)
    kc, vc = a.export_cache()
    ss = np.float32(0)
    for d in range(hd):
        ss = np.float32(ss + np.float32(k[0, d] * k[0, d]))
    inv = np.float32(1.0 / math.sqrt(float(np.float32(ss / np.float32(hd))) + 1e-6))
    expect = (k[0] * inv) * w          # position 0: rotation is the identity
    assert np.array_equal(kc[0, 0], expect.astype(np.float32))
    assert np.array_equal(vc[0, 0], k[0])  # V is neither normalised nor rotated


def test_llama3_scaled_freqs():
    # hf_loader.cr:235-265 with Llama-3.2 parameters
    hd, theta = 64, 500000.0
    f = O.llama3_rope_freqs(theta, hd, 32.0, 1.0, 4.0, 8192.0)
    base = np.array([1.0 / theta ** (2.0 * i / hd) for i in range(hd // 2)])
    assert f[0] == np.float32(base[0])                       # short wavelengths untouched
    assert np.isclose(f[-1], base[-1] / 32.0, rtol=1e-6)     # long wavelengths divided by factor
    assert np.all(np.diff(f) < 0)
    a = O.OracleAttention(4, 2, hd, theta, rope_freqs=f)
    assert np.array_equal(a.inv_freq(), f)


def test_bad_head_split_rejected():
    # llama_block.cr:80
    with pytest.raises(ValueError):
        O.OracleAttention(6, 4, 8)


# ---- Q8_0 weights and the host steps around the projections ----

def test_q8_quantiser_known_answers():
    """quantized_cuda_matrix.cr:84-110 on cases worked by hand: scale = max|w|/127 per block of 32
    inputs of one output, the extreme maps to +-127, an all-zero block gets scale 1, a ragged last
    block (K = 40) is its own block, halves round to even."""
    K, N = 40, 2
    w = np.zeros((K, N), np.float32)
    w[:32, 0] = np.linspace(-1.27, 1.27, 32, dtype=np.float32)      # block 0 of output 0: max 1.27 -> scale 0.01
    w[32:, 0] = 0.0                                                 # ragged block 1 of output 0: all zero
    w[0, 1], w[1, 1], w[2, 1] = 127.0, 0.5, 1.5                     # output 1, scale 1: ties 0.5 -> 0, 1.5 -> 2
    w[39, 1] = -3.0                                                 # ragged block of output 1: scale 3/127
    W = O.OracleQ8(w)
    assert W.q.shape == (2, 40) and W.scales.shape == (2, 2)
    assert W.scales[0, 0] == np.float32(np.float32(1.27) / np.float32(127.0)) and W.scales[0, 1] == 1.0
    assert W.q[0, 0] == -127 and W.q[0, 31] == 127 and not W.q[0, 32:].any()
    assert W.scales[1, 0] == 1.0 and list(W.q[1, :3]) == [127, 0, 2]
    assert W.scales[1, 1] == np.float32(np.float32(3.0) / np.float32(127.0)) and W.q[1, 39] == -127
    assert np.abs(W.dequantised() - w).max() <= 0.5 * W.scales.max() + 1e-7


def test_q8_gemv_follows_the_dequantised_product():
    rng = np.random.default_rng(8)
    K, N, M = 2048, 96, 3
    W = O.OracleQ8((0.02 * rng.standard_normal((K, N))).astype(np.float32))
    x = rng.standard_normal((M, K)).astype(np.float32)
    truth = x.astype(np.float64) @ W.dequantised().astype(np.float64)
    for fused in (0, 1):
        y = W.gemv(x, fused=fused, threads=2)
        assert np.abs(y - truth).max() <= 2e-6 * np.abs(truth).max()
    assert np.abs(W.gemv(x, fused=0) - W.gemv(x, fused=1)).max() <= 1e-6 * np.abs(truth).max()


def test_swiglu_activation_bias_and_greedy():
    rng = np.random.default_rng(9)
    g = rng.standard_normal(500).astype(np.float32) * 4
    u = rng.standard_normal(500).astype(np.float32)
    ref = ((g.astype(np.float64) / (1.0 + np.exp(-g.astype(np.float64)))) * u.astype(np.float64)).astype(np.float32)
    assert np.array_equal(O.swiglu_act(g, u), ref)
    # Sampler.greedy (sampler.cr:38-53): first index of the largest finite value; 0 if there is none
    assert O.greedy(np.array([1.0, 5.0, 5.0, np.inf, np.nan, -2.0], np.float32)) == 1
    assert O.greedy(np.array([np.nan, np.inf, -np.inf], np.float32)) == 0
    assert O.greedy(np.array([-3.0, -1.0, -2.0], np.float32)) == 1


def test_bf16_row_rounding_mode_is_the_plain_oracle_over_rounded_rows():
    """kv_rounding="bf16" (the library's opt-in cache format restated; not a reference behaviour):
    rounding is to nearest even, bit-identical to torch's, and attention in that mode equals the
    unrounded oracle attending over the rounded rows."""
    import torch
    from oracle import oracle as O
    rng = np.random.default_rng(31)
    x = (rng.standard_normal(200000) * 4).astype(np.float32)
    x[:3] = [1.00390625, 1.01171875, -1.00390625]
    r = O.round_bf16(x)
    assert np.array_equal(r, torch.from_numpy(x).to(torch.bfloat16).float().numpy())
    assert list(r[:3]) == [1.0, 1.015625, -1.0]
    H, KV, hd = 8, 2, 32
    qn = (1 + 0.02 * rng.standard_normal(hd)).astype(np.float32)
    a = O.OracleAttention(H, KV, hd, 10000.0, 1e-6, q_norm=qn, k_norm=qn, kv_rounding="bf16")
    b = O.OracleAttention(H, KV, hd, 10000.0, 1e-6, q_norm=qn, k_norm=qn)
    f = lambda *s: rng.standard_normal(s).astype(np.float32)
    q, k, v = f(40, H * hd), f(40, KV * hd), f(40, KV * hd)
    a.attend_cached(q, k, v)
    b.attend_cached(q, k, v)
    ka, va = a.export_cache(); kb, vb = b.export_cache()
    assert np.array_equal(ka, O.round_bf16(kb)) and np.array_equal(va, O.round_bf16(vb))
    q1, k1, v1 = f(1, H * hd), f(1, KV * hd), f(1, KV * hd)
    ya = a.attend_cached(q1, k1, v1)
    ka, va = a.export_cache()
    # mode 1 restarted from its own (representable) rows reproduces the step bit for bit; mode 0 from the
    # same rows differs only through the new token's unrounded row
    d = O.OracleAttention(H, KV, hd, 10000.0, 1e-6, q_norm=qn, k_norm=qn)
    d.import_cache(ka[:, :40], va[:, :40])
    e = O.OracleAttention(H, KV, hd, 10000.0, 1e-6, q_norm=qn, k_norm=qn, kv_rounding="bf16")
    e.import_cache(ka[:, :40], va[:, :40])
    assert np.array_equal(e.export_cache()[0], ka[:, :40])             # importing representable rows changes nothing
    yd = d.attend_cached(q1, k1, v1)
    ye = e.attend_cached(q1, k1, v1)
    assert np.array_equal(ya, ye)
    kd = d.export_cache()[0]
    assert np.array_equal(O.round_bf16(kd[:, 40]), ka[:, 40])
    assert not np.array_equal(yd, ye) and np.abs(yd - ye).max() < 0.05  # rounding the new row is visible, and small
