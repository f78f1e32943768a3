"""Q8_0 projections, the whole decoder block and the token loop on the device, through the
C ABI, against the CPU oracle (the reference's host arithmetic for RMSNorm / residual /
SwiGLU / bias / greedy, and its gemm_q8_f32 kernel's reduction order for the GEMVs) and
against the reference's own CUDA kernel compiled unmodified.

Tolerances: one GEMV max|y-ref|/max|ref| <= 1e-5 (the decode tolerance: the kernels sum in
a different order than the reference's 256 strided partials + tree); a whole block output
<= 3e-5 and last-row logits after two blocks <= 1e-4, the single-operation tolerance
compounded over the ten operations of a block; greedy tokens equal, judged by the
oracle's top-2 margin where they could differ."""
import ctypes as C

import numpy as np
import pytest

from helpers import DECODE_TOL, rel_err

pytestmark = pytest.mark.gpu

BLOCK_TOL = 3e-5
LOGIT_TOL = 1e-4


@pytest.fixture(scope="module")
def ctx():
    import shainet_b200 as S
    from shainet_b200 import build
    build.build()
    c = S.AttnContext(0)
    yield c
    c.close()


def _w(rng, K, N):
    return (0.02 * rng.standard_normal((K, N))).astype(np.float32)


def test_quantiser_matches_the_reference_algorithm_bit_for_bit(ctx):
    """from_simple (quantized_cuda_matrix.cr:74-115): int8 values and scales of the library's
    host quantiser equal the oracle's restatement, including a ragged last block, zero blocks
    and values at the clamp."""
    import shainet_b200 as S
    from oracle import oracle as O
    rng = np.random.default_rng(70)
    for K, N in ((2048, 64), (40, 7), (96, 33)):
        w = _w(rng, K, N)
        w[:32, 0] = 0.0
        w[5, 1] = 3.0
        ref = O.OracleQ8(w)
        W = S.Q8Weight.from_simple(ctx, w)
        q, s = W.export()
        assert np.array_equal(q, ref.q) and np.array_equal(s, ref.scales)
        W.close()


@pytest.mark.parametrize("K,N,M", [(2048, 2048, 1), (2048, 512, 1), (2048, 3072, 1), (8192, 2048, 1), (2048, 8192, 1),
                                   (4096, 4096, 1), (2048, 1001, 1), (2048, 512, 2), (2048, 640, 5), (2048, 256, 9),
                                   (96, 33, 3), (40, 7, 1), (4128, 64, 2)],
                         ids=lambda v: str(v))
def test_gemv_against_the_reference_kernels_arithmetic(ctx, K, N, M):
    """gemv_into (quantized_cuda_matrix.cr:143-153) = gemm_q8_f32_kernel (cuda_kernels.cu:581-614).
    LLaMA-3.2-1B's projection shapes, the stacked q|k|v, the FFN shapes, odd N, several rows
    (row tiles of 2 and 4 with a ragged last tile), and shapes outside the tuned path
    (K not a multiple of 2048, a ragged last scale block)."""
    import torch
    import shainet_b200 as S
    from oracle import oracle as O
    rng = np.random.default_rng(K * 7 + N + M)
    ref_w = O.OracleQ8(_w(rng, K, N))
    W = S.Q8Weight.from_quantized(ctx, ref_w.q, ref_w.scales)
    x = rng.standard_normal((M, K)).astype(np.float32)
    ref = ref_w.gemv(x)
    dev = torch.device("cuda:0")
    tx = torch.from_numpy(x).to(dev)
    ty = torch.full((M, N), float("nan"), device=dev)
    W.gemv_dev(tx.data_ptr(), ty.data_ptr(), M, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    ctx.sync()
    got = ty.cpu().numpy()
    assert np.isfinite(got).all()
    assert rel_err(got, ref) <= DECODE_TOL, rel_err(got, ref)
    # and against an f64 product with the dequantised weight
    truth = x.astype(np.float64) @ ref_w.dequantised().astype(np.float64)
    assert rel_err(got, truth) <= max(DECODE_TOL, rel_err(ref, truth))
    W.close()


def test_symbol_compatible_gemm_q8_f32_against_the_reference_kernel():
    """The reference's own gemm_q8_f32 (compiled unmodified from its CUDA file) and the library's
    symbol of the same name on the same device buffers; the oracle's restatement of the
    reference kernel's order is pinned by the same run (exact, or within 1e-6)."""
    import torch
    from oracle import build_oracle, oracle as O
    from shainet_b200 import _lib, build
    build.build()
    ref_so = build_oracle.build_reference_kernels()
    if ref_so is None:
        pytest.skip("the reference's CUDA kernels have not been built")
    ref_lib = C.CDLL(ref_so)
    ref_lib.gemm_q8_f32.argtypes = [C.c_void_p] * 4 + [C.c_int] * 3
    ref_lib.gemm_q8_f32.restype = None
    lib = _lib.load()
    dev = torch.device("cuda:0")
    rng = np.random.default_rng(616)
    for K, N, M in ((2048, 2048, 1), (2048, 512, 3), (96, 33, 2)):
        w = O.OracleQ8(_w(rng, K, N))
        x = rng.standard_normal((M, K)).astype(np.float32)
        tq = torch.from_numpy(w.q).to(dev)
        ts = torch.from_numpy(w.scales).to(dev)
        tx = torch.from_numpy(x).to(dev)
        y_ref = torch.zeros(M, N, device=dev)
        y_lib = torch.zeros(M, N, device=dev)
        torch.cuda.synchronize()
        ref_lib.gemm_q8_f32(tx.data_ptr(), tq.data_ptr(), ts.data_ptr(), y_ref.data_ptr(), M, N, K)
        lib.gemm_q8_f32(tx.data_ptr(), tq.data_ptr(), ts.data_ptr(), y_lib.data_ptr(), M, N, K)
        torch.cuda.synchronize()
        a, b = y_ref.cpu().numpy(), y_lib.cpu().numpy()
        assert rel_err(b, a) <= DECODE_TOL, rel_err(b, a)
        o_fused, o_plain = w.gemv(x, fused=1), w.gemv(x, fused=0)
        e = min(rel_err(o_fused, a), rel_err(o_plain, a))
        print(f"  gemm_q8_f32 {M}x{K}x{N}: oracle vs reference kernel {rel_err(o_fused, a):.2e} (fused) "
              f"{rel_err(o_plain, a):.2e} (unfused); library vs reference kernel {rel_err(b, a):.2e}")
        assert e <= 1e-6, e


def _make_block(ctx, rng, d, H, KV, hd, ffn, theta, eps, qk_norm=False, kv_format="f32"):
    """The same random block on both sides: (oracle block, library block, things to close)."""
    import shainet_b200 as S
    from oracle import oracle as O
    kw = {}
    if qk_norm:
        kw = dict(q_norm=(1 + 0.02 * rng.standard_normal(hd)).astype(np.float32),
                  k_norm=(1 + 0.02 * rng.standard_normal(hd)).astype(np.float32))
    norm1 = (1 + 0.05 * rng.standard_normal(d)).astype(np.float32)
    norm2 = (1 + 0.05 * rng.standard_normal(d)).astype(np.float32)
    shapes = dict(wq=(d, H * hd), wk=(d, KV * hd), wv=(d, KV * hd), wo=(H * hd, d))
    if ffn:
        shapes.update(gate=(d, ffn), up=(d, ffn), down=(ffn, d))
    ow = {k: O.OracleQ8(_w(rng, *s)) for k, s in shapes.items()}
    gw = {k: S.Q8Weight.from_quantized(ctx, w.q, w.scales) for k, w in ow.items()}
    oa = O.OracleAttention(H, KV, hd, theta, eps, kv_rounding="bf16" if kv_format == "bf16" else None, **kw)
    ga = S.LlamaAttention(ctx, H, KV, hd, theta, eps, kv_format=kv_format, **kw)
    ob = O.OracleQ8Block(oa, eps, norm1, ow["wq"], ow["wk"], ow["wv"], ow["wo"], norm2 if ffn else None,
                         ow.get("gate"), ow.get("up"), ow.get("down"))
    gb = S.LlamaBlock(ctx, ga, d, eps, norm1, gw["wq"], gw["wk"], gw["wv"], gw["wo"], norm2 if ffn else None,
                      gw.get("gate"), gw.get("up"), gw.get("down"))
    return ob, gb, [gb, ga] + list(gw.values())


@pytest.mark.parametrize("name,d,H,KV,hd,ffn,theta,eps,qk_norm",
                         [("llama1b", 2048, 32, 8, 64, 8192, 5e5, 1e-5, False),
                          ("qwen3_attention_only", 2048, 32, 4, 128, 0, 1e6, 1e-6, True),
                          ("tiny_generic_kernels", 96, 4, 2, 8, 160, 1e4, 1e-6, False)],
                         ids=lambda v: v if isinstance(v, str) else "")
def test_block_forward_cached_against_the_oracle(ctx, name, d, H, KV, hd, ffn, theta, eps, qk_norm):
    """LlamaBlock#forward_cached (llama_block.cr:189-196): a short prefill (several rows through
    the row-tiled GEMVs), then single-token steps through the one-launch q|k|v path and the
    fused decode kernel.  The second case is a block without FFN (it stays with the caller)."""
    rng = np.random.default_rng(1896)
    ob, gb, owned = _make_block(ctx, rng, d, H, KV, hd, ffn, theta, eps, qk_norm)
    for T in (5, 1, 1, 1):
        x = rng.standard_normal((T, d)).astype(np.float32)
        ref = ob.forward_cached(x)
        got = gb.forward_cached(x)
        e = rel_err(got, ref)
        assert e <= BLOCK_TOL, (name, T, e)
    assert gb.attn.cache_len == 8 == ob.attn.cache_len
    for o in owned:
        o.close()


def test_block_over_a_bf16_cache(ctx):
    """The same chain with the opt-in bfloat16 KV cache: the block's attention reads 16-bit rows (fp32
    image for the prefill rows, the fused kernel directly for single tokens); the oracle rounds its
    cache rows the same way."""
    rng = np.random.default_rng(1897)
    ob, gb, owned = _make_block(ctx, rng, 2048, 32, 8, 64, 8192, 5e5, 1e-5, False, kv_format="bf16")
    for T in (40, 1, 1, 1):
        x = rng.standard_normal((T, 2048)).astype(np.float32)
        e = rel_err(gb.forward_cached(x), ob.forward_cached(x))
        assert e <= BLOCK_TOL, (T, e)
    for o in owned:
        o.close()


def test_decoder_run_and_generate_against_the_oracle(ctx):
    """Network#run(Array(Int32)) + Sampler.greedy: two LLaMA-1B-width blocks, vocabulary 3001 (odd,
    so the last column pair is half empty), lm_head bias, final norm.  Logits of the prompt and of
    single-token calls against the oracle; then generate(): the greedy tokens of the device loop
    (no host round trip between steps) equal the oracle's."""
    import shainet_b200 as S
    from oracle import oracle as O
    rng = np.random.default_rng(2001)
    d, H, KV, hd, ffn, theta, eps, vocab, layers = 2048, 32, 8, 64, 4096, 5e5, 1e-5, 3001, 2
    pairs = [_make_block(ctx, rng, d, H, KV, hd, ffn, theta, eps) for _ in range(layers)]
    emb = _w(rng, vocab, d)
    final_norm = (1 + 0.05 * rng.standard_normal(d)).astype(np.float32)
    bias = (0.01 * rng.standard_normal(vocab)).astype(np.float32)
    o_head = O.OracleQ8(emb.T.copy())
    g_head = S.Q8Weight.from_quantized(ctx, o_head.q, o_head.scales)
    odec = O.OracleQ8Decoder(emb, [p[0] for p in pairs], final_norm, o_head, bias, eps)
    gdec = S.Decoder(ctx, [p[1] for p in pairs], emb, final_norm, g_head, bias, eps)
    prompt = rng.integers(0, vocab, 6)
    ref_logits, ref_tok = odec.run(prompt)
    got_logits, got_tok = gdec.run(prompt)
    assert rel_err(got_logits, ref_logits) <= LOGIT_TOL, rel_err(got_logits, ref_logits)
    assert got_tok == int(np.argmax(got_logits))
    for _ in range(3):
        fed = ref_tok                     # both sides are fed the oracle's token
        ref_logits, ref_tok = odec.run([fed])
        got_logits, got_tok2 = gdec.run([fed])
        assert rel_err(got_logits, ref_logits) <= LOGIT_TOL
        assert got_tok2 == int(np.argmax(got_logits))
    # generate from a fresh state on both sides
    for p in pairs:
        p[0].attn.clear_cache()
    gdec.clear_cache()
    steps = 24
    ref_toks, margins = odec.generate(prompt, steps)
    got_toks = gdec.generate(prompt, steps)
    assert all(g.attn.cache_len == len(prompt) + steps - 1 for _, g, _ in pairs)
    diff = next((i for i, (a, b) in enumerate(zip(got_toks.tolist(), ref_toks)) if a != b), None)
    if diff is not None:
        spread = float(np.ptp(ref_logits))
        assert margins[diff] <= LOGIT_TOL * spread, (diff, margins[diff], spread)
    assert len(set(ref_toks)) > 1
    gdec.close()
    g_head.close()
    for _, _, owned in pairs:
        for o in owned:
            o.close()


def test_greedy_on_the_device_takes_the_first_of_equal_logits(ctx):
    """sampler.cr:38-53: `v > best` keeps the first index among equal maxima; non-finite logits
    are skipped.  lm_head columns 5 and 9 are identical, so their logits tie exactly."""
    import shainet_b200 as S
    from oracle import oracle as O
    rng = np.random.default_rng(53)
    d, vocab = 2048, 64
    ob, gb, owned = _make_block(ctx, rng, d, 32, 8, 64, 0, 5e5, 1e-5)
    emb = _w(rng, vocab, d)
    head = _w(rng, d, vocab)
    head[:, 9] = head[:, 5]
    bias = np.zeros(vocab, np.float32)
    bias[[5, 9]] = 10.0            # the tied pair is the maximum
    bias[3] = np.inf               # a non-finite logit must not win
    o_head = O.OracleQ8(head)
    g_head = S.Q8Weight.from_quantized(ctx, o_head.q, o_head.scales)
    gdec = S.Decoder(ctx, [gb], emb, None, g_head, bias, 1e-5)
    logits, tok = gdec.run([1, 2, 3])
    assert logits[5] == logits[9] and np.isinf(logits[3])
    assert tok == 5 == O.greedy(logits)
    gdec.close()
    g_head.close()
    for o in owned:
        o.close()
