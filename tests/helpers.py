"""Shared pieces of the parity tests: shapes named by the benchmark configs,
seeded inputs, and the error measures written into the assertions."""
import numpy as np

# (num_heads, num_kv_heads, head_dim, rope_theta, qk_norm)
L1B = dict(H=32, KV=8, hd=64, theta=500000.0, qk_norm=False)     # LLaMA-3.2-1B attention
Q8B = dict(H=32, KV=8, hd=128, theta=1e6, qk_norm=True)          # Qwen3-8B attention
Q30 = dict(H=32, KV=4, hd=128, theta=1e6, qk_norm=True)          # Qwen3-30B-A3B attention

DECODE_TOL = 1e-5    # max |y - ref| / max |ref|, fp32 decode
SPEC_ABS_TOL = 1e-3  # the reference's own GPU-vs-CPU spec tolerance


def rel_err(y, ref):
    """max_i |y_i - ref_i| / max_i |ref_i| (outputs cross zero, so the error is
    normalised by the largest reference magnitude, not per element)."""
    y, ref = np.asarray(y, np.float64), np.asarray(ref, np.float64)
    return float(np.abs(y - ref).max() / max(np.abs(ref).max(), 1e-30))


def cosine(y, ref):
    y, ref = np.asarray(y, np.float64).ravel(), np.asarray(ref, np.float64).ravel()
    return float(y @ ref / (np.linalg.norm(y) * np.linalg.norm(ref)))


def norm_weights(rng, hd):
    return (1.0 + 0.02 * rng.standard_normal(hd)).astype(np.float32)


def make_pair(ctx, shape, rng, eps=1e-6, **extra):
    """An oracle attention state and a library attention state with the same parameters."""
    from oracle import oracle as O
    import shainet_b200 as S
    kw = dict(extra)
    cap = kw.pop("initial_capacity", 0)
    fmt = kw.pop("kv_format", "f32")   # "bf16": the library's opt-in 16-bit cache against the oracle's rounded rows
    reserve = kw.pop("reserve_capacity", 0)   # addresses reserved up front, memory mapped as the cache fills
    if shape.get("qk_norm"):
        kw.setdefault("q_norm", norm_weights(rng, shape["hd"]))
        kw.setdefault("k_norm", norm_weights(rng, shape["hd"]))
    o = O.OracleAttention(shape["H"], shape["KV"], shape["hd"], shape["theta"], eps,
                          kv_rounding="bf16" if fmt == "bf16" else None, **kw)
    g = S.LlamaAttention(ctx, shape["H"], shape["KV"], shape["hd"], shape["theta"], eps, initial_capacity=cap,
                         kv_format=fmt, reserve_capacity=reserve, **kw)
    return o, g


def qkv(rng, shape, T, dist="normal"):
    H, KV, hd = shape["H"], shape["KV"], shape["hd"]
    if dist == "uniform":
        f = lambda *s: rng.uniform(-1, 1, s).astype(np.float32)
    else:
        f = lambda *s: rng.standard_normal(s).astype(np.float32)
    return f(T, H * hd), f(T, KV * hd), f(T, KV * hd)
