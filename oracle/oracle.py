"""ctypes front end to the CPU oracle (``oracle/liboracle.so``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by ``__graft_entry__.smoke()``
and by ``bench.py``'s CPU-baseline / reference legs.  The shipped package never
imports it.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import build_oracle

_LIB = None


def _fp(a: np.ndarray):
    return a.ctypes.data_as(C.POINTER(C.c_float))


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def lib():
    global _LIB
    if _LIB is not None:
        return _LIB
    path = build_oracle.ORACLE_SO
    if not os.path.exists(path) or os.path.getmtime(path) < os.path.getmtime(
            os.path.join(build_oracle.HERE, "shainet_oracle.cpp")):
        build_oracle.build_oracle(force=True)
    L = C.CDLL(path)
    P, F, I, D = C.c_void_p, C.POINTER(C.c_float), C.c_int, C.c_double
    L.oracle_block_create.restype = P
    L.oracle_block_create.argtypes = [I, I, I, D, D]
    L.oracle_block_destroy.argtypes = [P]
    L.oracle_block_set_rope_freqs.argtypes = [P, F]
    L.oracle_block_set_qk_norm.argtypes = [P, F, F]
    L.oracle_block_set_bias.argtypes = [P, F, F, F]
    L.oracle_block_clear.argtypes = [P]
    L.oracle_block_set_kv_rounding.argtypes = [P, I]
    L.oracle_round_bf16.argtypes = [F, C.c_size_t, F]
    L.oracle_block_len.argtypes = [P]
    L.oracle_block_len.restype = I
    L.oracle_inv_freq.argtypes = [P, F]
    L.oracle_block_import.argtypes = [P, F, F, I]
    L.oracle_block_export.argtypes = [P, F, F]
    L.oracle_block_attend_cached.argtypes = [P, F, F, F, I, F, I, I]
    L.oracle_block_attend_only.argtypes = [P, F, I, I, F, I, I]
    L.oracle_block_attend_full.argtypes = [P, F, F, F, I, F]
    L.oracle_rope_apply.argtypes = [F, I, I, I, D, F]
    L.oracle_llama3_rope_freqs.argtypes = [D, I, D, D, D, D, F]
    L.oracle_matmul.argtypes = [F, F, I, I, I, F]
    L.oracle_rmsnorm.argtypes = [F, I, I, F, D, F]
    L.oracle_swiglu.argtypes = [F, I, I, I, F, F, F, F]
    L.oracle_add.argtypes = [F, F, C.c_size_t, F]
    L.oracle_max_threads.restype = I
    L.oracle_q8_quantize.argtypes = [F, I, I, P, F]
    L.oracle_q8_gemv.argtypes = [F, P, F, F, I, I, I, I, I]
    L.oracle_swiglu_act.argtypes = [F, F, C.c_size_t, F]
    L.oracle_add_bias_row.argtypes = [F, F, I]
    L.oracle_greedy.argtypes = [F, I]
    L.oracle_greedy.restype = I
    _LIB = L
    return L


def round_bf16(x) -> np.ndarray:
    """fp32 -> bfloat16 -> fp32, round to nearest even."""
    x = _f32(x)
    out = np.empty_like(x)
    lib().oracle_round_bf16(_fp(x), x.size, _fp(out))
    return out


class OracleAttention:
    """The attention state of the reference's ``LlamaBlock`` (per-kv-head growing
    K/V arrays and ``cache_len``; src/shainet/transformer/llama_block.cr:45-48)
    with its cached and uncached attention between the projections and o_proj."""

    def __init__(self, num_heads, num_kv_heads, head_dim, rope_theta=10000.0, eps=1e-6,
                 rope_freqs=None, q_norm=None, k_norm=None, b_q=None, b_k=None, b_v=None, kv_rounding=None):
        self.L = lib()
        self.num_heads, self.num_kv_heads, self.head_dim = num_heads, num_kv_heads, head_dim
        self.q_dim, self.kv_dim = num_heads * head_dim, num_kv_heads * head_dim
        self.h = self.L.oracle_block_create(num_heads, num_kv_heads, head_dim, rope_theta, eps)
        if not self.h:
            raise ValueError("bad head configuration")
        self._keep = []
        if kv_rounding not in (None, "bf16"):
            raise ValueError("kv_rounding is None (the reference's fp32 rows) or 'bf16'")
        if kv_rounding == "bf16":   # not a reference behaviour: the library's opt-in 16-bit cache, restated
            self.L.oracle_block_set_kv_rounding(self.h, 1)
        if rope_freqs is not None:
            f = _f32(rope_freqs)
            self.L.oracle_block_set_rope_freqs(self.h, _fp(f))
        if q_norm is not None or k_norm is not None:
            qn = _f32(q_norm) if q_norm is not None else None
            kn = _f32(k_norm) if k_norm is not None else None
            self.L.oracle_block_set_qk_norm(self.h, _fp(qn) if qn is not None else None,
                                            _fp(kn) if kn is not None else None)
        if b_q is not None or b_k is not None or b_v is not None:
            bs = [(_f32(b) if b is not None else None) for b in (b_q, b_k, b_v)]
            self.L.oracle_block_set_bias(self.h, *[(_fp(b) if b is not None else None) for b in bs])

    def __del__(self):
        try:
            if self.h:
                self.L.oracle_block_destroy(self.h)
                self.h = None
        except Exception:
            pass

    def clear_cache(self):
        self.L.oracle_block_clear(self.h)

    @property
    def cache_len(self) -> int:
        return self.L.oracle_block_len(self.h)

    def inv_freq(self) -> np.ndarray:
        out = np.empty(self.head_dim // 2, np.float32)
        self.L.oracle_inv_freq(self.h, _fp(out))
        return out

    def import_cache(self, k, v):
        k, v = _f32(k), _f32(v)
        assert k.shape == v.shape and k.shape[0] == self.num_kv_heads and k.shape[2] == self.head_dim
        self.L.oracle_block_import(self.h, _fp(k), _fp(v), k.shape[1])

    def export_cache(self):
        n = self.cache_len
        k = np.empty((self.num_kv_heads, n, self.head_dim), np.float32)
        v = np.empty_like(k)
        self.L.oracle_block_export(self.h, _fp(k), _fp(v))
        return k, v

    def attend_cached(self, q, k_new, v_new, threads=1, mode=0) -> np.ndarray:
        q, k_new, v_new = _f32(q), _f32(k_new), _f32(v_new)
        T = q.shape[0]
        assert q.shape == (T, self.q_dim) and k_new.shape == (T, self.kv_dim) and v_new.shape == k_new.shape
        out = np.empty((T, self.q_dim), np.float32)
        self.L.oracle_block_attend_cached(self.h, _fp(q), _fp(k_new), _fp(v_new), T, _fp(out), threads, mode)
        return out

    def attend_only(self, q, start_pos, threads=1, mode=0) -> np.ndarray:
        q = _f32(q)
        T = q.shape[0]
        out = np.empty((T, self.q_dim), np.float32)
        self.L.oracle_block_attend_only(self.h, _fp(q), T, start_pos, _fp(out), threads, mode)
        return out

    def attend_full(self, q, k, v) -> np.ndarray:
        q, k, v = _f32(q), _f32(k), _f32(v)
        S = q.shape[0]
        out = np.empty((S, self.q_dim), np.float32)
        self.L.oracle_block_attend_full(self.h, _fp(q), _fp(k), _fp(v), S, _fp(out))
        return out


def rope_apply(x, start_pos=0, theta=10000.0) -> np.ndarray:
    x = _f32(x)
    out = np.empty_like(x)
    lib().oracle_rope_apply(_fp(x), x.shape[0], x.shape[1], start_pos, theta, _fp(out))
    return out


def llama3_rope_freqs(theta, head_dim, factor, low_freq_factor, high_freq_factor, old_ctx) -> np.ndarray:
    out = np.empty(head_dim // 2, np.float32)
    lib().oracle_llama3_rope_freqs(theta, head_dim, factor, low_freq_factor, high_freq_factor, old_ctx, _fp(out))
    return out


def matmul(a, b) -> np.ndarray:
    a, b = _f32(a), _f32(b)
    out = np.empty((a.shape[0], b.shape[1]), np.float32)
    lib().oracle_matmul(_fp(a), _fp(b), a.shape[0], a.shape[1], b.shape[1], _fp(out))
    return out


def rmsnorm(x, gamma, eps) -> np.ndarray:
    x, gamma = _f32(x), _f32(gamma)
    out = np.empty_like(x)
    lib().oracle_rmsnorm(_fp(x), x.shape[0], x.shape[1], _fp(gamma), eps, _fp(out))
    return out


def swiglu(x, gate_w, up_w, down_w) -> np.ndarray:
    x, gate_w, up_w, down_w = _f32(x), _f32(gate_w), _f32(up_w), _f32(down_w)
    out = np.empty((x.shape[0], down_w.shape[1]), np.float32)
    lib().oracle_swiglu(_fp(x), x.shape[0], x.shape[1], gate_w.shape[1], _fp(gate_w), _fp(up_w), _fp(down_w), _fp(out))
    return out


def add(a, b) -> np.ndarray:
    a, b = _f32(a), _f32(b)
    out = np.empty_like(a)
    lib().oracle_add(_fp(a), _fp(b), a.size, _fp(out))
    return out


def max_threads() -> int:
    return lib().oracle_max_threads()


class OracleLlamaBlock:
    """Whole decoder block on the host (norm1 -> attention -> residual -> norm2 ->
    SwiGLU -> residual; src/shainet/transformer/llama_block.cr:179-196), used only
    to replay the reference's cache-consistency spec.  Weights are [in, out]."""

    def __init__(self, d_model, num_heads, num_kv_heads, head_dim, eps, rope_theta, w):
        self.attn = OracleAttention(num_heads, num_kv_heads, head_dim, rope_theta, eps)
        self.eps, self.w = eps, w

    def _wrap(self, x, attn_fn):
        w = self.w
        normed = rmsnorm(x, w["norm1"], self.eps)
        q, k, v = matmul(normed, w["w_q"]), matmul(normed, w["w_k"]), matmul(normed, w["w_v"])
        a = matmul(attn_fn(q, k, v), w["w_o"])
        h = add(x, a)
        n2 = rmsnorm(h, w["norm2"], self.eps)
        return add(h, swiglu(n2, w["gate"], w["up"], w["down"]))

    def forward(self, x):
        return self._wrap(x, self.attn.attend_full)

    def forward_cached(self, x):
        return self._wrap(x, self.attn.attend_cached)

    def clear_cache(self):
        self.attn.clear_cache()


class OracleQ8:
    """A Q8_0 weight as the reference holds it (QuantizedCudaMatrix,
    src/shainet/math/quantized_cuda_matrix.cr): quantised from an fp32 matrix [K, N]."""

    def __init__(self, w):
        w = _f32(w)
        self.K, self.N = w.shape
        self.q = np.empty((self.N, self.K), np.int8)
        self.scales = np.empty((self.N, (self.K + 31) // 32), np.float32)
        lib().oracle_q8_quantize(_fp(w), self.K, self.N, self.q.ctypes.data_as(C.c_void_p), _fp(self.scales))

    def dequantised(self) -> np.ndarray:
        """[K, N] fp32: q * scale."""
        s = np.repeat(self.scales, 32, axis=1)[:, :self.K]
        return (self.q.astype(np.float32) * s).T.copy()

    def gemv(self, x, fused=1, threads=None) -> np.ndarray:
        """y = x . dequant(W) in the reduction order of the reference's gemm_q8_f32_kernel."""
        x = _f32(x)
        M = x.shape[0]
        assert x.shape == (M, self.K)
        y = np.empty((M, self.N), np.float32)
        lib().oracle_q8_gemv(_fp(x), self.q.ctypes.data_as(C.c_void_p), _fp(self.scales), _fp(y), M, self.N, self.K, fused,
                             threads or max_threads())
        return y


def swiglu_act(gate, up) -> np.ndarray:
    gate, up = _f32(gate), _f32(up)
    out = np.empty_like(gate)
    lib().oracle_swiglu_act(_fp(gate), _fp(up), gate.size, _fp(out))
    return out


def greedy(logits) -> int:
    logits = _f32(logits).reshape(-1)
    return lib().oracle_greedy(_fp(logits), logits.size)


class OracleQ8Block:
    """LlamaBlock#forward_cached (llama_block.cr:189-196) with Q8_0 projections: the host
    steps in the reference's arithmetic, the GEMVs in its kernel's order."""

    def __init__(self, attn: OracleAttention, eps, norm1, wq, wk, wv, wo, norm2=None, gate=None, up=None, down=None):
        self.attn, self.eps = attn, eps
        self.norm1, self.norm2 = _f32(norm1), (None if norm2 is None else _f32(norm2))
        self.wq, self.wk, self.wv, self.wo, self.gate, self.up, self.down = wq, wk, wv, wo, gate, up, down

    def forward_cached(self, x, threads=None) -> np.ndarray:
        x = _f32(x)
        n = rmsnorm(x, self.norm1, self.eps)
        a = self.attn.attend_cached(self.wq.gemv(n), self.wk.gemv(n), self.wv.gemv(n), threads=threads or max_threads())
        h = add(x, self.wo.gemv(a))
        if self.gate is None:
            return h
        n2 = rmsnorm(h, self.norm2, self.eps)
        hidden = swiglu_act(self.gate.gemv(n2), self.up.gemv(n2))
        return add(h, self.down.gemv(hidden))


class OracleQ8Decoder:
    """Network#run with use_kv_cache (src/shainet/basic/network_run.cr:185-264): embedding gather,
    blocks, final norm, Q8_0 lm_head on the last row, bias, and Sampler.greedy."""

    def __init__(self, embedding, blocks, final_norm, lm_head: OracleQ8, lm_bias, eps):
        self.embedding, self.blocks = _f32(embedding), blocks
        self.final_norm = None if final_norm is None else _f32(final_norm)
        self.lm_head, self.eps = lm_head, eps
        self.lm_bias = None if lm_bias is None else _f32(lm_bias)

    def run(self, ids):
        x = self.embedding[np.asarray(ids, np.int64)]
        for b in self.blocks:
            x = b.forward_cached(x)
        last = x[-1:]
        if self.final_norm is not None:
            last = rmsnorm(last, self.final_norm, self.eps)
        logits = self.lm_head.gemv(last)[0]
        if self.lm_bias is not None:
            lib().oracle_add_bias_row(_fp(logits), _fp(self.lm_bias), logits.size)
        return logits, greedy(logits)

    def generate(self, prompt, steps):
        toks, margins = [], []
        logits, tok = self.run(prompt)
        for i in range(steps):
            top = np.sort(logits)[-2:]
            margins.append(float(top[1] - top[0]))
            toks.append(tok)
            if i + 1 < steps:
                logits, tok = self.run([tok])
        return toks, margins
