"""Host-side mirror of the attention state and calls of SHAInet's ``LlamaBlock``
(src/shainet/transformer/llama_block.cr) over the libshainet_attn C ABI.

``AttnContext`` stands for the class-level scratch of the reference block,
``KVCache`` for one block's ``@k_cache/@v_cache/@cache_len`` and device mirror,
``LlamaAttention`` for the slice of ``attention_cached_cpu`` between the q/k/v
projections and ``o_proj`` (bias, QK-norm, RoPE, append, attention).  Method
names follow the reference (``forward_cached``, ``clear_cache``).
"""
from __future__ import annotations

import ctypes as C
import math

import numpy as np

from . import _lib
from ._lib import (F_GENERIC, F_SPLITK, F_TENSOR, F_UNFUSED, F_INPUTS_READY, F_TICKET_MERGE, F_TENSOR_1CTA,  # noqa: F401
                   ShainetAttnError, check)


def _fp(a: np.ndarray):
    return a.ctypes.data_as(C.POINTER(C.c_float))


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _opt(a):
    return (None, None) if a is None else (lambda x: (x, _fp(x)))(_f32(a))


CUDA_STREAM_LEGACY = 1  # cudaStreamLegacy: the handle that names the legacy default stream explicitly


def _stream_arg(stream):
    """None -> NULL (the context's own stream); 0 -> the legacy default stream,
    which has to be named by its explicit handle because NULL is taken; any
    other integer is a cudaStream_t."""
    if stream is None:
        return None
    return C.c_void_p(CUDA_STREAM_LEGACY if stream == 0 else stream)


def device_count() -> int:
    return _lib.load().shainet_attn_device_count()


def default_scale(head_dim: int) -> float:
    """f32(1/sqrt(head_dim)) as llama_block.cr:249 computes it."""
    return float(np.float32(1.0 / math.sqrt(float(head_dim))))


class AttnContext:
    def __init__(self, device: int = 0):
        self.L = _lib.load()
        h = C.c_void_p()
        check(self.L.shainet_attn_ctx_create(C.byref(h), device))
        self.h = h
        self.device = device

    def sync(self):
        check(self.L.shainet_attn_ctx_sync(self.h))

    def scratch_bytes(self) -> int:
        return self.L.shainet_attn_ctx_scratch_bytes(self.h)

    def set_lse_out(self, ptr):
        """Device pointer (int) that receives max + ln(sum) per (sequence, head) of every
        fused decode call, or None to stop."""
        check(self.L.shainet_attn_ctx_set_lse_out(self.h, ptr))

    def merge_parts(self, gathered_ptr: int, world: int, seq_parts: int, heads_per_rank: int, head_dim: int,
                    out_ptr: int, stream=None):
        check(self.L.shainet_attn_merge_parts(self.h, gathered_ptr, world, seq_parts, heads_per_rank, head_dim, out_ptr,
                                              _stream_arg(stream)))

    # ---- exchange of head outputs between the GPUs of one box ----
    def comm_create(self, data_floats: int) -> bytes:
        """Allocate this rank's exchange buffer; returns its inter-process handle."""
        buf = C.create_string_buffer(_lib.COMM_HANDLE_BYTES)
        check(self.L.shainet_attn_comm_create(self.h, data_floats, buf))
        return buf.raw

    def comm_open(self, handles, rank: int):
        """Map the other ranks' exchange buffers; `handles` in rank order (own included)."""
        blob = b"".join(handles)
        assert len(blob) == _lib.COMM_HANDLE_BYTES * len(handles)
        check(self.L.shainet_attn_comm_open(self.h, blob, len(handles), rank))

    def comm_set_target(self, out_offset: int, lse_offset: int, epoch: int):
        """Arm the next fused decode call to store its head rows (and log-sum-exp values when
        lse_offset >= 0) into every rank's buffer as {value, epoch} words."""
        check(self.L.shainet_attn_comm_set_target(self.h, out_offset, lse_offset, epoch))

    def comm_wait(self, offset: int, count: int, epoch: int, stream=None):
        """Enqueue the wait for the words [offset, offset + count) of this rank's buffer to carry
        `epoch`; it also unpacks them into the float area."""
        check(self.L.shainet_attn_comm_wait(self.h, offset, count, epoch, _stream_arg(stream)))

    def comm_set_wait_limit_ms(self, ms: int):
        """Limit of the device-side polls for other ranks' exchange words (default 1000 ms)."""
        check(self.L.shainet_attn_comm_set_wait_limit_ms(self.h, ms))

    def comm_data_ptr(self) -> int:
        p = C.c_void_p()
        check(self.L.shainet_attn_comm_data_ptr(self.h, C.byref(p)))
        return p.value

    def comm_read(self, offset: int, host: np.ndarray, stream=None):
        assert host.dtype == np.float32 and host.flags.c_contiguous
        check(self.L.shainet_attn_comm_read(self.h, offset, _fp(host), host.size, _stream_arg(stream)))

    def timing_enable(self, on: bool):
        check(self.L.shainet_attn_ctx_timing_enable(self.h, int(on)))

    def timing_read(self):
        """(summed device ms of the bracketed attention launches, their count); clears the record."""
        ms, n = C.c_double(), C.c_int()
        check(self.L.shainet_attn_ctx_timing_read(self.h, C.byref(ms), C.byref(n)))
        return ms.value, n.value

    def close(self):
        if getattr(self, "h", None):
            check(self.L.shainet_attn_ctx_destroy(self.h))
            self.h = None


KV_FORMATS = {"f32": 0, "bf16": 1}


class KVCache:
    """One block's device KV cache.  ``kv_format`` "f32" is the reference's layout
    (llama_block.cr:45-56); "bf16" is this library's opt-in that rounds the rows to
    bfloat16 as they are appended (no counterpart in the reference)."""

    def __init__(self, ctx: AttnContext, num_heads: int, num_kv_heads: int, head_dim: int, initial_capacity: int = 0,
                 kv_format: str = "f32", reserve_capacity: int = 0):
        self.ctx, self.L = ctx, ctx.L
        self.num_heads, self.num_kv_heads, self.head_dim = num_heads, num_kv_heads, head_dim
        self.q_dim, self.kv_dim = num_heads * head_dim, num_kv_heads * head_dim
        if kv_format not in KV_FORMATS:
            raise ValueError(f"kv_format must be one of {sorted(KV_FORMATS)}")
        h = C.c_void_p()
        if reserve_capacity:
            # addresses for reserve_capacity rows, memory mapped behind them as the cache fills (no copy on growth)
            check(self.L.shainet_attn_kv_create_reserved(ctx.h, C.byref(h), num_heads, num_kv_heads, head_dim,
                                                         reserve_capacity, KV_FORMATS[kv_format]))
            self.h = h
            if initial_capacity:
                self.reserve(initial_capacity)
        else:
            check(self.L.shainet_attn_kv_create_fmt(ctx.h, C.byref(h), num_heads, num_kv_heads, head_dim, initial_capacity,
                                                    KV_FORMATS[kv_format]))
            self.h = h

    @property
    def kv_format(self) -> str:
        code = check(self.L.shainet_attn_kv_format(self.h))
        return {v: k for k, v in KV_FORMATS.items()}[code]

    def close(self):
        if getattr(self, "h", None):
            check(self.L.shainet_attn_kv_destroy(self.h))
            self.h = None

    def __len__(self) -> int:
        return check(self.L.shainet_attn_kv_len(self.h))

    @property
    def capacity(self) -> int:
        return check(self.L.shainet_attn_kv_capacity(self.h))

    def reset(self):
        check(self.L.shainet_attn_kv_reset(self.h))

    def truncate(self, n: int):
        check(self.L.shainet_attn_kv_truncate(self.h, n))

    def reserve(self, total_len: int):
        check(self.L.shainet_attn_kv_reserve(self.h, total_len))

    def set_rope_theta(self, theta: float):
        check(self.L.shainet_attn_kv_set_rope_theta(self.h, theta))

    def set_rope(self, inv_freq):
        f = _f32(inv_freq)
        check(self.L.shainet_attn_kv_set_rope(self.h, _fp(f), f.size))

    def set_qk_norm(self, q_weight, k_weight, eps: float):
        q, qp = _opt(q_weight)
        k, kp = _opt(k_weight)
        check(self.L.shainet_attn_kv_set_qk_norm(self.h, qp, kp, eps))

    def set_bias(self, b_q, b_k, b_v):
        (q, qp), (k, kp), (v, vp) = _opt(b_q), _opt(b_k), _opt(b_v)
        check(self.L.shainet_attn_kv_set_bias(self.h, qp, kp, vp))

    def export(self, n: int | None = None):
        n = len(self) if n is None else n
        k = np.empty((self.num_kv_heads, n, self.head_dim), np.float32)
        v = np.empty_like(k)
        check(self.L.shainet_attn_kv_export(self.h, _fp(k), _fp(v), n))
        return k, v

    def import_(self, k, v):
        k, v = _f32(k), _f32(v)
        if k.shape != v.shape or k.ndim != 3 or k.shape[0] != self.num_kv_heads or k.shape[2] != self.head_dim:
            raise ValueError("cache arrays must be [num_kv_heads, len, head_dim]")
        check(self.L.shainet_attn_kv_import(self.h, _fp(k), _fp(v), k.shape[1]))

    def fill_normal(self, n: int, seed: int):
        check(self.L.shainet_attn_kv_fill_normal(self.h, n, seed))

    def device_ptrs(self):
        k, v = C.c_void_p(), C.c_void_p()
        check(self.L.shainet_attn_kv_device_ptrs(self.h, C.byref(k), C.byref(v)))
        return k.value, v.value


class LlamaAttention:
    """Attention part of ``LlamaBlock``: same constructor meaning for
    ``num_heads, num_kv_heads, head_dim, rope_theta, eps`` (llama_block.cr:73-92),
    same optional ``rope_freqs``, ``q_norm/k_norm`` and ``b_q/b_k/b_v`` properties,
    ``forward_cached`` taking the projection outputs where the reference calls
    ``attention_heads_gpu`` (:292-296), ``clear_cache`` for ``clear_cache!``."""

    def __init__(self, ctx: AttnContext, num_heads: int, num_kv_heads: int | None = None, head_dim: int = 64,
                 rope_theta: float = 10000.0, eps: float = 1e-6, rope_freqs=None, q_norm=None, k_norm=None,
                 b_q=None, b_k=None, b_v=None, initial_capacity: int = 0, kv_format: str = "f32", reserve_capacity: int = 0):
        num_kv_heads = num_heads if num_kv_heads is None else num_kv_heads
        self.ctx = ctx
        self.cache = KVCache(ctx, num_heads, num_kv_heads, head_dim, initial_capacity, kv_format, reserve_capacity)
        self.num_heads, self.num_kv_heads, self.head_dim = num_heads, num_kv_heads, head_dim
        self.q_dim, self.kv_dim = self.cache.q_dim, self.cache.kv_dim
        self.scale = default_scale(head_dim)
        if rope_freqs is not None:
            self.cache.set_rope(rope_freqs)
        else:
            self.cache.set_rope_theta(rope_theta)
        if q_norm is not None or k_norm is not None:
            self.cache.set_qk_norm(q_norm, k_norm, eps)
        if b_q is not None or b_k is not None or b_v is not None:
            self.cache.set_bias(b_q, b_k, b_v)

    @property
    def cache_len(self) -> int:
        return len(self.cache)

    def clear_cache(self):
        self.cache.reset()

    def forward_cached(self, q, k_new, v_new, flags: int = 0) -> np.ndarray:
        """Host arrays in, host array out (the reference's SimpleMatrix path)."""
        q, k_new, v_new = _f32(q), _f32(k_new), _f32(v_new)
        T = q.shape[0]
        if q.shape != (T, self.q_dim) or k_new.shape != (T, self.kv_dim) or v_new.shape != (T, self.kv_dim):
            raise ValueError("q must be [T, num_heads*head_dim]; k_new, v_new [T, num_kv_heads*head_dim]")
        out = np.empty((T, self.q_dim), np.float32)
        check(self.ctx.L.shainet_attn_forward_host(self.ctx.h, self.cache.h, _fp(q), _fp(k_new), _fp(v_new), _fp(out),
                                                   T, self.scale, flags))
        return out

    def forward_cached_dev(self, q_ptr: int, k_ptr: int, v_ptr: int, out_ptr: int, new_tokens: int, stream=None,
                           flags: int = 0):
        """Device pointers (ints) on a caller stream (see _stream_arg); asynchronous."""
        check(self.ctx.L.shainet_attn_forward_dev(self.ctx.h, self.cache.h, q_ptr, k_ptr, v_ptr, out_ptr, new_tokens,
                                                  self.scale, flags, _stream_arg(stream)))

    def forward_cached_dev_at(self, q_ptr: int, k_ptr, v_ptr, out_ptr: int, position: int, append: bool, stream=None,
                              flags: int = 0):
        """One decode token of a sequence that is split over ranks: RoPE position
        `position`; this rank stores and sees the token's k/v row only if `append`."""
        check(self.ctx.L.shainet_attn_forward_dev_at(self.ctx.h, self.cache.h, q_ptr, k_ptr, v_ptr, out_ptr, position,
                                                     int(append), self.scale, flags, _stream_arg(stream)))

    def forward_cached_dev_exchange(self, q_ptr: int, k_ptr, v_ptr, out_ptr: int, position: int, append: bool,
                                    out_offset: int, lse_offset: int, wait_offset: int, wait_count: int, epoch: int,
                                    stream=None, flags: int = 0):
        """One decode token on a rank of a sharded model: attention over this rank's rows, head
        rows (and log-sum-exp values when lse_offset >= 0) delivered into every rank's exchange
        buffer by the kernel, then the wait for (and unpacking of) the float range
        [wait_offset, wait_offset + wait_count) of this rank's buffer, in one foreign call."""
        check(self.ctx.L.shainet_attn_forward_dev_exchange(
            self.ctx.h, self.cache.h, q_ptr, k_ptr, v_ptr, out_ptr, position, int(append), self.scale, flags,
            out_offset, lse_offset, wait_offset, wait_count, epoch, _stream_arg(stream)))

    def forward_cached_dev_exchange_merge(self, q_ptr: int, k_ptr, v_ptr, out_ptr: int, position: int, append: bool,
                                          slot_offset: int, seq_parts: int, epoch: int, out_full_ptr: int, stream=None,
                                          flags: int = 0):
        """forward_cached_dev_exchange for a sequence split over the ranks of a head group: the slot
        [slot_offset, slot_offset + world * heads * (head_dim + 1)) holds [rank][rows | log-sum-exp]; one
        kernel waits for all ranks and merges each group's parts into out_full_ptr."""
        check(self.ctx.L.shainet_attn_forward_dev_exchange_merge(
            self.ctx.h, self.cache.h, q_ptr, k_ptr, v_ptr, out_ptr, position, int(append), self.scale, flags,
            slot_offset, seq_parts, epoch, out_full_ptr, _stream_arg(stream)))

    def close(self):
        self.cache.close()


def forward_batched_dev(ctx: AttnContext, caches, q_ptr: int, k_ptr: int, v_ptr: int, out_ptr: int, scale: float,
                        stream=None, flags: int = 0):
    """One decode token for every cache in ``caches`` (lock step), one launch set."""
    arr = (C.c_void_p * len(caches))(*[c.h for c in caches])
    check(ctx.L.shainet_attn_forward_batched_dev(ctx.h, arr, len(caches), q_ptr, k_ptr, v_ptr, out_ptr, scale, flags,
                                                 _stream_arg(stream)))


class Q8Weight:
    """The reference's ``QuantizedCudaMatrix`` (src/shainet/math/quantized_cuda_matrix.cr): a
    weight [K, N] held on the device as Q8_0.  ``from_simple`` quantises an fp32 matrix,
    ``from_quantized`` uploads int8 values [N, K] and scales [N, ceil(K/32)]."""

    def __init__(self, ctx: AttnContext, handle, K: int, N: int):
        self.ctx, self.h, self.K, self.N = ctx, handle, K, N

    @classmethod
    def from_simple(cls, ctx: AttnContext, w):
        w = _f32(w)
        h = C.c_void_p()
        check(ctx.L.shainet_attn_q8_create(ctx.h, C.byref(h), _fp(w), w.shape[0], w.shape[1]))
        return cls(ctx, h, w.shape[0], w.shape[1])

    @classmethod
    def from_quantized(cls, ctx: AttnContext, q, scales):
        q = np.ascontiguousarray(q, np.int8)
        scales = _f32(scales)
        N, K = q.shape
        h = C.c_void_p()
        check(ctx.L.shainet_attn_q8_create_raw(ctx.h, C.byref(h), q.ctypes.data_as(C.c_void_p), _fp(scales), K, N))
        return cls(ctx, h, K, N)

    @classmethod
    def wrap(cls, ctx: AttnContext, q_ptr: int, scales_ptr: int, K: int, N: int):
        """Adopt device arrays the caller owns (int8 [N, K], fp32 [N, ceil(K/32)]) without copying."""
        h = C.c_void_p()
        check(ctx.L.shainet_attn_q8_wrap(ctx.h, C.byref(h), q_ptr, scales_ptr, K, N))
        return cls(ctx, h, K, N)

    def export(self):
        q = np.empty((self.N, self.K), np.int8)
        s = np.empty((self.N, (self.K + 31) // 32), np.float32)
        check(self.ctx.L.shainet_attn_q8_export(self.h, q.ctypes.data_as(C.c_void_p), _fp(s)))
        return q, s

    def gemv_dev(self, x_ptr: int, y_ptr: int, rows: int, stream=None):
        """``gemv_into``: y[rows, N] = x[rows, K] . dequant(W), device pointers."""
        check(self.ctx.L.shainet_attn_q8_gemv_dev(self.ctx.h, self.h, x_ptr, y_ptr, rows, _stream_arg(stream)))

    def close(self):
        if getattr(self, "h", None):
            check(self.ctx.L.shainet_attn_q8_destroy(self.h))
            self.h = None


class LlamaBlock:
    """``LlamaBlock`` with every step of ``forward_cached`` on the device
    (src/shainet/transformer/llama_block.cr:189-196): the attention state is a
    ``LlamaAttention``, the projections and the FFN are ``Q8Weight`` objects."""

    def __init__(self, ctx: AttnContext, attn: LlamaAttention, d_model: int, eps: float, norm1, wq, wk, wv, wo,
                 norm2=None, gate=None, up=None, down=None):
        self.ctx, self.attn, self.d_model = ctx, attn, d_model
        self._keep = (wq, wk, wv, wo, gate, up, down)
        n1, n1p = _opt(norm1)
        n2, n2p = _opt(norm2)
        hp = lambda w: None if w is None else w.h
        h = C.c_void_p()
        check(ctx.L.shainet_attn_block_create(ctx.h, C.byref(h), attn.cache.h, d_model, n1p, wq.h, wk.h, wv.h, wo.h, n2p,
                                              hp(gate), hp(up), hp(down), eps))
        self.h = h

    def forward_cached(self, x) -> np.ndarray:
        """Host rows in, host rows out: one copy each way."""
        x = _f32(x)
        out = np.empty_like(x)
        check(self.ctx.L.shainet_attn_block_forward_host(self.ctx.h, self.h, _fp(x), _fp(out), x.shape[0]))
        return out

    def forward_cached_dev(self, x_ptr: int, out_ptr: int, new_tokens: int, stream=None):
        check(self.ctx.L.shainet_attn_block_forward_dev(self.ctx.h, self.h, x_ptr, out_ptr, new_tokens, _stream_arg(stream)))

    def clear_cache(self):
        self.attn.clear_cache()

    def close(self):
        if getattr(self, "h", None):
            check(self.ctx.L.shainet_attn_block_destroy(self.h))
            self.h = None


class Decoder:
    """The token loop of ``Network#run`` with ``use_kv_cache`` (src/shainet/basic/network_run.cr:185-264,
    294-315) plus ``Sampler.greedy``, resident on the device."""

    def __init__(self, ctx: AttnContext, blocks, embedding, final_norm, lm_head: Q8Weight, lm_bias=None, eps: float = 1e-6):
        self.ctx, self.blocks, self.lm_head = ctx, list(blocks), lm_head
        emb = _f32(embedding)
        self.vocab, self.d_model = emb.shape
        fn, fnp = _opt(final_norm)
        lb, lbp = _opt(lm_bias)
        arr = (C.c_void_p * len(self.blocks))(*[b.h for b in self.blocks])
        h = C.c_void_p()
        check(ctx.L.shainet_attn_decoder_create(ctx.h, C.byref(h), arr, len(self.blocks), _fp(emb), self.vocab, fnp, lm_head.h,
                                                lbp, eps))
        self.h = h

    def run(self, ids, want_logits: bool = True):
        """``run(Array(Int32))``: (logits of the last row or None, greedy token)."""
        ids = np.ascontiguousarray(ids, np.int32)
        logits = np.empty(self.vocab, np.float32) if want_logits else None
        tok = C.c_int32(-1)
        check(self.ctx.L.shainet_attn_decoder_run(self.ctx.h, self.h, ids.ctypes.data_as(C.POINTER(C.c_int32)), ids.size,
                                                  _fp(logits) if want_logits else None, C.byref(tok)))
        return logits, tok.value

    def generate(self, prompt, steps: int) -> np.ndarray:
        """Greedy tokens of `steps` steps after the prompt; nothing visits the host in between."""
        ids = np.ascontiguousarray(prompt, np.int32)
        out = np.empty(steps, np.int32)
        check(self.ctx.L.shainet_attn_decoder_generate(self.ctx.h, self.h, ids.ctypes.data_as(C.POINTER(C.c_int32)), ids.size,
                                                       steps, out.ctypes.data_as(C.POINTER(C.c_int32))))
        return out

    def clear_cache(self):
        for b in self.blocks:
            b.clear_cache()

    def close(self):
        if getattr(self, "h", None):
            check(self.ctx.L.shainet_attn_decoder_destroy(self.h))
            self.h = None
