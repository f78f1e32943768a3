"""ctypes binding of libshainet_attn.so (declarations follow include/shainet_attn.h).

There is no fallback: if the library is missing, loading raises."""
from __future__ import annotations

import ctypes as C
import os

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG, "lib", "libshainet_attn.so")

OK = 0
E_INVALID, E_CUDA, E_NOMEM, E_UNSUPPORTED, E_DEVICE_WAIT, E_STATE = -1, -2, -3, -4, -5, -6
F_GENERIC, F_SPLITK, F_TENSOR, F_UNFUSED, F_INPUTS_READY, F_TICKET_MERGE, F_TENSOR_1CTA = 1, 2, 4, 8, 16, 32, 64

_F = C.POINTER(C.c_float)
_P = C.c_void_p

# name -> (restype, argtypes); every symbol include/shainet_attn.h declares
COMM_HANDLE_BYTES = 64  # SHAINET_ATTN_COMM_HANDLE_BYTES

SIGNATURES = {
    "shainet_attn_version": (C.c_int, []),
    "shainet_attn_device_count": (C.c_int, []),
    "shainet_attn_last_error": (C.c_char_p, []),
    "shainet_attn_ctx_create": (C.c_int, [C.POINTER(_P), C.c_int]),
    "shainet_attn_ctx_destroy": (C.c_int, [_P]),
    "shainet_attn_ctx_sync": (C.c_int, [_P]),
    "shainet_attn_ctx_scratch_bytes": (C.c_size_t, [_P]),
    "shainet_attn_ctx_timing_enable": (C.c_int, [_P, C.c_int]),
    "shainet_attn_ctx_timing_read": (C.c_int, [_P, C.POINTER(C.c_double), C.POINTER(C.c_int)]),
    "shainet_attn_kv_create": (C.c_int, [_P, C.POINTER(_P), C.c_int, C.c_int, C.c_int, C.c_int]),
    "shainet_attn_kv_create_fmt": (C.c_int, [_P, C.POINTER(_P), C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]),
    "shainet_attn_kv_format": (C.c_int, [_P]),
    "shainet_attn_kv_create_reserved": (C.c_int, [_P, C.POINTER(_P), C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]),
    "shainet_attn_kv_destroy": (C.c_int, [_P]),
    "shainet_attn_kv_reset": (C.c_int, [_P]),
    "shainet_attn_kv_len": (C.c_int, [_P]),
    "shainet_attn_kv_capacity": (C.c_int, [_P]),
    "shainet_attn_kv_reserve": (C.c_int, [_P, C.c_int]),
    "shainet_attn_kv_truncate": (C.c_int, [_P, C.c_int]),
    "shainet_attn_kv_set_rope_theta": (C.c_int, [_P, C.c_double]),
    "shainet_attn_kv_set_rope": (C.c_int, [_P, _F, C.c_int]),
    "shainet_attn_kv_set_qk_norm": (C.c_int, [_P, _F, _F, C.c_double]),
    "shainet_attn_kv_set_bias": (C.c_int, [_P, _F, _F, _F]),
    "shainet_attn_kv_export": (C.c_int, [_P, _F, _F, C.c_int]),
    "shainet_attn_kv_import": (C.c_int, [_P, _F, _F, C.c_int]),
    "shainet_attn_kv_fill_normal": (C.c_int, [_P, C.c_int, C.c_uint64]),
    "shainet_attn_kv_device_ptrs": (C.c_int, [_P, C.POINTER(_P), C.POINTER(_P)]),
    "shainet_attn_forward_host": (C.c_int, [_P, _P, _F, _F, _F, _F, C.c_int, C.c_float, C.c_uint]),
    "shainet_attn_forward_dev": (C.c_int, [_P, _P, _P, _P, _P, _P, C.c_int, C.c_float, C.c_uint, _P]),
    "shainet_attn_forward_dev_at": (C.c_int, [_P, _P, _P, _P, _P, _P, C.c_int, C.c_int, C.c_float, C.c_uint, _P]),
    "shainet_attn_ctx_set_lse_out": (C.c_int, [_P, _P]),
    "shainet_attn_merge_parts": (C.c_int, [_P, _P, C.c_int, C.c_int, C.c_int, C.c_int, _P, _P]),
    "shainet_attn_comm_create": (C.c_int, [_P, C.c_size_t, _P]),
    "shainet_attn_comm_open": (C.c_int, [_P, _P, C.c_int, C.c_int]),
    "shainet_attn_comm_set_target": (C.c_int, [_P, C.c_longlong, C.c_longlong, C.c_uint]),
    "shainet_attn_comm_wait": (C.c_int, [_P, C.c_longlong, C.c_longlong, C.c_uint, _P]),
    "shainet_attn_forward_dev_exchange": (C.c_int, [_P, _P, _P, _P, _P, _P, C.c_int, C.c_int, C.c_float, C.c_uint,
                                                    C.c_longlong, C.c_longlong, C.c_longlong, C.c_longlong, C.c_uint, _P]),
    "shainet_attn_forward_dev_exchange_merge": (C.c_int, [_P, _P, _P, _P, _P, _P, C.c_int, C.c_int, C.c_float, C.c_uint,
                                                          C.c_longlong, C.c_int, C.c_uint, _P, _P]),
    "shainet_attn_comm_set_wait_limit_ms": (C.c_int, [_P, C.c_int]),
    "shainet_attn_comm_read": (C.c_int, [_P, C.c_longlong, C.POINTER(C.c_float), C.c_size_t, _P]),
    "shainet_attn_comm_data_ptr": (C.c_int, [_P, C.POINTER(_P)]),
    "shainet_attn_forward_batched_dev": (C.c_int, [_P, C.POINTER(_P), C.c_int, _P, _P, _P, _P, C.c_float,
                                                   C.c_uint, _P]),
    "shainet_attn_q8_create": (C.c_int, [_P, C.POINTER(_P), _F, C.c_int, C.c_int]),
    "shainet_attn_q8_create_raw": (C.c_int, [_P, C.POINTER(_P), _P, _F, C.c_int, C.c_int]),
    "shainet_attn_q8_wrap": (C.c_int, [_P, C.POINTER(_P), _P, _P, C.c_int, C.c_int]),
    "shainet_attn_q8_destroy": (C.c_int, [_P]),
    "shainet_attn_q8_export": (C.c_int, [_P, _P, _F]),
    "shainet_attn_q8_gemv_dev": (C.c_int, [_P, _P, _P, _P, C.c_int, _P]),
    "gemm_q8_f32": (None, [_P, _P, _P, _P, C.c_int, C.c_int, C.c_int]),
    "shainet_attn_block_create": (C.c_int, [_P, C.POINTER(_P), _P, C.c_int, _F, _P, _P, _P, _P, _F, _P, _P, _P, C.c_double]),
    "shainet_attn_block_destroy": (C.c_int, [_P]),
    "shainet_attn_block_forward_dev": (C.c_int, [_P, _P, _P, _P, C.c_int, _P]),
    "shainet_attn_block_forward_host": (C.c_int, [_P, _P, _F, _F, C.c_int]),
    "shainet_attn_decoder_create": (C.c_int, [_P, C.POINTER(_P), C.POINTER(_P), C.c_int, _F, C.c_int, _F, _P, _F, C.c_double]),
    "shainet_attn_decoder_destroy": (C.c_int, [_P]),
    "shainet_attn_decoder_run": (C.c_int, [_P, _P, C.POINTER(C.c_int32), C.c_int, _F, C.POINTER(C.c_int32)]),
    "shainet_attn_decoder_generate": (C.c_int, [_P, _P, C.POINTER(C.c_int32), C.c_int, C.c_int, C.POINTER(C.c_int32)]),
    "shainet_attn_decode_noalloc": (C.c_int, [_P, _P, _P, _P, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float, _P]),
    "kv_cache_append_f32": (None, [_P, _P, _P, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]),
    "attention_kv_f32": (None, [_P, _P, _P, _P, _P, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                C.c_float]),
}

_lib = None


class ShainetAttnError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"libshainet_attn error {code}: {message}")
        self.code = code


def load() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m shainet_b200.build` (needs nvcc, sm_100a). "
                "There is no CPU or PyTorch fallback for this path.")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)  # AttributeError if the build lost a symbol
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def check(rc: int) -> int:
    if rc < 0:
        raise ShainetAttnError(rc, load().shainet_attn_last_error().decode("utf-8", "replace"))
    return rc
