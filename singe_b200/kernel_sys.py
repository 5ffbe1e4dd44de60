"""ctypes binding of ``libsinge_kernel_sys.so`` -- the same symbols a Rust ``singe-kernel-sys`` would bind.

The library is the product; this module only declares argument types.  There is no fallback of any
kind: if the shared library has not been built, importing :func:`lib` raises, and every compute
entry point needs a CUDA device.
"""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libsinge_kernel_sys.so")

OK = 0
ERR_INVALID_LENGTH = 1
ERR_LENGTH_TOO_SHORT = 2
ERR_LENGTH_EXCEEDS_I32 = 3
ERR_NULL_POINTER = 4
ERR_SIZE_OVERFLOW = 5
ERR_UNSUPPORTED_WIDTH = 6
ERR_UNSUPPORTED_CONFIGURATION = 7
ERR_LENGTH_MISMATCH = 8
ERR_INDEX_OUT_OF_BOUNDS = 9
ERR_INVALID_ARGUMENT = 10
ERR_OUT_OF_RANGE = 11
ERR_AUTOTUNE_DURING_CAPTURE = 12
ERR_STATIC_SCRATCH_EXCEEDED = 13
ERR_CUDA_BASE = 1000

STATUS_INDEX_OUT_OF_BOUNDS = 1
STATUS_WAIT_TIMEOUT = 2

HINT_STABLE_WEIGHTS = 1
HINT_STABLE_PAGING = 2

_p = ctypes.c_void_p
_z = ctypes.c_size_t
_i = ctypes.c_int
_f = ctypes.c_float

# name -> argument types (every function returns int unless listed in _RESTYPES)
SIGNATURES = {
    "singe_kernel_sys_version": [],
    "singe_status_string": [_i],
    "singe_take_device_error": [_p],
    "singe_release_workspaces": [],
    "singe_warm_l2_with_next_launch": [_p, _z],
    "singe_kv_cache_write_bf16": [_p, _p, _p, _p, _p, _p, _p, _i, _z, _z, _z, _z, _z, _p],
    "singe_kv_cache_write_f16": [_p, _p, _p, _p, _p, _p, _p, _i, _z, _z, _z, _z, _z, _p],
    "singe_kv_cache_write_f32": [_p, _p, _p, _p, _p, _p, _p, _i, _z, _z, _z, _z, _z, _p],
    "singe_paged_kv_decode_attention_bf16": [_p, _p, _p, _p, _p, _p, _p, _z, _z, _z, _z, _z, _z, _z, _f],
    "singe_paged_kv_decode_attention_f16": [_p, _p, _p, _p, _p, _p, _p, _z, _z, _z, _z, _z, _z, _z, _f],
    "singe_paged_kv_decode_attention_f32": [_p, _p, _p, _p, _p, _p, _p, _z, _z, _z, _z, _z, _z, _z, _f],
    "singe_paged_kv_decode_attention_static_bf16": [_p, _p, _p, _p, _p, _p, _p, _z, _z, _z, _z, _z, _z, _z, _f],
    "singe_paged_kv_decode_attention_static_scratch_floats": [],
    "singe_paged_kv_decode_split_tokens": [_z, _z, _z],
    "singe_paged_kv_decode_default_splits": [_z, _z, _z, _z],
    "singe_paged_kv_decode_splitk_bf16": [_p, _p, _p, _p, _p, _p, _p, _p, _z, _z, _z, _z, _z, _z, _z, _z, _f],
    "singe_fmha_decode_splitk_reduce_f32": [_p, _p, _p, _p, _p, _p, _p, _z, _z, _z, _z, _z, _z, _f],
    "singe_splitk_reduce_f32": [_p, _p, _p, _p, _z, _z, _z, _z, _z, _z, _z, _z, _z, _z, _z],
    "singe_paged_kv_decode_splitk_reduce_bf16": [_p, _p, _p, _p, _p, _p, _p, _p, _p, _z, _z, _z, _z, _z, _z, _z, _z,
                                                 _f],
    "singe_paged_kv_decode_splitk_reduce_f16": [_p, _p, _p, _p, _p, _p, _p, _p, _p, _z, _z, _z, _z, _z, _z, _z, _z,
                                                _f],
    "singe_paged_kv_decode_step_bf16": [_p, _p, _p, _p, _p, _p, _p, _p, _p, _z, _z, _z, _z, _z, _z, _z, _z,
                                        _f, ctypes.c_uint, _p],
    "singe_paged_kv_decode_set_prefetch": [_i],
    "singe_decode_step_attention_bf16": [_p, _p, _p, _p, _p, _z, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i, _z, _z, _z, _z,
                                         _z, _z, _z, _z, _z, _f, ctypes.c_uint, _p, _p],
    "singe_rotary_paged_kv_decode_attention_bf16": [_p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i, _z, _z, _z, _z,
                                                    _z, _z, _z, _z, _z, _f, _i, _p, _f, ctypes.c_uint],
    "singe_paged_attention_bf16": [_p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i, _z, _z, _z, _z, _z, _z, _z, _z, _f, _i,
                                   _z, _p],
    "singe_paged_attention_f32": [_p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i, _z, _z, _z, _z, _z, _z, _z, _z, _f, _i,
                                  _z, _p],
    "singe_paged_attention_options_bf16": [_p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i, _z, _z, _z, _z, _z, _z, _z, _z,
                                           _f, _i, _z, _f, _p],
    "singe_paged_attention_options_f32": [_p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i, _z, _z, _z, _z, _z, _z, _z, _z,
                                          _f, _i, _z, _f, _p],
    "singe_attend_f32": [_p, _p, _p, _p, _p, _z, _z, _z, _z, _z, _z, _f, _i, _z, _f, _p],
    "singe_paged_kv_prefill_attention_bf16": [_p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _z, _z, _z, _z, _z, _z, _z, _z,
                                              _i, _f],
    "singe_paged_kv_prefill_attention_f16": [_p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _z, _z, _z, _z, _z, _z, _z, _z,
                                             _i, _f],
    "singe_paged_kv_prefill_attention_f32": [_p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _z, _z, _z, _z, _z, _z, _z, _z,
                                             _i, _f],
    "singe_ragged_kv_prefill_attention_bf16": [_p, _p, _p, _p, _p, _p, _p, _p, _p, _z, _z, _z, _z, _z, _z, _i, _f],
    "singe_ragged_kv_prefill_attention_f16": [_p, _p, _p, _p, _p, _p, _p, _p, _p, _z, _z, _z, _z, _z, _z, _i, _f],
    "singe_ragged_kv_prefill_attention_f32": [_p, _p, _p, _p, _p, _p, _p, _p, _p, _z, _z, _z, _z, _z, _z, _i, _f],
    "singe_ragged_kv_prefill_attention_cache_write_bf16": [_p, _p, _p, _p, _p, _p, _p, _p, _p, _z, _z, _z, _z, _z, _z,
                                                           _i, _f, _p, _p, _p, _p, _i, _z, _z, _p],
    "singe_fmha_prefill_lse_f32": [_p, _p, _p, _p, _p, _p, _z, _z, _z, _z, _z, _z, _f, _i],
    "singe_fmha_prefill_lse_bf16": [_p, _p, _p, _p, _p, _p, _z, _z, _z, _z, _z, _z, _f, _i],
    "singe_fmha_prefill_lse_f16": [_p, _p, _p, _p, _p, _p, _z, _z, _z, _z, _z, _z, _f, _i],
    "singe_scaled_dot_product_attention_f32": [_p, _p, _p, _p, _p, _z, _z, _z, _z, _z, _z, _f, _i, _z],
    "singe_matmul_bf16_bf16": [_p, _p, _p, _p, _z, _z, _z, _z, _z, _z, _i, _i],
    "singe_matmul_bf16_f32": [_p, _p, _p, _p, _z, _z, _z, _z, _z, _z, _i, _i],
    "singe_matmul_bf16_swiglu_bf16": [_p, _p, _p, _p, _z, _z, _z, _z, _z, _z],
    "singe_matmul_set_tuning": [_i, _i],
    "singe_matmul_set_splits": [_i],
    "singe_matmul_set_staging": [_i, _i],
    "singe_linear_bf16": [_p, _p, _p, _p, _z, _z, _z, _z, _z, _z, _i, ctypes.c_uint],
    "singe_embedding_bf16": [_p, _p, _p, _p, _i, _z, _z, _z, _p],
    "singe_add_rms_norm_bf16": [_p, _p, _p, _p, _p, _z, _z, _f],
    "singe_rotary_cache_write_bf16": [_p, _p, _p, _z, _p, _p, _p, _p, _p, _p, _p, _i, _z, _z, _z, _z, _z, _z, _z,
                                      _p],
    "singe_rotary_norm_cache_write_bf16": [_p, _p, _p, _z, _p, _p, _p, _p, _p, _p, _p, _i, _z, _z, _z, _z, _z, _z, _z,
                                           _i, _p, _i, _p, _f, _p],
    "singe_silu_mul_bf16": [_p, _p, _p, _p, _z, _z, _z],
    "singe_argmax_bf16": [_p, _p, _p, _p, _z, _z, _z, ctypes.c_int64],
    "singe_peer_buffer_create": [_z, ctypes.POINTER(ctypes.c_void_p), _p],
    "singe_peer_buffer_open": [_p, ctypes.POINTER(ctypes.c_void_p)],
    "singe_peer_buffer_close": [_p],
    "singe_peer_buffer_destroy": [_p],
    "singe_allreduce_add_rms_norm_bf16": [_p, _p, _p, _p, _p, _p, _p, _i, _i, _z, _z, _f, _p],
    "singe_allreduce_two_phase_add_rms_norm_bf16": [_p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _z, _z, _f, _i, _p],
}

_RESTYPES = {
    "singe_status_string": ctypes.c_char_p,
    "singe_paged_kv_decode_split_tokens": ctypes.c_size_t,
    "singe_paged_kv_decode_default_splits": ctypes.c_size_t,
    "singe_paged_kv_decode_attention_static_scratch_floats": ctypes.c_size_t,
}

_lib = None


def lib() -> ctypes.CDLL:
    """Loads the in-tree shared library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m singe_b200.build` "
                "(there is no CPU or PyTorch fallback for these operators)")
        handle = ctypes.CDLL(LIB_PATH)
        for name, argtypes in SIGNATURES.items():
            function = getattr(handle, name)  # AttributeError if the library lacks a declared symbol
            function.argtypes = argtypes
            function.restype = _RESTYPES.get(name, ctypes.c_int)
        _lib = handle
    return _lib


def status_string(status: int) -> str:
    return lib().singe_status_string(status).decode()
