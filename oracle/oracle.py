"""ctypes front end of the CPU restatement in ``oracle.c``.

TEST INFRASTRUCTURE ONLY.  The tests, the smoke check and the benchmark's CPU-baseline leg import
this module to check (or time) the reference's algorithm; the shipped package never does.

Every wrapper takes and returns numpy arrays and cites the reference function it restates through
the C function it calls.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")

OK = 0
INDEX_OUT_OF_BOUNDS = 1
INVALID = 2
LENGTH_TOO_SHORT = 3
SIZE_OVERFLOW = 4
LENGTH_MISMATCH = 5


def build(force: bool = False) -> str:
    """Compiles ``oracle.c`` with the Makefile beside it and returns the library path."""
    source = os.path.join(_HERE, "oracle.c")
    stale = not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(source)
    if force or stale:
        subprocess.run(["make", "-C", _HERE, "-B", "liboracle.so"], check=True, capture_output=True)
    return _LIB_PATH


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
        _lib.oracle_max_threads.restype = ctypes.c_int
        _lib.oracle_f32_to_bf16_bits.restype = ctypes.c_uint16
        _lib.oracle_f32_to_bf16_bits.argtypes = [ctypes.c_float]
    return _lib


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _ptr(a):
    return a.ctypes.data_as(ctypes.c_void_p)


_sz = ctypes.c_size_t
_f = ctypes.c_float
_i = ctypes.c_int


def set_threads(threads: int) -> None:
    lib().oracle_set_threads(_i(threads))


def max_threads() -> int:
    return int(lib().oracle_max_threads())


def round_to_bf16(values: np.ndarray) -> np.ndarray:
    """Rounds f32 values to the nearest bf16 (ties to even) and widens them back to f32."""
    out = _f32(values).copy()
    lib().oracle_round_to_bf16(_ptr(out), _sz(out.size))
    return out


def f32_to_bf16_bits(values: np.ndarray) -> np.ndarray:
    """Raw bf16 bit patterns (uint16) of f32 values, rounding to nearest even."""
    v = _f32(values)
    bits = v.view(np.uint32).astype(np.uint64)
    nan = (bits & 0x7FFFFFFF) > 0x7F800000
    rounded = ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16).astype(np.uint16)
    rounded[nan] = ((bits[nan] >> 16) | 0x40).astype(np.uint16)
    return rounded


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def paged_kv_decode_attention_f32(query, key_cache, value_cache, actual_seq_lens, block_table, *, batch, heads,
                                  kv_heads, head_dim, block_size, block_table_batch_stride, scale):
    query, key_cache, value_cache = _f32(query), _f32(key_cache), _f32(value_cache)
    lens = np.ascontiguousarray(actual_seq_lens, dtype=np.int32)
    table = np.ascontiguousarray(block_table, dtype=np.uint32)
    out = np.zeros(batch * heads * head_dim, dtype=np.float32)
    lib().oracle_paged_kv_decode_attention_f32(
        _ptr(out), _ptr(query), _ptr(key_cache), _ptr(value_cache), _ptr(lens), _ptr(table), _sz(batch), _sz(heads),
        _sz(kv_heads), _sz(head_dim), _sz(block_size), _sz(block_table_batch_stride), _f(scale))
    return out.reshape(batch, heads, head_dim)


def paged_kv_prefill_attention_f32(query, key_cache, value_cache, lens_q, lens_kv, offsets, block_table, *, batch,
                                   total_query_tokens, heads, kv_heads, head_dim, block_size,
                                   block_table_batch_stride, causal, scale):
    query, key_cache, value_cache = _f32(query), _f32(key_cache), _f32(value_cache)
    lens_q = np.ascontiguousarray(lens_q, dtype=np.int32)
    lens_kv = np.ascontiguousarray(lens_kv, dtype=np.int32)
    offsets = np.ascontiguousarray(offsets, dtype=np.int32)
    table = np.ascontiguousarray(block_table, dtype=np.uint32)
    out = np.zeros(total_query_tokens * heads * head_dim, dtype=np.float32)
    lse = np.zeros(total_query_tokens * heads, dtype=np.float32)
    lib().oracle_paged_kv_prefill_attention_f32(
        _ptr(out), _ptr(lse), _ptr(query), _ptr(key_cache), _ptr(value_cache), _ptr(lens_q), _ptr(lens_kv),
        _ptr(offsets), _ptr(table), _sz(batch), _sz(total_query_tokens), _sz(heads), _sz(kv_heads), _sz(head_dim),
        _sz(block_size), _sz(block_table_batch_stride), _i(int(causal)), _f(scale))
    return out.reshape(total_query_tokens, heads, head_dim), lse.reshape(total_query_tokens, heads)


def ragged_kv_prefill_attention_f32(query, key, value, lens_q, lens_kv, offsets, *, batch, total_query_tokens, heads,
                                    kv_heads, head_dim, causal, scale):
    query, key, value = _f32(query), _f32(key), _f32(value)
    lens_q = np.ascontiguousarray(lens_q, dtype=np.int32)
    lens_kv = np.ascontiguousarray(lens_kv, dtype=np.int32)
    offsets = np.ascontiguousarray(offsets, dtype=np.int32)
    out = np.zeros(total_query_tokens * heads * head_dim, dtype=np.float32)
    lse = np.zeros(total_query_tokens * heads, dtype=np.float32)
    lib().oracle_ragged_kv_prefill_attention_f32(
        _ptr(out), _ptr(lse), _ptr(query), _ptr(key), _ptr(value), _ptr(lens_q), _ptr(lens_kv), _ptr(offsets),
        _sz(batch), _sz(total_query_tokens), _sz(heads), _sz(kv_heads), _sz(head_dim), _i(int(causal)), _f(scale))
    return out.reshape(total_query_tokens, heads, head_dim), lse.reshape(total_query_tokens, heads)


def fmha_prefill_lse_f32(query, key, value, *, batch, query_len, key_len, heads, kv_heads, head_dim, scale, causal):
    query, key, value = _f32(query), _f32(key), _f32(value)
    out = np.zeros(batch * query_len * heads * head_dim, dtype=np.float32)
    lse = np.zeros(batch * heads * query_len, dtype=np.float32)
    lib().oracle_fmha_prefill_lse_f32(
        _ptr(out), _ptr(lse), _ptr(query), _ptr(key), _ptr(value), _sz(batch), _sz(query_len), _sz(key_len),
        _sz(heads), _sz(kv_heads), _sz(head_dim), _f(scale), _i(int(causal)))
    return out.reshape(batch, query_len, heads, head_dim), lse.reshape(batch, heads, query_len)


def sliding_window_attention_f32(query, key, value, *, batch, query_len, key_len, heads, kv_heads, head_dim,
                                 query_start, key_start, window, scale, output_scale):
    query, key, value = _f32(query), _f32(key), _f32(value)
    out = np.zeros(batch * query_len * heads * head_dim, dtype=np.float32)
    lib().oracle_sliding_window_attention_f32(
        _ptr(out), _ptr(query), _ptr(key), _ptr(value), _sz(batch), _sz(query_len), _sz(key_len), _sz(heads),
        _sz(kv_heads), _sz(head_dim), _sz(query_start), _sz(key_start), _sz(window), _f(scale), _f(output_scale))
    return out


def splitk_reduce_f32(attn, lse, *, batch, heads, splits, head_dim):
    attn, lse = _f32(attn), _f32(lse)
    out = np.zeros(batch * heads * head_dim, dtype=np.float32)
    lib().oracle_splitk_reduce_f32(_ptr(out), _ptr(attn), _ptr(lse), _sz(batch), _sz(heads), _sz(splits),
                                   _sz(head_dim))
    return out.reshape(batch, heads, head_dim)


def scaled_dot_product_attention_f32(query, key, value, *, scale, causal, window=0):
    """Dense [B, H, L, D] attention; ``key``/``value`` already carry one head per query head."""
    query, key, value = _f32(query), _f32(key), _f32(value)
    b, h, l, d = query.shape
    s, dv = key.shape[2], value.shape[3]
    out = np.zeros((b, h, l, dv), dtype=np.float32)
    lib().oracle_scaled_dot_product_attention_f32(
        _ptr(out), _ptr(query), _ptr(key), _ptr(value), _sz(b * h), _sz(l), _sz(s), _sz(d), _sz(dv), _f(scale),
        _i(int(causal)), _sz(window))
    return out


def attend_options_f32(query, key, value, *, scale, causal, window=0, softcap=0.0, sinks=None):
    """Dense [B, H, L, D] attention with the score cap and per-head sink logits of ``Tensor::attend``."""
    query, key, value = _f32(query), _f32(key), _f32(value)
    b, h, l, d = query.shape
    s, dv = key.shape[2], value.shape[3]
    out = np.zeros((b, h, l, dv), dtype=np.float32)
    sink_values = None if sinks is None else _f32(sinks)
    lib().oracle_attend_options_f32(
        _ptr(out), _ptr(query), _ptr(key), _ptr(value), _sz(b * h), _sz(l), _sz(s), _sz(d), _sz(dv), _f(scale),
        _i(int(causal)), _sz(window), _f(softcap), None if sink_values is None else _ptr(sink_values), _sz(h))
    return out


def check_paged_values(query_offsets, page_offsets, pages, last_page_lengths, *, tokens, cache_pages, page_size):
    qo = np.ascontiguousarray(query_offsets, dtype=np.int64)
    po = np.ascontiguousarray(page_offsets, dtype=np.int64)
    pg = np.ascontiguousarray(pages, dtype=np.int64)
    lp = np.ascontiguousarray(last_page_lengths, dtype=np.int64)
    return int(lib().oracle_check_paged_values(_ptr(qo), _ptr(po), _ptr(pg), _sz(pg.size), _ptr(lp), _sz(lp.size),
                                               ctypes.c_int64(tokens), ctypes.c_int64(cache_pages),
                                               ctypes.c_int64(page_size)))


def attend_paged_f32(query, key_cache, value_cache, query_offsets, page_offsets, pages, last_page_lengths, *, scale,
                     causal=True, window=0, softcap=0.0):
    """Tensor-surface paged attention: returns (status, out [T, H, D], lse [T, H] base 2)."""
    query, key_cache, value_cache = _f32(query), _f32(key_cache), _f32(value_cache)
    tokens, heads, head_dim = query.shape
    cache_pages, page_size, kv_heads, _ = key_cache.shape
    qo = np.ascontiguousarray(query_offsets, dtype=np.int64)
    po = np.ascontiguousarray(page_offsets, dtype=np.int64)
    pg = np.ascontiguousarray(pages, dtype=np.int64)
    lp = np.ascontiguousarray(last_page_lengths, dtype=np.int64)
    out = np.zeros((tokens, heads, head_dim), dtype=np.float32)
    lse = np.zeros((tokens, heads), dtype=np.float32)
    status = lib().oracle_attend_paged_options_f32(
        _ptr(out), _ptr(lse), _ptr(query), _ptr(key_cache), _ptr(value_cache), _ptr(qo), _ptr(po), _ptr(pg),
        _sz(pg.size), _ptr(lp), _sz(lp.size), _sz(tokens), _sz(heads), _sz(kv_heads), _sz(head_dim), _sz(page_size),
        _sz(cache_pages), _f(scale), _i(int(causal)), _sz(window), _f(softcap))
    return int(status), out, lse


def matmul_f32(lhs, rhs, *, rows, columns, reduction, lhs_row_stride, rhs_row_stride, transpose_lhs, transpose_rhs):
    lhs, rhs = _f32(lhs), _f32(rhs)
    out = np.zeros(rows * columns, dtype=np.float32)
    lib().oracle_matmul_f32(_ptr(out), _ptr(lhs), _ptr(rhs), _sz(rows), _sz(columns), _sz(reduction),
                            _sz(lhs_row_stride), _sz(rhs_row_stride), _i(int(transpose_lhs)), _i(int(transpose_rhs)))
    return out


def matmul_strided_f32(lhs, rhs, output, *, rows, columns, reduction, lhs_strides, rhs_strides):
    """Returns the status; ``output`` (f32, rows*columns) is overwritten in place."""
    lhs, rhs = _f32(lhs), _f32(rhs)
    assert output.dtype == np.float32 and output.flags.c_contiguous
    return int(lib().oracle_matmul_strided_f32(
        _ptr(lhs), _sz(lhs.size), _ptr(rhs), _sz(rhs.size), _ptr(output), _sz(output.size), _sz(rows), _sz(columns),
        _sz(reduction), _sz(lhs_strides[0]), _sz(lhs_strides[1]), _sz(rhs_strides[0]), _sz(rhs_strides[1])))


def linear_bf16(x_bits, w_bits, *, m, n, k):
    """Y = X . W^T on raw bf16 bits, rounded once to bf16 (returns uint16 bits [m, n])."""
    x = np.ascontiguousarray(x_bits, dtype=np.uint16)
    w = np.ascontiguousarray(w_bits, dtype=np.uint16)
    y = np.zeros(m * n, dtype=np.uint16)
    lib().oracle_linear_bf16(_ptr(y), _ptr(x), _ptr(w), _sz(m), _sz(n), _sz(k))
    return y.reshape(m, n)


def linear_bf16_f32(x_bits, w_bits, *, m, n, k):
    x = np.ascontiguousarray(x_bits, dtype=np.uint16)
    w = np.ascontiguousarray(w_bits, dtype=np.uint16)
    y = np.zeros(m * n, dtype=np.float32)
    lib().oracle_linear_bf16_f32(_ptr(y), _ptr(x), _ptr(w), _sz(m), _sz(n), _sz(k))
    return y.reshape(m, n)


def kv_cache_write(cache: np.ndarray, rows: np.ndarray, write_pages, write_slots) -> int:
    """In-place slot-mapped write of ``rows`` [T, ...] into ``cache`` [P, S, ...]; returns the status."""
    assert cache.flags.c_contiguous and rows.flags.c_contiguous and cache.dtype == rows.dtype
    pages, page_size = cache.shape[0], cache.shape[1]
    row_bytes = int(np.prod(cache.shape[2:])) * cache.dtype.itemsize
    wp = np.ascontiguousarray(write_pages, dtype=np.int64)
    ws = np.ascontiguousarray(write_slots, dtype=np.int64)
    return int(lib().oracle_kv_cache_write(_ptr(cache), _ptr(rows), _ptr(wp), _ptr(ws), _sz(wp.size), _sz(pages),
                                           _sz(page_size), _sz(row_bytes)))


def rms_norm_f32(x, weight, eps):
    x, weight = _f32(x), _f32(weight)
    rows, width = x.shape
    out = np.zeros_like(x)
    lib().oracle_rms_norm_f32(_ptr(out), _ptr(x), _ptr(weight), _sz(rows), _sz(width), _f(eps))
    return out
