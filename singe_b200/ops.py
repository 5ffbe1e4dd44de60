"""Host-side mirror of the reference's operator API over the C ABI, for tests, benches and the decode step.

Names, argument order and error behaviour follow ``singe_kernel::cuda::{attention, matmul}`` and the
``singe::Tensor`` ops they serve: a config object validates dimensions (``Error::InvalidLength``,
``LengthExceedsI32``), buffer lengths are checked as "at least" (``LengthTooShort``), and the launch is
enqueue-only on the given stream.  Tensors are torch CUDA tensors used purely as device buffers; every
function hands raw pointers to ``libsinge_kernel_sys.so``.  Nothing here computes anything itself.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from . import kernel_sys as ks


class SingeError(RuntimeError):
    """A non-zero status of the C ABI; ``code`` is one of the ``ERR_*`` constants of ``kernel_sys``."""

    def __init__(self, code: int, where: str = ""):
        self.code = code
        try:
            text = ks.status_string(code)
        except Exception:  # pragma: no cover - library missing
            text = "?"
        super().__init__(f"{where}: status {code} ({text})" if where else f"status {code} ({text})")


def _check(code: int, where: str) -> None:
    if code != ks.OK:
        raise SingeError(code, where)


def _stream(stream) -> int:
    if stream is None:
        stream = torch.cuda.current_stream()
    return int(stream.cuda_stream)


def _ptr(tensor) -> int | None:
    return None if tensor is None else int(tensor.data_ptr())


def _ensure(tensor: torch.Tensor, minimum: int, name: str) -> None:
    """ensure_len_at_least (singe-kernel/src/cuda/attention/mod.rs): storage may be longer, never shorter."""
    if tensor.numel() < minimum:
        raise SingeError(ks.ERR_LENGTH_TOO_SHORT, f"{name}: minimum {minimum}, actual {tensor.numel()}")


_I32_MAX = 2**31 - 1


def _suffix(dtype: torch.dtype) -> str:
    return {torch.bfloat16: "bf16", torch.float16: "f16", torch.float32: "f32"}[dtype]


# ------------------------------------------------------------------------------------------------
# configs (singe-kernel/src/cuda/attention/mod.rs:81-123)
# ------------------------------------------------------------------------------------------------

@dataclass(frozen=True)
class PagedKvDecodeAttentionConfig:
    batch: int
    heads: int
    kv_heads: int
    head_dim: int
    block_size: int
    physical_blocks: int
    block_table_batch_stride: int
    scale: float

    @classmethod
    def contiguous(cls, batch, heads, kv_heads, head_dim, block_size, physical_blocks, block_table_batch_stride,
                   scale):
        config = cls(batch, heads, kv_heads, head_dim, block_size, physical_blocks, block_table_batch_stride, scale)
        config.validate()
        return config

    def validate(self) -> None:
        # validate_paged_kv_decode_attention_config (singe-kernel/src/cuda/attention/mod.rs:2963-2985)
        dims = (self.batch, self.heads, self.kv_heads, self.head_dim, self.block_size, self.physical_blocks,
                self.block_table_batch_stride)
        if any(d == 0 for d in dims) or self.heads % self.kv_heads != 0 or not math.isfinite(self.scale):
            raise SingeError(ks.ERR_INVALID_LENGTH, "PagedKvDecodeAttentionConfig")
        if any(d > _I32_MAX for d in dims):
            raise SingeError(ks.ERR_LENGTH_EXCEEDS_I32, "PagedKvDecodeAttentionConfig")

    def validate_lengths(self, out, query, key_cache, value_cache, actual_seq_lens, block_table) -> None:
        self.validate()
        output_len = self.batch * self.heads * self.head_dim
        cache_len = self.physical_blocks * self.block_size * self.kv_heads * self.head_dim
        _ensure(out, output_len, "out")
        _ensure(query, output_len, "query")
        _ensure(key_cache, cache_len, "key_cache")
        _ensure(value_cache, cache_len, "value_cache")
        _ensure(actual_seq_lens, self.batch, "actual_seq_lens")
        _ensure(block_table, self.batch * self.block_table_batch_stride, "block_table")


@dataclass(frozen=True)
class PagedKvPrefillAttentionConfig:
    batch: int
    total_query_tokens: int
    heads: int
    kv_heads: int
    head_dim: int
    block_size: int
    physical_blocks: int
    block_table_batch_stride: int
    causal: bool
    scale: float

    def validate(self) -> None:
        dims = (self.batch, self.total_query_tokens, self.heads, self.kv_heads, self.head_dim, self.block_size,
                self.physical_blocks, self.block_table_batch_stride)
        if any(d == 0 for d in dims) or self.heads % self.kv_heads != 0 or not math.isfinite(self.scale):
            raise SingeError(ks.ERR_INVALID_LENGTH, "PagedKvPrefillAttentionConfig")
        if any(d > _I32_MAX for d in dims):
            raise SingeError(ks.ERR_LENGTH_EXCEEDS_I32, "PagedKvPrefillAttentionConfig")


@dataclass(frozen=True)
class RaggedKvPrefillAttentionConfig:
    batch: int
    total_query_tokens: int
    total_kv_tokens: int
    heads: int
    kv_heads: int
    head_dim: int
    causal: bool
    scale: float

    def validate(self) -> None:
        dims = (self.batch, self.total_query_tokens, self.total_kv_tokens, self.heads, self.kv_heads, self.head_dim)
        if any(d == 0 for d in dims) or self.heads % self.kv_heads != 0 or not math.isfinite(self.scale):
            raise SingeError(ks.ERR_INVALID_LENGTH, "RaggedKvPrefillAttentionConfig")
        if any(d > _I32_MAX for d in dims):
            raise SingeError(ks.ERR_LENGTH_EXCEEDS_I32, "RaggedKvPrefillAttentionConfig")


@dataclass(frozen=True)
class MatmulConfig:
    """singe-kernel/src/cuda/matmul.rs:45-55; ``row_major_transposed_rhs`` is the linear-layer layout (:218-230)."""
    rows: int
    columns: int
    reduction: int
    lhs_row_stride: int
    rhs_row_stride: int
    output_row_stride: int
    transpose_lhs: bool
    transpose_rhs: bool

    @classmethod
    def row_major(cls, rows, columns, reduction):
        """lhs [M, K], rhs [K, N] (:190-202)."""
        return cls(rows, columns, reduction, reduction, columns, columns, False, False)

    @classmethod
    def row_major_transposed_lhs(cls, rows, columns, reduction):
        """lhs [K, M], rhs [K, N] (:204-216)."""
        return cls(rows, columns, reduction, rows, columns, columns, True, False)

    @classmethod
    def row_major_transposed_rhs(cls, rows, columns, reduction):
        return cls(rows, columns, reduction, reduction, reduction, columns, False, True)

    @classmethod
    def row_major_transposed_inputs(cls, rows, columns, reduction):
        """lhs [K, M], rhs [N, K] (:232-244)."""
        return cls(rows, columns, reduction, rows, reduction, columns, True, True)


# ------------------------------------------------------------------------------------------------
# operators
# ------------------------------------------------------------------------------------------------

def kv_cache_write(key_cache, value_cache, keys, values, write_pages, write_slots, status=None, stream=None):
    """KvCache::write (singe/src/nn/decode/cache.rs:97-101): caches [P,S,G,D], rows [T,G,D], indices [T] i32/i64."""
    pages, page_size, kv_heads, head_dim = key_cache.shape
    tokens = keys.shape[0]
    width = write_pages.element_size()
    assert write_slots.element_size() == width and width in (4, 8)
    fn = getattr(ks.lib(), f"singe_kv_cache_write_{_suffix(key_cache.dtype)}")
    _check(fn(_stream(stream), _ptr(key_cache), _ptr(value_cache), _ptr(keys), _ptr(values), _ptr(write_pages),
              _ptr(write_slots), width, tokens, kv_heads, head_dim, pages, page_size, _ptr(status)),
           "kv_cache_write")


def paged_kv_decode_attention(out, query, key_cache, value_cache, actual_seq_lens, block_table,
                              config: PagedKvDecodeAttentionConfig, stream=None):
    """singe_kernel::cuda::attention::paged_kv_decode_attention_{f32,f16,bf16} (paged.rs:118-249)."""
    config.validate_lengths(out, query, key_cache, value_cache, actual_seq_lens, block_table)
    fn = getattr(ks.lib(), f"singe_paged_kv_decode_attention_{_suffix(query.dtype)}")
    _check(fn(_stream(stream), _ptr(out), _ptr(query), _ptr(key_cache), _ptr(value_cache), _ptr(actual_seq_lens),
              _ptr(block_table), config.batch, config.heads, config.kv_heads, config.head_dim, config.block_size,
              config.physical_blocks, config.block_table_batch_stride, config.scale),
           "paged_kv_decode_attention")


def paged_kv_decode_split_tokens(key_len_bound: int, max_splits: int, block_size: int) -> int:
    return int(ks.lib().singe_paged_kv_decode_split_tokens(key_len_bound, max_splits, block_size))


def paged_kv_decode_splitk(attn_scratch, lse_scratch, query, key_cache, value_cache, actual_seq_lens, block_table,
                           config: PagedKvDecodeAttentionConfig, max_splits: int, stream=None):
    """Partials only: attn [B,H,max_splits,D] f32, lse [B,H,max_splits] f32 (natural log)."""
    config.validate()
    rows = config.batch * config.heads * max_splits
    _ensure(attn_scratch, rows * config.head_dim, "attn_scratch")
    _ensure(lse_scratch, rows, "lse_scratch")
    _check(ks.lib().singe_paged_kv_decode_splitk_bf16(
        _stream(stream), _ptr(attn_scratch), _ptr(lse_scratch), _ptr(query), _ptr(key_cache), _ptr(value_cache),
        _ptr(actual_seq_lens), _ptr(block_table), config.batch, config.heads, config.kv_heads, config.head_dim,
        config.block_size, config.physical_blocks, config.block_table_batch_stride, max_splits, config.scale),
        "paged_kv_decode_splitk")


def paged_kv_decode_splitk_reduce(out, attn_scratch, lse_scratch, query, key_cache, value_cache, actual_seq_lens,
                                  block_table, config: PagedKvDecodeAttentionConfig, max_splits: int, stream=None):
    """Decode + combine with caller scratch (the shape of fmha_decode_splitk_reduce_f32, fmha.rs:1155-1251)."""
    config.validate_lengths(out, query, key_cache, value_cache, actual_seq_lens, block_table)
    if max_splits == 0:
        raise SingeError(ks.ERR_INVALID_LENGTH, "max_splits")
    rows = config.batch * config.heads * max_splits
    _ensure(attn_scratch, rows * config.head_dim, "attn_scratch")
    _ensure(lse_scratch, rows, "lse_scratch")
    fn = getattr(ks.lib(), f"singe_paged_kv_decode_splitk_reduce_{_suffix(query.dtype)}")
    _check(fn(_stream(stream), _ptr(out), _ptr(attn_scratch), _ptr(lse_scratch), _ptr(query), _ptr(key_cache),
              _ptr(value_cache), _ptr(actual_seq_lens), _ptr(block_table), config.batch, config.heads,
              config.kv_heads, config.head_dim, config.block_size, config.physical_blocks,
              config.block_table_batch_stride, max_splits, config.scale),
           "paged_kv_decode_splitk_reduce")


def splitk_reduce_f32(out, attn_splitk, lse_splitk, batch, heads, splits, head_dim, stream=None):
    """splitk_reduce_f32 with SplitKReduceConfig::contiguous strides (mod.rs:2320-2340)."""
    _ensure(attn_splitk, batch * heads * splits * head_dim, "attn_splitk")
    _ensure(lse_splitk, batch * heads * splits, "lse_splitk")
    _ensure(out, batch * heads * head_dim, "out")
    _check(ks.lib().singe_splitk_reduce_f32(
        _stream(stream), _ptr(out), _ptr(attn_splitk), _ptr(lse_splitk), batch, heads, splits, head_dim,
        heads * splits * head_dim, splits * head_dim, head_dim, heads * splits, splits, heads * head_dim, head_dim),
        "splitk_reduce_f32")


def paged_attention(query, key_cache, value_cache, query_offsets, page_offsets, pages, last_page_lengths, *,
                    scale=None, causal=True, window=0, status=None, stream=None):
    """Tensor::paged_attention (singe/src/tensor/neural.rs:405-457): returns (out [T,H,D], lse [T,H] base 2)."""
    tokens, heads, head_dim = query.shape
    cache_pages, page_size, kv_heads, _ = key_cache.shape
    if scale is None:
        scale = 1.0 / math.sqrt(head_dim)
    out = torch.zeros_like(query)
    lse = torch.full((tokens, heads), float("-inf"), dtype=torch.float32, device=query.device)
    width = query_offsets.element_size()
    fn = getattr(ks.lib(), f"singe_paged_attention_{_suffix(query.dtype)}")
    _check(fn(_stream(stream), _ptr(out), _ptr(lse), _ptr(query), _ptr(key_cache), _ptr(value_cache),
              _ptr(query_offsets), _ptr(page_offsets), _ptr(pages), _ptr(last_page_lengths), width, tokens, heads,
              kv_heads, head_dim, page_size, cache_pages, last_page_lengths.numel(), pages.numel(), scale,
              int(causal), window, _ptr(status)),
           "paged_attention")
    return out, lse


def paged_kv_prefill_attention(out, lse, query, key_cache, value_cache, lens_q, lens_kv, offsets, block_table,
                               config: PagedKvPrefillAttentionConfig, stream=None):
    """paged_kv_prefill_attention_{f32,bf16} (singe-kernel/src/cuda/attention/paged.rs:256-420)."""
    config.validate()
    _ensure(out, config.total_query_tokens * config.heads * config.head_dim, "out")
    _ensure(lse, config.total_query_tokens * config.heads, "lse")
    _ensure(query, config.total_query_tokens * config.heads * config.head_dim, "query")
    for name, t in (("lens_q", lens_q), ("lens_kv", lens_kv), ("offsets", offsets)):
        _ensure(t, config.batch, name)
    _ensure(block_table, config.batch * config.block_table_batch_stride, "block_table")
    fn = getattr(ks.lib(), f"singe_paged_kv_prefill_attention_{_suffix(query.dtype)}")
    _check(fn(_stream(stream), _ptr(out), _ptr(lse), _ptr(query), _ptr(key_cache), _ptr(value_cache), _ptr(lens_q),
              _ptr(lens_kv), _ptr(offsets), _ptr(block_table), config.batch, config.total_query_tokens, config.heads,
              config.kv_heads, config.head_dim, config.block_size, config.physical_blocks,
              config.block_table_batch_stride, int(config.causal), config.scale),
           "paged_kv_prefill_attention")


def ragged_kv_prefill_attention(out, lse, query, key, value, lens_q, lens_kv, offsets,
                                config: RaggedKvPrefillAttentionConfig, stream=None, cache_write=None):
    """ragged_kv_prefill_attention_{f32,bf16} (paged.rs:422-576).

    ``cache_write`` = (key_cache, value_cache, write_pages, write_slots, status) also stores every K/V row
    into the paged caches in the same call.
    """
    config.validate()
    _ensure(out, config.total_query_tokens * config.heads * config.head_dim, "out")
    _ensure(lse, config.total_query_tokens * config.heads, "lse")
    _ensure(query, config.total_query_tokens * config.heads * config.head_dim, "query")
    _ensure(key, config.total_kv_tokens * config.kv_heads * config.head_dim, "key")
    _ensure(value, config.total_kv_tokens * config.kv_heads * config.head_dim, "value")
    for name, t in (("lens_q", lens_q), ("lens_kv", lens_kv), ("offsets", offsets)):
        _ensure(t, config.batch, name)
    if cache_write is None:
        fn = getattr(ks.lib(), f"singe_ragged_kv_prefill_attention_{_suffix(query.dtype)}")
        _check(fn(_stream(stream), _ptr(out), _ptr(lse), _ptr(query), _ptr(key), _ptr(value), _ptr(lens_q),
                  _ptr(lens_kv), _ptr(offsets), config.batch, config.total_query_tokens, config.total_kv_tokens,
                  config.heads, config.kv_heads, config.head_dim, int(config.causal), config.scale),
               "ragged_kv_prefill_attention")
        return
    key_cache, value_cache, write_pages, write_slots, status = cache_write
    pages, page_size = key_cache.shape[0], key_cache.shape[1]
    _check(ks.lib().singe_ragged_kv_prefill_attention_cache_write_bf16(
        _stream(stream), _ptr(out), _ptr(lse), _ptr(query), _ptr(key), _ptr(value), _ptr(lens_q), _ptr(lens_kv),
        _ptr(offsets), config.batch, config.total_query_tokens, config.total_kv_tokens, config.heads, config.kv_heads,
        config.head_dim, int(config.causal), config.scale, _ptr(key_cache), _ptr(value_cache), _ptr(write_pages),
        _ptr(write_slots), write_pages.element_size(), pages, page_size, _ptr(status)),
        "ragged_kv_prefill_attention_cache_write")


def fmha_prefill_lse(out, lse, query, key, value, *, batch, query_len, key_len, heads, kv_heads, head_dim, scale,
                     causal, stream=None):
    """fmha_prefill_lse_{f32,bf16} (singe-kernel/src/cuda/attention/fmha.rs:48-790): BSHD, lse [B,H,L] natural."""
    fn = getattr(ks.lib(), f"singe_fmha_prefill_lse_{_suffix(query.dtype)}")
    _check(fn(_stream(stream), _ptr(out), _ptr(lse), _ptr(query), _ptr(key), _ptr(value), batch, query_len, key_len,
              heads, kv_heads, head_dim, scale, int(causal)), "fmha_prefill_lse")


def scaled_dot_product_attention(query, key, value, *, scale=None, causal=False, window=0, stream=None):
    """Tensor::attend (singe/src/tensor/neural.rs:25-183): [B,H,L,D] over [B,G,S,D], f32."""
    batch, heads, query_len, head_dim = query.shape
    kv_heads, key_len = key.shape[1], key.shape[2]
    if scale is None:
        scale = 1.0 / math.sqrt(head_dim)
    out = torch.empty_like(query)
    _check(ks.lib().singe_scaled_dot_product_attention_f32(
        _stream(stream), _ptr(out), _ptr(query), _ptr(key), _ptr(value), batch, heads, kv_heads, query_len, key_len,
        head_dim, scale, int(causal), window), "scaled_dot_product_attention")
    return out


def matmul_bf16(out, lhs, rhs, config: MatmulConfig, stream=None):
    """matmul_bf16_f32 when ``out`` is f32 (singe-kernel/src/cuda/matmul.rs:1302-1339), else the Tensor-surface
    bf16 result of Linear::forward (singe/src/nn/layers/linear/mod.rs:49-70)."""
    name = "singe_matmul_bf16_f32" if out.dtype == torch.float32 else "singe_matmul_bf16_bf16"
    _check(getattr(ks.lib(), name)(
        _stream(stream), _ptr(out), _ptr(lhs), _ptr(rhs), config.rows, config.columns, config.reduction,
        config.lhs_row_stride, config.rhs_row_stride, config.output_row_stride, int(config.transpose_lhs),
        int(config.transpose_rhs)), name)


def linear(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor | None = None, stream=None) -> torch.Tensor:
    """Linear::forward: y[M,N] = x[M,K] . weight[N,K]^T in bf16 with f32 accumulation."""
    m, k = x.shape
    n = weight.shape[0]
    if out is None:
        out = torch.empty((m, n), dtype=torch.bfloat16, device=x.device)
    matmul_bf16(out, x, weight, MatmulConfig(m, n, k, x.stride(0), weight.stride(0), out.stride(0), False, True),
                stream)
    return out


def take_device_error() -> int:
    """Reads and clears the library's sticky device error word (synchronises)."""
    import ctypes

    word = ctypes.c_uint32(0)
    _check(ks.lib().singe_take_device_error(ctypes.byref(word)), "take_device_error")
    return int(word.value)
