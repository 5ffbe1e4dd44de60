// Host-side mirror of the reference's operator API for the attention-and-linear path, in C++ over the C ABI.
//
// The reference's host layer is Rust (`singe_kernel::cuda::{attention, matmul}`): config structs with a
// validating constructor, `validate_lengths` on the element counts of every buffer ("at least" semantics), and
// thin `unsafe fn` wrappers that enqueue one launch.  This header restates that layer with the same names,
// argument meaning and error variants, so a test written against the reference's validation tests
// (singe-kernel/src/cuda/attention/tests.rs:283-400) reads the same here.  It owns no device memory and
// launches nothing itself: every operator forwards to a `singe_*` symbol of libsinge_kernel_sys.so.
#pragma once

#include <cmath>
#include <cstddef>
#include <cstdint>
#include <initializer_list>

#include "../../include/singe_kernel_sys.h"

namespace singe_kernel {

// singe-kernel/src/error.rs:13-189 (the variants this path can return)
enum class Error : int {
    Ok = SINGE_OK,
    InvalidLength = SINGE_ERR_INVALID_LENGTH,
    LengthTooShort = SINGE_ERR_LENGTH_TOO_SHORT,
    LengthExceedsI32 = SINGE_ERR_LENGTH_EXCEEDS_I32,
    NullPointer = SINGE_ERR_NULL_POINTER,
    SizeOverflow = SINGE_ERR_SIZE_OVERFLOW,
    UnsupportedWidth = SINGE_ERR_UNSUPPORTED_WIDTH,
    UnsupportedConfiguration = SINGE_ERR_UNSUPPORTED_CONFIGURATION,
    LengthMismatch = SINGE_ERR_LENGTH_MISMATCH,
    Cuda = SINGE_ERR_CUDA_BASE,
};

inline Error from_sys(int status) {
    if (status >= SINGE_ERR_CUDA_BASE) return Error::Cuda;
    return static_cast<Error>(status);
}

// A device buffer as the reference's DeviceInput / DeviceOutput present it: a raw pointer and an element count.
template <typename T>
struct DeviceSlice {
    T *ptr;
    size_t len;
};

namespace detail {

constexpr size_t kI32Max = 2147483647u;

inline bool checked_mul(size_t a, size_t b, size_t &out) { return !__builtin_mul_overflow(a, b, &out); }

// checked_element_count (singe-kernel/src/cuda/attention/mod.rs): product or SizeOverflow
inline Error element_count(size_t a, size_t b, size_t &out) {
    return checked_mul(a, b, out) ? Error::Ok : Error::SizeOverflow;
}

inline Error ensure_len_at_least(size_t actual, size_t minimum) {
    return actual < minimum ? Error::LengthTooShort : Error::Ok;
}

inline bool fits_i32(size_t value) { return value <= kI32Max; }

}  // namespace detail

#define SINGE_HOST_TRY(expr)                                  \
    do {                                                      \
        ::singe_kernel::Error singe_host_error_ = (expr);     \
        if (singe_host_error_ != ::singe_kernel::Error::Ok) { \
            return singe_host_error_;                         \
        }                                                     \
    } while (0)

// ---- PagedKvDecodeAttentionConfig: singe-kernel/src/cuda/attention/mod.rs:81-90, 686-744, 2963-2985 ----
struct PagedKvDecodeAttentionConfig {
    size_t batch, heads, kv_heads, head_dim, block_size, physical_blocks, block_table_batch_stride;
    float scale;

    static Error contiguous(size_t batch, size_t heads, size_t kv_heads, size_t head_dim, size_t block_size,
                            size_t physical_blocks, size_t block_table_batch_stride, float scale,
                            PagedKvDecodeAttentionConfig &out) {
        out = {batch, heads, kv_heads, head_dim, block_size, physical_blocks, block_table_batch_stride, scale};
        return out.validate();
    }

    Error validate() const {
        if (batch == 0 || heads == 0 || kv_heads == 0 || head_dim == 0 || block_size == 0 || physical_blocks == 0 ||
            block_table_batch_stride == 0 || heads % kv_heads != 0 || !std::isfinite(scale)) {
            return Error::InvalidLength;
        }
        for (size_t extent : {batch, heads, kv_heads, head_dim, block_size, physical_blocks, block_table_batch_stride}) {
            if (!detail::fits_i32(extent)) return Error::LengthExceedsI32;
        }
        return Error::Ok;
    }

    Error validate_lengths(size_t out_len, size_t query_len, size_t key_cache_len, size_t value_cache_len,
                           size_t actual_seq_lens_len, size_t block_table_len) const {
        SINGE_HOST_TRY(validate());
        size_t output_len, cache_block_len, cache_len, table_len, tmp;
        SINGE_HOST_TRY(detail::element_count(batch, heads, tmp));
        SINGE_HOST_TRY(detail::element_count(tmp, head_dim, output_len));
        SINGE_HOST_TRY(detail::element_count(block_size, kv_heads, tmp));
        SINGE_HOST_TRY(detail::element_count(tmp, head_dim, cache_block_len));
        SINGE_HOST_TRY(detail::element_count(physical_blocks, cache_block_len, cache_len));
        SINGE_HOST_TRY(detail::ensure_len_at_least(out_len, output_len));
        SINGE_HOST_TRY(detail::ensure_len_at_least(query_len, output_len));
        SINGE_HOST_TRY(detail::ensure_len_at_least(key_cache_len, cache_len));
        SINGE_HOST_TRY(detail::ensure_len_at_least(value_cache_len, cache_len));
        SINGE_HOST_TRY(detail::ensure_len_at_least(actual_seq_lens_len, batch));
        SINGE_HOST_TRY(detail::element_count(batch, block_table_batch_stride, table_len));
        return detail::ensure_len_at_least(block_table_len, table_len);
    }
};

// ---- PagedKvPrefillAttentionConfig: mod.rs:97-110, 746-818, 2987-3011 ----
struct PagedKvPrefillAttentionConfig {
    size_t batch, total_query_tokens, heads, kv_heads, head_dim, block_size, physical_blocks, block_table_batch_stride;
    bool causal;
    float scale;

    static Error contiguous(size_t batch, size_t total_query_tokens, size_t heads, size_t kv_heads, size_t head_dim,
                            size_t block_size, size_t physical_blocks, size_t block_table_batch_stride, bool causal,
                            float scale, PagedKvPrefillAttentionConfig &out) {
        out = {batch, total_query_tokens, heads, kv_heads, head_dim, block_size, physical_blocks,
               block_table_batch_stride, causal, scale};
        return out.validate();
    }

    Error validate() const {
        if (batch == 0 || total_query_tokens == 0 || heads == 0 || kv_heads == 0 || head_dim == 0 || block_size == 0 ||
            physical_blocks == 0 || block_table_batch_stride == 0 || heads % kv_heads != 0 || !std::isfinite(scale)) {
            return Error::InvalidLength;
        }
        for (size_t extent : {batch, total_query_tokens, heads, kv_heads, head_dim, block_size, physical_blocks,
                              block_table_batch_stride}) {
            if (!detail::fits_i32(extent)) return Error::LengthExceedsI32;
        }
        return Error::Ok;
    }

    Error validate_lengths(size_t out_len, size_t lse_len, size_t query_len, size_t key_cache_len,
                           size_t value_cache_len, size_t lens_q_len, size_t lens_kv_len, size_t offsets_len,
                           size_t block_table_len) const {
        SINGE_HOST_TRY(validate());
        size_t output_len, lse_needed, cache_block_len, cache_len, table_len, tmp;
        SINGE_HOST_TRY(detail::element_count(total_query_tokens, heads, lse_needed));
        SINGE_HOST_TRY(detail::element_count(lse_needed, head_dim, output_len));
        SINGE_HOST_TRY(detail::element_count(block_size, kv_heads, tmp));
        SINGE_HOST_TRY(detail::element_count(tmp, head_dim, cache_block_len));
        SINGE_HOST_TRY(detail::element_count(physical_blocks, cache_block_len, cache_len));
        SINGE_HOST_TRY(detail::ensure_len_at_least(out_len, output_len));
        SINGE_HOST_TRY(detail::ensure_len_at_least(lse_len, lse_needed));
        SINGE_HOST_TRY(detail::ensure_len_at_least(query_len, output_len));
        SINGE_HOST_TRY(detail::ensure_len_at_least(key_cache_len, cache_len));
        SINGE_HOST_TRY(detail::ensure_len_at_least(value_cache_len, cache_len));
        SINGE_HOST_TRY(detail::ensure_len_at_least(lens_q_len, batch));
        SINGE_HOST_TRY(detail::ensure_len_at_least(lens_kv_len, batch));
        SINGE_HOST_TRY(detail::ensure_len_at_least(offsets_len, batch));
        SINGE_HOST_TRY(detail::element_count(batch, block_table_batch_stride, table_len));
        return detail::ensure_len_at_least(block_table_len, table_len);
    }
};

// ---- RaggedKvPrefillAttentionConfig: mod.rs:112-123, 820-882, 3013-3040 ----
struct RaggedKvPrefillAttentionConfig {
    size_t batch, total_query_tokens, total_kv_tokens, heads, kv_heads, head_dim;
    bool causal;
    float scale;

    static Error contiguous(size_t batch, size_t total_query_tokens, size_t total_kv_tokens, size_t heads,
                            size_t kv_heads, size_t head_dim, bool causal, float scale,
                            RaggedKvPrefillAttentionConfig &out) {
        out = {batch, total_query_tokens, total_kv_tokens, heads, kv_heads, head_dim, causal, scale};
        return out.validate();
    }

    Error validate() const {
        if (batch == 0 || total_query_tokens == 0 || total_kv_tokens == 0 || heads == 0 || kv_heads == 0 ||
            head_dim == 0 || heads % kv_heads != 0 || !std::isfinite(scale)) {
            return Error::InvalidLength;
        }
        for (size_t extent : {batch, total_query_tokens, total_kv_tokens, heads, kv_heads, head_dim}) {
            if (!detail::fits_i32(extent)) return Error::LengthExceedsI32;
        }
        return Error::Ok;
    }

    Error validate_lengths(size_t out_len, size_t lse_len, size_t query_len, size_t key_len, size_t value_len,
                           size_t lens_q_len, size_t lens_kv_len, size_t offsets_len) const {
        SINGE_HOST_TRY(validate());
        size_t output_len, lse_needed, kv_len, tmp;
        SINGE_HOST_TRY(detail::element_count(total_query_tokens, heads, lse_needed));
        SINGE_HOST_TRY(detail::element_count(lse_needed, head_dim, output_len));
        SINGE_HOST_TRY(detail::element_count(total_kv_tokens, kv_heads, tmp));
        SINGE_HOST_TRY(detail::element_count(tmp, head_dim, kv_len));
        SINGE_HOST_TRY(detail::ensure_len_at_least(out_len, output_len));
        SINGE_HOST_TRY(detail::ensure_len_at_least(lse_len, lse_needed));
        SINGE_HOST_TRY(detail::ensure_len_at_least(query_len, output_len));
        SINGE_HOST_TRY(detail::ensure_len_at_least(key_len, kv_len));
        SINGE_HOST_TRY(detail::ensure_len_at_least(value_len, kv_len));
        SINGE_HOST_TRY(detail::ensure_len_at_least(lens_q_len, batch));
        SINGE_HOST_TRY(detail::ensure_len_at_least(lens_kv_len, batch));
        return detail::ensure_len_at_least(offsets_len, batch);
    }
};

// ---- SplitKReduceConfig: mod.rs:2320-2370 (contiguous strides and padded-stride reach) ----
struct SplitKReduceConfig {
    size_t batch, heads, splits, head_dim;
    size_t attn_batch_stride, attn_head_stride, attn_split_stride, lse_batch_stride, lse_head_stride,
        output_batch_stride, output_head_stride;

    static Error contiguous(size_t batch, size_t heads, size_t splits, size_t head_dim, SplitKReduceConfig &out) {
        size_t split_values, output_values, attn_batch, lse_batch;
        SINGE_HOST_TRY(detail::element_count(splits, head_dim, split_values));
        SINGE_HOST_TRY(detail::element_count(heads, head_dim, output_values));
        SINGE_HOST_TRY(detail::element_count(heads, split_values, attn_batch));
        SINGE_HOST_TRY(detail::element_count(heads, splits, lse_batch));
        out = {batch, heads, splits, head_dim, attn_batch, split_values, head_dim, lse_batch, splits, output_values,
               head_dim};
        return Error::Ok;
    }

    // Reach of a [batch][heads][splits][head_dim] view with the configured strides: last element + 1.
    Error validate_lengths(size_t out_len, size_t attn_len, size_t lse_len) const {
        if (batch == 0 || heads == 0 || splits == 0 || head_dim == 0) return Error::InvalidLength;
        const size_t attn_reach = (batch - 1) * attn_batch_stride + (heads - 1) * attn_head_stride +
                                  (splits - 1) * attn_split_stride + head_dim;
        const size_t lse_reach = (batch - 1) * lse_batch_stride + (heads - 1) * lse_head_stride + splits;
        const size_t out_reach = (batch - 1) * output_batch_stride + (heads - 1) * output_head_stride + head_dim;
        SINGE_HOST_TRY(detail::ensure_len_at_least(attn_len, attn_reach));
        SINGE_HOST_TRY(detail::ensure_len_at_least(lse_len, lse_reach));
        return detail::ensure_len_at_least(out_len, out_reach);
    }
};

// ---- MatmulConfig: singe-kernel/src/cuda/matmul.rs:45-55, 218-230; validate_matmul :2977-3020 ----
struct MatmulConfig {
    size_t rows, columns, reduction, lhs_row_stride, rhs_row_stride, output_row_stride;
    bool transpose_lhs, transpose_rhs;

    static MatmulConfig row_major(size_t rows, size_t columns, size_t reduction) {
        return {rows, columns, reduction, reduction, columns, columns, false, false};
    }

    static MatmulConfig row_major_transposed_lhs(size_t rows, size_t columns, size_t reduction) {
        return {rows, columns, reduction, rows, columns, columns, true, false};
    }

    static MatmulConfig row_major_transposed_inputs(size_t rows, size_t columns, size_t reduction) {
        return {rows, columns, reduction, rows, reduction, columns, true, true};
    }

    static MatmulConfig row_major_transposed_rhs(size_t rows, size_t columns, size_t reduction) {
        return {rows, columns, reduction, reduction, reduction, columns, false, true};
    }

    Error validate_lengths(size_t out_len, size_t lhs_len, size_t rhs_len) const {
        const size_t lhs_min = transpose_lhs ? rows : reduction;
        const size_t rhs_min = transpose_rhs ? reduction : columns;
        if (rows == 0 || columns == 0 || reduction == 0 || lhs_row_stride < lhs_min || rhs_row_stride < rhs_min ||
            output_row_stride < columns) {
            return Error::InvalidLength;
        }
        auto reach = [](size_t r, size_t c, size_t stride) { return (r - 1) * stride + c; };  // strided_matrix_reach
        const size_t lhs_reach = transpose_lhs ? reach(reduction, rows, lhs_row_stride) : reach(rows, reduction, lhs_row_stride);
        const size_t rhs_reach =
            transpose_rhs ? reach(columns, reduction, rhs_row_stride) : reach(reduction, columns, rhs_row_stride);
        SINGE_HOST_TRY(detail::ensure_len_at_least(lhs_len, lhs_reach));
        SINGE_HOST_TRY(detail::ensure_len_at_least(rhs_len, rhs_reach));
        return detail::ensure_len_at_least(out_len, reach(rows, columns, output_row_stride));
    }
};

// ---- operators: validate lengths like the Rust wrapper, then enqueue through the C ABI ----
namespace cuda {
namespace attention {

// singe-kernel/src/cuda/attention/paged.rs:210-249
inline Error paged_kv_decode_attention_bf16(singe_stream_t stream, DeviceSlice<void> out, DeviceSlice<const void> query,
                                           DeviceSlice<const void> key_cache, DeviceSlice<const void> value_cache,
                                           DeviceSlice<const int32_t> actual_seq_lens,
                                           DeviceSlice<const uint32_t> block_table,
                                           const PagedKvDecodeAttentionConfig &config) {
    SINGE_HOST_TRY(config.validate_lengths(out.len, query.len, key_cache.len, value_cache.len, actual_seq_lens.len,
                                           block_table.len));
    return from_sys(singe_paged_kv_decode_attention_bf16(
        stream, out.ptr, query.ptr, key_cache.ptr, value_cache.ptr, actual_seq_lens.ptr, block_table.ptr, config.batch,
        config.heads, config.kv_heads, config.head_dim, config.block_size, config.physical_blocks,
        config.block_table_batch_stride, config.scale));
}

// singe-kernel/src/cuda/attention/paged.rs:490-576
inline Error ragged_kv_prefill_attention_bf16(singe_stream_t stream, DeviceSlice<void> out, DeviceSlice<float> lse,
                                             DeviceSlice<const void> query, DeviceSlice<const void> key,
                                             DeviceSlice<const void> value, DeviceSlice<const int32_t> lens_q,
                                             DeviceSlice<const int32_t> lens_kv, DeviceSlice<const int32_t> offsets,
                                             const RaggedKvPrefillAttentionConfig &config) {
    SINGE_HOST_TRY(config.validate_lengths(out.len, lse.len, query.len, key.len, value.len, lens_q.len, lens_kv.len,
                                           offsets.len));
    return from_sys(singe_ragged_kv_prefill_attention_bf16(
        stream, out.ptr, lse.ptr, query.ptr, key.ptr, value.ptr, lens_q.ptr, lens_kv.ptr, offsets.ptr, config.batch,
        config.total_query_tokens, config.total_kv_tokens, config.heads, config.kv_heads, config.head_dim,
        config.causal ? 1 : 0, config.scale));
}

// singe-kernel/src/cuda/attention/paged.rs:479-530
inline Error ragged_kv_prefill_attention_f16(singe_stream_t stream, DeviceSlice<void> out, DeviceSlice<float> lse,
                                            DeviceSlice<const void> query, DeviceSlice<const void> key,
                                            DeviceSlice<const void> value, DeviceSlice<const int32_t> lens_q,
                                            DeviceSlice<const int32_t> lens_kv, DeviceSlice<const int32_t> offsets,
                                            const RaggedKvPrefillAttentionConfig &config) {
    SINGE_HOST_TRY(config.validate_lengths(out.len, lse.len, query.len, key.len, value.len, lens_q.len, lens_kv.len,
                                           offsets.len));
    return from_sys(singe_ragged_kv_prefill_attention_f16(
        stream, out.ptr, lse.ptr, query.ptr, key.ptr, value.ptr, lens_q.ptr, lens_kv.ptr, offsets.ptr, config.batch,
        config.total_query_tokens, config.total_kv_tokens, config.heads, config.kv_heads, config.head_dim,
        config.causal ? 1 : 0, config.scale));
}

// singe-kernel/src/cuda/attention/splitk.rs:187-284
inline Error splitk_reduce_f32(singe_stream_t stream, DeviceSlice<float> out, DeviceSlice<const float> attn_splitk,
                              DeviceSlice<const float> lse_splitk, const SplitKReduceConfig &config) {
    SINGE_HOST_TRY(config.validate_lengths(out.len, attn_splitk.len, lse_splitk.len));
    return from_sys(singe_splitk_reduce_f32(stream, out.ptr, attn_splitk.ptr, lse_splitk.ptr, config.batch,
                                            config.heads, config.splits, config.head_dim, config.attn_batch_stride,
                                            config.attn_head_stride, config.attn_split_stride, config.lse_batch_stride,
                                            config.lse_head_stride, config.output_batch_stride,
                                            config.output_head_stride));
}

}  // namespace attention

namespace matmul {

// singe-kernel/src/cuda/matmul.rs:1302-1339
inline Error matmul_bf16_f32(singe_stream_t stream, DeviceSlice<float> out, DeviceSlice<const void> lhs,
                            DeviceSlice<const void> rhs, const MatmulConfig &config) {
    SINGE_HOST_TRY(config.validate_lengths(out.len, lhs.len, rhs.len));
    return from_sys(singe_matmul_bf16_f32(stream, out.ptr, lhs.ptr, rhs.ptr, config.rows, config.columns,
                                          config.reduction, config.lhs_row_stride, config.rhs_row_stride,
                                          config.output_row_stride, config.transpose_lhs ? 1 : 0,
                                          config.transpose_rhs ? 1 : 0));
}

}  // namespace matmul
}  // namespace cuda

}  // namespace singe_kernel
