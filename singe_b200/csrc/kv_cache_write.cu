// Slot-mapped KV-cache write: cache[pages[t], slots[t], :, :] = rows[t, :, :] for keys and values in
// one launch.  Meaning follows KvCache::write (singe/src/nn/decode/cache.rs:97-101) = index_put_ at the
// step's (page, slot) pairs, whose CPU form is singe/src/backend/cpu/shape/multi_index.rs:95-125,204-236:
// a negative index wraps by its extent, anything still outside is refused.  On the device a refused row
// is dropped and reported through the status word, as singe_rotary_cache_write does
// (singe/src/backend/cuda/kernel_plan/source/rotary_cache.rs:238-427).
//
// The copy is pure HBM traffic (row_bytes read + row_bytes written per token and tensor), so the kernel
// is a grid-stride loop of 128-bit loads and stores, four independent chunks per thread per trip.
#include "common.cuh"

namespace singe {
namespace {

template <typename Index>
__device__ __forceinline__ bool resolve_slot(const Index *pages, const Index *slots, size_t token, long long page_count,
                                             long long page_size, long long &row) {
    long long page = static_cast<long long>(pages[token]);
    long long slot = static_cast<long long>(slots[token]);
    if (page < 0) page += page_count;
    if (slot < 0) slot += page_size;
    if (page < 0 || page >= page_count || slot < 0 || slot >= page_size) {
        return false;
    }
    row = page * page_size + slot;
    return true;
}

// Vector = uint4 (16 bytes) on the fast path, or a 2/4-byte word when rows or pointers are not 16-byte aligned.
template <typename Vector, typename Index, int UNROLL>
__global__ void __launch_bounds__(256) kv_cache_write_kernel(Vector *__restrict__ key_cache,
                                                             Vector *__restrict__ value_cache,
                                                             const Vector *__restrict__ keys,
                                                             const Vector *__restrict__ values,
                                                             const Index *__restrict__ write_pages,
                                                             const Index *__restrict__ write_slots, size_t tokens,
                                                             size_t row_vectors, long long page_count,
                                                             long long page_size, int tensors, uint32_t *status) {
    const size_t per_token = row_vectors * static_cast<size_t>(tensors);
    const size_t total = tokens * per_token;
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    size_t index = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    for (; index < total; index += stride * UNROLL) {
        Vector data[UNROLL];
        Vector *target[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const size_t at = index + static_cast<size_t>(u) * stride;
            target[u] = nullptr;
            if (at < total) {
                const size_t token = at / per_token;
                const size_t rest = at - token * per_token;
                const int which = rest >= row_vectors ? 1 : 0;
                const size_t column = rest - static_cast<size_t>(which) * row_vectors;
                long long row;
                if (resolve_slot(write_pages, write_slots, token, page_count, page_size, row)) {
                    const Vector *source = which ? values : keys;
                    Vector *cache = which ? value_cache : key_cache;
                    data[u] = source[token * row_vectors + column];
                    target[u] = cache + static_cast<size_t>(row) * row_vectors + column;
                } else if (column == 0 && which == 0) {
                    report_status(status, kStatusIndexOutOfBounds);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            if (target[u] != nullptr) {
                *target[u] = data[u];
            }
        }
    }
}

template <typename Vector, typename Index>
int launch_write(cudaStream_t stream, void *key_cache, void *value_cache, const void *keys, const void *values,
                 const void *write_pages, const void *write_slots, size_t tokens, size_t row_bytes, size_t pages,
                 size_t page_size, int tensors, uint32_t *status) {
    constexpr int kUnroll = 4;
    const size_t row_vectors = row_bytes / sizeof(Vector);
    const size_t total = tokens * row_vectors * static_cast<size_t>(tensors);
    const size_t per_block = 256 * kUnroll;
    size_t blocks = (total + per_block - 1) / per_block;
    const size_t cap = static_cast<size_t>(device_sm_count()) * 8;
    if (blocks > cap) blocks = cap;
    if (blocks == 0) return SINGE_OK;
    kv_cache_write_kernel<Vector, Index, kUnroll><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
        static_cast<Vector *>(key_cache), static_cast<Vector *>(value_cache), static_cast<const Vector *>(keys),
        static_cast<const Vector *>(values), static_cast<const Index *>(write_pages),
        static_cast<const Index *>(write_slots), tokens, row_vectors, static_cast<long long>(pages),
        static_cast<long long>(page_size), tensors, status);
    return launch_status();
}

bool aligned16(const void *pointer) { return (reinterpret_cast<uintptr_t>(pointer) & 15u) == 0; }

}  // namespace

// Shared by the three dtype entry points; `element_bytes` is 2 or 4.
int kv_cache_write(cudaStream_t stream, void *key_cache, void *value_cache, const void *keys, const void *values,
                   const void *write_pages, const void *write_slots, int index_width, size_t tokens, size_t kv_heads,
                   size_t head_dim, size_t pages, size_t page_size, uint32_t *status, size_t element_bytes) {
    if (tokens == 0 || kv_heads == 0 || head_dim == 0 || pages == 0 || page_size == 0) {
        return SINGE_ERR_INVALID_LENGTH;
    }
    if (index_width != 4 && index_width != 8) {
        return SINGE_ERR_INVALID_ARGUMENT;
    }
    if (!fits_i32(tokens) || !fits_i32(kv_heads) || !fits_i32(head_dim) || !fits_i32(pages) || !fits_i32(page_size)) {
        return SINGE_ERR_LENGTH_EXCEEDS_I32;
    }
    if (key_cache == nullptr || keys == nullptr || write_pages == nullptr || write_slots == nullptr) {
        return SINGE_ERR_NULL_POINTER;
    }
    if ((value_cache == nullptr) != (values == nullptr)) {
        return SINGE_ERR_NULL_POINTER;
    }
    const int tensors = values == nullptr ? 1 : 2;
    size_t row_elements;
    if (__builtin_mul_overflow(kv_heads, head_dim, &row_elements)) return SINGE_ERR_SIZE_OVERFLOW;
    size_t row_bytes;
    if (__builtin_mul_overflow(row_elements, element_bytes, &row_bytes)) return SINGE_ERR_SIZE_OVERFLOW;
    const bool wide = row_bytes % 16 == 0 && aligned16(key_cache) && aligned16(keys) &&
                      (values == nullptr || (aligned16(value_cache) && aligned16(values)));
    const void *value_source = values == nullptr ? keys : values;
    void *value_target = value_cache == nullptr ? key_cache : value_cache;
#define SINGE_WRITE(Vector)                                                                                         \
    (index_width == 8 ? launch_write<Vector, long long>(stream, key_cache, value_target, keys, value_source,       \
                                                        write_pages, write_slots, tokens, row_bytes, pages,        \
                                                        page_size, tensors, status)                                \
                      : launch_write<Vector, int>(stream, key_cache, value_target, keys, value_source, write_pages, \
                                                  write_slots, tokens, row_bytes, pages, page_size, tensors, status))
    if (wide) return SINGE_WRITE(uint4);
    if (element_bytes == 4) return SINGE_WRITE(uint32_t);
    return SINGE_WRITE(uint16_t);
#undef SINGE_WRITE
}

}  // namespace singe
