// Slot-mapped KV-cache write: cache[pages[t], slots[t], :, :] = rows[t, :, :] for keys and values in
// one launch.  Meaning follows KvCache::write (singe/src/nn/decode/cache.rs:97-101) = index_put_ at the
// step's (page, slot) pairs, whose CPU form is singe/src/backend/cpu/shape/multi_index.rs:95-125,204-236:
// a negative index wraps by its extent, anything still outside is refused.  On the device a refused row
// is dropped and reported through the status word, as singe_rotary_cache_write does
// (singe/src/backend/cuda/kernel_plan/source/rotary_cache.rs:238-427).
//
// The copy is pure HBM traffic (row_bytes read + row_bytes written per token and tensor).  Large writes of whole
// 256 B - 3 KB rows go through the bulk-copy engine (kv_cache_write_bulk_kernel below: 20 us = 6.3 TB/s on the
// 15,360-token prompt write); everything else takes a grid-stride loop of 128-bit loads and stores, two independent
// chunks per thread per trip (measured best of 2 / 4 / 8: 22.9 / 29.4 / 38.8 us on the same write).
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

// ---- rows staged through shared memory by the bulk-copy engine ----
// A row (one token's K or V, all heads) is one cp.async.bulk load into a shared-memory stage and one cp.async.bulk
// store from it, so the data never passes through registers and a warp keeps kStages rows in flight with two
// instructions per row.  Every warp owns a ring of stages and walks units (token, tensor) in batches of 32: the lanes
// resolve the 32 (page, slot) pairs together, then lane 0 issues loads kAhead units ahead of the stores.  A stage is
// reused once the store that read it has finished reading (cp.async.bulk.wait_group.read); every mbarrier wait is
// bounded.  Rows that fail the index check are skipped and reported, as in the register kernel.
constexpr int kBulkWarps = 4;

__device__ __forceinline__ void bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

__device__ __forceinline__ void bulk_store(void *dst, uint32_t src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src), "r"(bytes)
                 : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

template <int PENDING>
__device__ __forceinline__ void bulk_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(PENDING) : "memory");
}

template <typename Index, int STAGES, int AHEAD>
__global__ void __launch_bounds__(kBulkWarps * 32)
    kv_cache_write_bulk_kernel(uint8_t *key_cache, uint8_t *value_cache, const uint8_t *keys, const uint8_t *values,
                               const Index *write_pages, const Index *write_slots, size_t tokens, uint32_t row_bytes,
                               long long page_count, long long page_size, int tensors, uint32_t *status) {
    static_assert(AHEAD >= 1 && AHEAD < STAGES, "loads run ahead of stores inside the ring");
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 127u) & ~127u;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t ring = base + warp * STAGES * row_bytes;
    const uint32_t bars = base + kBulkWarps * STAGES * row_bytes + warp * STAGES * 8;
    // where the row parked in each stage goes (written and read by lane 0 only)
    uint8_t **targets = reinterpret_cast<uint8_t **>(smem_raw + (base - raw) + kBulkWarps * STAGES * row_bytes +
                                                     kBulkWarps * STAGES * 8) + warp * STAGES;
    if (lane == 0) {
        for (int s = 0; s < STAGES; ++s) mbar_init(bars + s * 8, 1);
        mbar_init_fence();
    }
    __syncwarp();

    const size_t units = tokens * static_cast<size_t>(tensors);
    const size_t warps = static_cast<size_t>(gridDim.x) * kBulkWarps;
    const size_t me = static_cast<size_t>(blockIdx.x) * kBulkWarps + warp;
    bool failed = false;
    int issued = 0;  // loads issued so far by this warp (stage = issued % STAGES, use = issued / STAGES)
    int stored = 0;  // stores issued so far
    auto store_oldest = [&]() {
        // store number `stored` reads stage stored % STAGES, filled by load number `stored`
        const int s = stored % STAGES;
        if (!mbar_wait(bars + s * 8, (stored / STAGES) & 1)) {
            failed = true;
            return;
        }
        bulk_store(targets[s], ring + s * row_bytes, row_bytes);
        ++stored;
    };
    for (size_t first = me * 32; first < units && !failed; first += warps * 32) {
        // the lanes resolve the batch's 32 units together
        const size_t unit = first + lane;
        const uint8_t *source = nullptr;
        uint8_t *target = nullptr;
        if (unit < units) {
            const size_t token = unit / tensors;
            const int which = static_cast<int>(unit - token * tensors);
            long long row;
            if (resolve_slot(write_pages, write_slots, token, page_count, page_size, row)) {
                source = (which ? values : keys) + token * row_bytes;
                target = (which ? value_cache : key_cache) + static_cast<size_t>(row) * row_bytes;
            } else if (which == 0) {
                report_status(status, kStatusIndexOutOfBounds);
            }
        }
        const unsigned valid = __ballot_sync(0xffffffffu, target != nullptr);
        for (int j = 0; j < 32; ++j) {
            if (((valid >> j) & 1u) == 0) continue;
            const uint8_t *from = reinterpret_cast<const uint8_t *>(
                __shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(source), j));
            uint8_t *to = reinterpret_cast<uint8_t *>(
                __shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(target), j));
            if (lane == 0 && !failed) {
                if (issued - stored == AHEAD) store_oldest();
                if (!failed) {
                    const int s = issued % STAGES;
                    // The store that last read this stage is number issued - STAGES; at least STAGES - AHEAD younger
                    // stores have been issued since, so once no more than that many are pending it has finished.
                    if (issued >= STAGES) bulk_wait_read<STAGES - AHEAD>();
                    mbar_expect_tx(bars + s * 8, row_bytes);
                    bulk_load(ring + s * row_bytes, from, row_bytes, bars + s * 8);
                    targets[s] = to;
                    ++issued;
                }
            }
        }
        failed = __shfl_sync(0xffffffffu, failed ? 1 : 0, 0) != 0;
    }
    if (lane == 0) {
        while (stored < issued && !failed) store_oldest();
        asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");  // the stores have landed before the CTA leaves
        if (failed) {
            report_status(status, kStatusWaitTimeout);
            linger_after_timeout();
        }
    }
}

template <typename Index>
int launch_write_bulk(cudaStream_t stream, void *key_cache, void *value_cache, const void *keys, const void *values,
                      const void *write_pages, const void *write_slots, size_t tokens, size_t row_bytes, size_t pages,
                      size_t page_size, int tensors, uint32_t *status) {
    constexpr int kStages = 8;
    constexpr int kAhead = 4;
    const size_t smem = kBulkWarps * kStages * row_bytes + 2 * kBulkWarps * kStages * 8 + 128;
    static int configured[kMaxDevices] = {0};
    SINGE_CUDA_TRY(ensure_dynamic_shared(kv_cache_write_bulk_kernel<Index, kStages, kAhead>, 100 * 1024, configured));
    const size_t units = tokens * static_cast<size_t>(tensors);
    size_t blocks = (units + kBulkWarps * 32 - 1) / (kBulkWarps * 32);
    const size_t resident = 227 * 1024 / smem;
    const size_t cap = static_cast<size_t>(device_sm_count()) * (resident < 1 ? 1 : resident);
    if (blocks > cap) blocks = cap;
    kv_cache_write_bulk_kernel<Index, kStages, kAhead><<<static_cast<unsigned>(blocks), kBulkWarps * 32, smem, stream>>>(
        static_cast<uint8_t *>(key_cache), static_cast<uint8_t *>(value_cache), static_cast<const uint8_t *>(keys),
        static_cast<const uint8_t *>(values), static_cast<const Index *>(write_pages),
        static_cast<const Index *>(write_slots), tokens, static_cast<uint32_t>(row_bytes),
        static_cast<long long>(pages), static_cast<long long>(page_size), tensors, status);
    return launch_status();
}

template <typename Vector, typename Index>
int launch_write(cudaStream_t stream, void *key_cache, void *value_cache, const void *keys, const void *values,
                 const void *write_pages, const void *write_slots, size_t tokens, size_t row_bytes, size_t pages,
                 size_t page_size, int tensors, uint32_t *status) {
    constexpr int kUnroll = 2;
    constexpr int kBlocksPerSm = 8;
    const size_t row_vectors = row_bytes / sizeof(Vector);
    const size_t total = tokens * row_vectors * static_cast<size_t>(tensors);
    const size_t per_block = 256 * kUnroll;
    size_t blocks = (total + per_block - 1) / per_block;
    const size_t cap = static_cast<size_t>(device_sm_count()) * kBlocksPerSm;
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
    // Whole rows through the bulk-copy engine when a warp's ring of 8 rows fits (rows of 256 B .. 3 KB) and there are
    // enough rows to fill the machine; short or odd rows keep the register kernel.
    if (wide && row_bytes >= 256 && row_bytes <= 3072 &&
        tokens * static_cast<size_t>(tensors) >= 4096) {
        return index_width == 8
                   ? launch_write_bulk<long long>(stream, key_cache, value_target, keys, value_source, write_pages,
                                                  write_slots, tokens, row_bytes, pages, page_size, tensors, status)
                   : launch_write_bulk<int>(stream, key_cache, value_target, keys, value_source, write_pages,
                                            write_slots, tokens, row_bytes, pages, page_size, tensors, status);
    }
    if (wide) return SINGE_WRITE(uint4);
    if (element_bytes == 4) return SINGE_WRITE(uint32_t);
    return SINGE_WRITE(uint16_t);
#undef SINGE_WRITE
}

}  // namespace singe
