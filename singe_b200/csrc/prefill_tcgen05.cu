// Packed variable-length flash-attention prefill on the tcgen05 tensor core (bf16, head_dim 128, GQA).
//
// Meaning: ragged_kv_prefill_attention (singe-kernel/src/cpu/attention.rs:1343-1420): sequence b owns query
// tokens [offsets[b], offsets[b] + lens_q[b]) and key rows [offsets[b], offsets[b] + lens_kv[b]) of the packed
// tensors; causal hides key_index > query_index (sequence-local); out [T, H, D] and a natural-log LSE [T, H],
// -1.0e20 for a row that sees no key.  Replaces singe_tcgen05_attention
// (singe/src/backend/cuda/kernel_plan/source/tcgen05_attention.rs:76-258), which is single-stage, cp.async-fed and
// rescales the output through tensor memory on every tile.
//
// One CTA = one 128-row query tile of one (sequence, head); two CTAs share an SM so that one's softmax overlaps
// the other's tensor work.  Roles:
//   warps 0-3  softmax, one query row per thread (row = tensor-memory lane): two passes over S in tensor memory
//              (row max, then exp2 / row sum / bf16 pack), P written back over S with tcgen05.st, output rescaled
//              in tensor memory only when the running max grew by more than 2^8 (the stale max stays baked into P,
//              O and the row sum, so the result is exact), epilogue O / sum -> bf16 and the LSE.
//   warp 4     MMA issuer and tensor-memory owner: S = Q K^T as 8 x tcgen05.mma 128x128x16 (both operands K-major
//              in shared memory), O += P V as 8 x tcgen05.mma with P read from tensor memory and V MN-major.
//   warp 5     TMA producer: Q once, then one K tile and one V tile (128 keys x 128 dims, two SWIZZLE_128B boxes
//              each) per step, released by tcgen05.commit as soon as the MMA that read them retires.
// Tensor memory per CTA: S/P columns [0,128), O columns [128,256).  Shared memory: Q, K, V tiles of 32 KB each.
// Query tiles are dispatched heaviest-first (highest tile index first), since a causal tile's work grows with
// its index.  Every mbarrier wait is bounded; on a timeout the CTA records status 2, frees tensor memory and leaves.
#include "common.cuh"
#include "tcgen05.cuh"

namespace singe {

namespace {

constexpr int kPrefillThreads = 192;
constexpr int kTile = 128;           // query rows and keys per tile
constexpr int kHeadDim = 128;
constexpr int kHalfTileBytes = kTile * 128;       // one TMA box: 128 rows x 128 bytes
constexpr int kTileBytes = 2 * kHalfTileBytes;    // 32 KB
constexpr int kMaxRankTiles = 2048;               // heaviest-first dispatch handles sequences up to 256 Ki tokens
constexpr float kRescaleThreshold = 8.0f;         // log2 units

struct PrefillParams {
    __nv_bfloat16 *out;
    float *lse;
    const int32_t *lens_q;
    const int32_t *lens_kv;
    const int32_t *offsets;
    int batch;
    int heads;
    int kv_heads;
    int total_q;
    int total_kv;
    int causal;
    float scale_log2;
    uint32_t *error;
};

__device__ __forceinline__ float exp2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__global__ void __launch_bounds__(kPrefillThreads, 2)
    prefill_tcgen05_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap k_map,
                           const __grid_constant__ CUtensorMap v_map, const PrefillParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    const uint32_t q_smem = base;
    const uint32_t k_smem = base + kTileBytes;
    const uint32_t v_smem = base + 2 * kTileBytes;
    const uint32_t bars = base + 3 * kTileBytes;
    const uint32_t bar_q_full = bars;
    const uint32_t bar_k_full = bars + 8;
    const uint32_t bar_v_full = bars + 16;
    const uint32_t bar_k_empty = bars + 24;
    const uint32_t bar_v_empty = bars + 32;
    const uint32_t bar_s_full = bars + 40;
    const uint32_t bar_p_full = bars + 48;
    const uint32_t bar_o_full = bars + 56;
    const uint32_t tmem_holder = bars + 64;
    int *counts = reinterpret_cast<int *>(smem_raw + (bars + 128 - raw));  // [kMaxRankTiles] scratch for dispatch
    volatile uint32_t *holder_ptr = reinterpret_cast<volatile uint32_t *>(smem_raw + (tmem_holder - raw));
    volatile int *picked = reinterpret_cast<volatile int *>(smem_raw + (tmem_holder + 8 - raw));  // [2]

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const int head = blockIdx.y;

    // ---- which (sequence, query tile) is this CTA?  rank 0 = highest tile index over all sequences ----
    {
        int tmax = 0;
        for (int b = 0; b < p.batch; ++b) {
            const int n = (max(p.lens_q[b], 0) + kTile - 1) / kTile;
            tmax = max(tmax, n);
        }
        tmax = min(tmax, kMaxRankTiles);
        for (int t = tid; t < tmax; t += kPrefillThreads) {
            int count = 0;
            for (int b = 0; b < p.batch; ++b) {
                count += ((max(p.lens_q[b], 0) + kTile - 1) / kTile) > t ? 1 : 0;
            }
            counts[t] = count;
        }
        __syncthreads();
        if (tid == 0) {
            int rank = blockIdx.x;
            int chosen_tile = -1, chosen_seq = -1;
            for (int t = tmax - 1; t >= 0; --t) {
                if (rank < counts[t]) {
                    chosen_tile = t;
                    break;
                }
                rank -= counts[t];
            }
            if (chosen_tile >= 0) {
                for (int b = 0; b < p.batch; ++b) {
                    if (((max(p.lens_q[b], 0) + kTile - 1) / kTile) > chosen_tile) {
                        if (rank == 0) {
                            chosen_seq = b;
                            break;
                        }
                        --rank;
                    }
                }
            }
            picked[0] = chosen_seq;
            picked[1] = chosen_tile;
        }
        __syncthreads();
    }
    const int seq = picked[0];
    const int tile = picked[1];
    if (seq < 0 || tile < 0) {
        return;  // more CTAs were launched than there are query tiles
    }
    const int len_q = max(p.lens_q[seq], 0);
    const int len_kv = max(p.lens_kv[seq], 0);
    const int offset = p.offsets[seq];
    const int q_first = tile * kTile;                       // sequence-local index of the tile's first query
    const int q_last = min(q_first + kTile, len_q) - 1;     // and of its last real query
    // keys any row of the tile can see
    int visible = len_kv;
    if (p.causal) visible = min(visible, q_last + 1);
    const int key_tiles = (visible + kTile - 1) / kTile;
    const int kv_head = head / (p.heads / p.kv_heads);
    const bool in_bounds = offset >= 0 && offset + len_q <= p.total_q && offset + len_kv <= p.total_kv;

    if (key_tiles == 0 || !in_bounds) {
        // No key is visible (or the sequence's extents are inconsistent): rows get zeros and LSE -1e20.
        if (!in_bounds) {
            if (tid == 0) report_status(p.error, kStatusIndexOutOfBounds);
            return;
        }
        if (warp < 4) {
            const int row = q_first + warp * 32 + lane;
            if (row < len_q) {
                const size_t token = static_cast<size_t>(offset) + row;
                uint4 *dst = reinterpret_cast<uint4 *>(p.out + (token * p.heads + head) * kHeadDim);
#pragma unroll
                for (int i = 0; i < kHeadDim / 8; ++i) dst[i] = make_uint4(0u, 0u, 0u, 0u);
                p.lse[token * p.heads + head] = -1.0e20f;
            }
        }
        return;
    }

    if (tid == 0) {
        for (int i = 0; i < 8; ++i) {
            mbar_init(bars + 8 * i, i == 6 ? 4 : 1);  // p_full takes one arrival per softmax warp
        }
        mbar_init_fence();
    }
    if (warp == 4) {
        tmem_alloc(tmem_holder, 256);
        tmem_relinquish();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *holder_ptr;
    const uint32_t tmem_s = tmem_base;         // S (f32) and, packed over its first 64 columns, P (bf16 pairs)
    const uint32_t tmem_o = tmem_base + 128;   // O (f32)

    bool failed = false;

    if (warp == 5) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            prefetch_tensor_map(&q_map);
            prefetch_tensor_map(&k_map);
            prefetch_tensor_map(&v_map);
            mbar_expect_tx(bar_q_full, kTileBytes);
            tma_load_3d(q_smem, &q_map, bar_q_full, 0, head, offset + q_first);
            tma_load_3d(q_smem + kHalfTileBytes, &q_map, bar_q_full, 64, head, offset + q_first);
        }
        for (int j = 0; j < key_tiles; ++j) {
            const int row0 = offset + j * kTile;
            int ok = 1;
            if (lane == 0 && j > 0) ok = mbar_wait(bar_k_empty, (j - 1) & 1) ? 1 : 0;
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) {
                failed = true;
                break;
            }
            if (lane == 0) {
                mbar_expect_tx(bar_k_full, kTileBytes);
                tma_load_3d(k_smem, &k_map, bar_k_full, 0, kv_head, row0);
                tma_load_3d(k_smem + kHalfTileBytes, &k_map, bar_k_full, 64, kv_head, row0);
            }
            if (lane == 0 && j > 0) ok = mbar_wait(bar_v_empty, (j - 1) & 1) ? 1 : 0;
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) {
                failed = true;
                break;
            }
            if (lane == 0) {
                mbar_expect_tx(bar_v_full, kTileBytes);
                tma_load_3d(v_smem, &v_map, bar_v_full, 0, kv_head, row0);
                tma_load_3d(v_smem + kHalfTileBytes, &v_map, bar_v_full, 64, kv_head, row0);
            }
        }
    } else if (warp == 4) {
        // ---------------- MMA issuer ----------------
        constexpr uint32_t kIdescQK = make_instr_desc(kTile, kTile, true, 0, 0);      // A, B K-major
        constexpr uint32_t kIdescPV = make_instr_desc(kTile, kHeadDim, true, 0, 1);   // B (V) MN-major
        if (!__all_sync(0xffffffffu, mbar_wait(bar_q_full, 0) ? 1 : 0)) {
            failed = true;
        }
        for (int j = 0; j < key_tiles && !failed; ++j) {
            const uint32_t parity = j & 1;
            if (!__all_sync(0xffffffffu, mbar_wait(bar_k_full, parity) ? 1 : 0)) {
                failed = true;
                break;
            }
            tcgen05_fence_after();
            if (lane == 0) {
#pragma unroll
                for (int ks = 0; ks < kHeadDim / 16; ++ks) {
                    const uint32_t within = (ks >> 2) * kHalfTileBytes + (ks & 3) * 32;
                    umma_ss(tmem_s, make_smem_desc(q_smem + within, 16, 1024),
                            make_smem_desc(k_smem + within, 16, 1024), kIdescQK, ks > 0 ? 1u : 0u);
                }
                tcgen05_commit(bar_k_empty);
                tcgen05_commit(bar_s_full);
            }
            __syncwarp();
            if (!__all_sync(0xffffffffu, mbar_wait(bar_p_full, parity) ? 1 : 0)) {
                failed = true;
                break;
            }
            if (!__all_sync(0xffffffffu, mbar_wait(bar_v_full, parity) ? 1 : 0)) {
                failed = true;
                break;
            }
            tcgen05_fence_after();
            if (lane == 0) {
#pragma unroll
                for (int ks = 0; ks < kTile / 16; ++ks) {
                    // 16 keys per step: P advances 8 packed columns, V advances two 8-row groups (2 x 1024 bytes);
                    // the second 64 dims of V are the next box, 16 KB further (leading byte offset).
                    umma_ts(tmem_o, tmem_s + ks * 8, make_smem_desc(v_smem + ks * 2048, kHalfTileBytes, 1024),
                            kIdescPV, (j > 0 || ks > 0) ? 1u : 0u);
                }
                tcgen05_commit(bar_v_empty);
                if (j == key_tiles - 1) {
                    tcgen05_commit(bar_o_full);
                }
            }
            __syncwarp();
        }
    } else {
        // ---------------- softmax / correction / epilogue: one query row per thread ----------------
        const int row = q_first + warp * 32 + lane;          // sequence-local query index
        const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
        float used_max = -INFINITY;   // the max baked into P, O and row_sum
        float row_sum = 0.0f;
        for (int j = 0; j < key_tiles; ++j) {
            if (!__all_sync(0xffffffffu, mbar_wait(bar_s_full, j & 1) ? 1 : 0)) {
                failed = true;
                break;
            }
            tcgen05_fence_after();
            const int key0 = j * kTile;
            // last key this row may see in this tile (exclusive), relative to key0
            int limit = len_kv - key0;
            if (p.causal) limit = min(limit, row + 1 - key0);
            limit = row < len_q ? limit : 0;
            const bool partial = __any_sync(0xffffffffu, limit < kTile);

            // pass 1: row max of the scaled scores
            float tile_max = -INFINITY;
#pragma unroll 1
            for (int c = 0; c < kTile; c += 32) {
                uint32_t r[32];
                tmem_ld_x32(tmem_s + lane_base + c, r);
                tmem_wait_ld();
                if (partial) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        if (c + i < limit) tile_max = fmaxf(tile_max, __uint_as_float(r[i]));
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) tile_max = fmaxf(tile_max, __uint_as_float(r[i]));
                }
            }
            tile_max *= p.scale_log2;  // scale > 0 keeps the order; a negative scale is handled below
            if (p.scale_log2 < 0.0f) {
                // rare: recompute with the sign applied (max of s*scale is scale * min of s)
                tile_max = -INFINITY;
#pragma unroll 1
                for (int c = 0; c < kTile; c += 32) {
                    uint32_t r[32];
                    tmem_ld_x32(tmem_s + lane_base + c, r);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        if (c + i < limit) tile_max = fmaxf(tile_max, __uint_as_float(r[i]) * p.scale_log2);
                    }
                }
            }
            const float wanted = fmaxf(used_max, tile_max);
            // Rescale O only when some row's max grew past the threshold; then every row of the warp re-bases.
            const bool grow = wanted > used_max + kRescaleThreshold || (used_max == -INFINITY && wanted > -INFINITY);
            if (__any_sync(0xffffffffu, grow)) {
                const float factor = used_max == -INFINITY ? 0.0f : exp2_approx(used_max - wanted);
                if (j > 0) {
                    row_sum *= factor;
#pragma unroll 1
                    for (int c = 0; c < kHeadDim; c += 32) {
                        uint32_t r[32];
                        tmem_ld_x32(tmem_o + lane_base + c, r);
                        tmem_wait_ld();
#pragma unroll
                        for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * factor);
                        tmem_st_x32(tmem_o + lane_base + c, r);
                    }
                    tmem_wait_st();
                }
                used_max = wanted;
            }
            // pass 2: P = exp2(s * scale - used_max), row sum, bf16 pairs back into tensor memory
            const float bias = used_max == -INFINITY ? 0.0f : -used_max;
#pragma unroll 1
            for (int c = 0; c < kTile; c += 32) {
                uint32_t r[32];
                tmem_ld_x32(tmem_s + lane_base + c, r);
                tmem_wait_ld();
                uint32_t packed[16];
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    float a = exp2_approx(fmaf(__uint_as_float(r[i]), p.scale_log2, bias));
                    float b = exp2_approx(fmaf(__uint_as_float(r[i + 1]), p.scale_log2, bias));
                    if (partial) {
                        a = (c + i < limit) ? a : 0.0f;
                        b = (c + i + 1 < limit) ? b : 0.0f;
                    }
                    row_sum += a + b;
                    packed[i >> 1] = pack2<__nv_bfloat16>(a, b);
                }
                tmem_st_x16(tmem_s + lane_base + (c >> 1), packed);
            }
            tmem_wait_st();
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(bar_p_full);
            }
        }
        // ---- epilogue ----
        if (!failed) {
            if (!__all_sync(0xffffffffu, mbar_wait(bar_o_full, 0) ? 1 : 0)) {
                failed = true;
            }
        }
        if (!failed) {
            tcgen05_fence_after();
            const bool real = row < len_q;
            const bool empty = row_sum == 0.0f;
            const float inverse = empty ? 0.0f : 1.0f / row_sum;
            const size_t token = static_cast<size_t>(offset) + (real ? row : 0);
            __nv_bfloat16 *dst = p.out + (token * p.heads + head) * kHeadDim;
#pragma unroll 1
            for (int c = 0; c < kHeadDim; c += 32) {
                uint32_t r[32];
                tmem_ld_x32(tmem_o + lane_base + c, r);
                tmem_wait_ld();
                if (real) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint4 word;
                        word.x = pack2<__nv_bfloat16>(__uint_as_float(r[i]) * inverse, __uint_as_float(r[i + 1]) * inverse);
                        word.y = pack2<__nv_bfloat16>(__uint_as_float(r[i + 2]) * inverse, __uint_as_float(r[i + 3]) * inverse);
                        word.z = pack2<__nv_bfloat16>(__uint_as_float(r[i + 4]) * inverse, __uint_as_float(r[i + 5]) * inverse);
                        word.w = pack2<__nv_bfloat16>(__uint_as_float(r[i + 6]) * inverse, __uint_as_float(r[i + 7]) * inverse);
                        if (empty) word = make_uint4(0u, 0u, 0u, 0u);
                        *reinterpret_cast<uint4 *>(dst + c + i) = word;
                    }
                }
            }
            if (real) {
                p.lse[token * p.heads + head] =
                    empty ? -1.0e20f : (used_max + log2f(row_sum)) * 0.6931471805599453f;
            }
        }
    }
    if (failed && lane == 0) {
        report_status(p.error, kStatusWaitTimeout);
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 4) {
        tcgen05_fence_after();
        tmem_dealloc(tmem_base, 256);
    }
}

constexpr int kPrefillSmem = 3 * kTileBytes + 128 + kMaxRankTiles * 4 + 1024;

}  // namespace

bool prefill_fast_path(size_t heads, size_t kv_heads, size_t head_dim, size_t total_query_tokens, const void *query,
                       const void *key, const void *value, const void *out) {
    // The heaviest-first dispatch table holds kMaxRankTiles query tiles per sequence.
    if (total_query_tokens / kTile + 1 > kMaxRankTiles) return false;
    const uintptr_t all = reinterpret_cast<uintptr_t>(query) | reinterpret_cast<uintptr_t>(key) |
                          reinterpret_cast<uintptr_t>(value) | reinterpret_cast<uintptr_t>(out);
    return head_dim == kHeadDim && heads % kv_heads == 0 && heads <= 65535 && (all & 15u) == 0;
}

int prefill_tcgen05_bf16(cudaStream_t stream, void *out, float *lse, const void *query, const void *key,
                         const void *value, const int32_t *lens_q, const int32_t *lens_kv, const int32_t *offsets,
                         size_t batch, size_t total_query_tokens, size_t total_kv_tokens, size_t heads,
                         size_t kv_heads, size_t head_dim, int causal, float scale) {
    if (head_dim != kHeadDim) return SINGE_ERR_UNSUPPORTED_WIDTH;
    SINGE_CUDA_TRY(cudaFuncSetAttribute(prefill_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        kPrefillSmem));
    CUtensorMap q_map, k_map, v_map;
    const uint32_t box[3] = {64, 1, kTile};
    {
        const uint64_t dims[3] = {kHeadDim, heads, total_query_tokens};
        const uint64_t strides[2] = {kHeadDim * 2, kHeadDim * 2 * heads};
        SINGE_TRY(encode_tensor_map(&q_map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, query, dims, strides, box,
                                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B));
    }
    {
        const uint64_t dims[3] = {kHeadDim, kv_heads, total_kv_tokens};
        const uint64_t strides[2] = {kHeadDim * 2, kHeadDim * 2 * kv_heads};
        SINGE_TRY(encode_tensor_map(&k_map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, key, dims, strides, box,
                                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B));
        SINGE_TRY(encode_tensor_map(&v_map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, value, dims, strides, box,
                                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B));
    }
    PrefillParams params;
    params.out = static_cast<__nv_bfloat16 *>(out);
    params.lse = lse;
    params.lens_q = lens_q;
    params.lens_kv = lens_kv;
    params.offsets = offsets;
    params.batch = static_cast<int>(batch);
    params.heads = static_cast<int>(heads);
    params.kv_heads = static_cast<int>(kv_heads);
    params.total_q = static_cast<int>(total_query_tokens);
    params.total_kv = static_cast<int>(total_kv_tokens);
    params.causal = causal ? 1 : 0;
    params.scale_log2 = scale * 1.4426950408889634f;
    params.error = device_error_word();
    // Upper bound on query tiles: every sequence can add one partial tile.
    const size_t tiles = total_query_tokens / kTile + batch;
    if (tiles > 0x7fffffffull) return SINGE_ERR_LENGTH_EXCEEDS_I32;
    dim3 grid(static_cast<unsigned>(tiles), static_cast<unsigned>(heads));
    prefill_tcgen05_kernel<<<grid, kPrefillThreads, kPrefillSmem, stream>>>(q_map, k_map, v_map, params);
    return launch_status();
}

}  // namespace singe
