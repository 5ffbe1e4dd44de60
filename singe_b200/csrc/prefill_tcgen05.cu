// Packed variable-length flash-attention prefill on the tcgen05 tensor core (bf16, head_dim 128, GQA).
//
// Meaning: ragged_kv_prefill_attention (singe-kernel/src/cpu/attention.rs:1343-1420): sequence b owns query
// tokens [offsets[b], offsets[b] + lens_q[b]) and key rows [offsets[b], offsets[b] + lens_kv[b]) of the packed
// tensors; causal hides key_index > query_index (sequence-local); out [T, H, D] and a natural-log LSE [T, H],
// -1.0e20 for a row that sees no key.  Replaces singe_tcgen05_attention
// (singe/src/backend/cuda/kernel_plan/source/tcgen05_attention.rs:76-258), which is single-stage, cp.async-fed and
// rescales the output through tensor memory on every tile.
//
// One CTA = 256 consecutive query rows of one (sequence, head), handled as two 128-row tiles A and B that take
// turns on the tensor core, so the softmax of one tile runs while the other tile's MMAs execute.  Roles:
//   warps 0-7  softmax of whichever tile has scores ready (A, B, A, B ...).  A row (= tensor-memory lane) is shared
//              by two threads, 64 score columns each, so one tile's softmax is short enough to hide behind the
//              other tile's MMAs.  Scores are pulled into registers once (row max, then exp2 / row sum / bf16
//              pack), P is written back over S with tcgen05.st, O is rescaled in tensor memory only when the
//              running max grew by more than 2^8 (the stale max stays baked into P, O and the row sum, so the
//              result is exact), epilogue O / sum -> bf16 + LSE.
//              A quarter of the exponentials are evaluated as a polynomial on the FMA pipe: the special-function
//              unit delivers 16 exp2 per clock per SM, which at head_dim 128 is exactly as much time as the MMAs.
//   warp 8     MMA issuer and tensor-memory owner.  Issue order per key tile j:
//                 PV_A(j), QK_A(j+1), PV_B(j), QK_B(j+1)
//              (S = Q K^T: 8 x tcgen05.mma 128x128x16, both operands K-major in shared memory; O += P V: 8 x
//              tcgen05.mma with P read from tensor memory and V MN-major), so softmax_A(j) overlaps PV_B(j-1) and
//              QK_B(j), softmax_B(j) overlaps PV_A(j) and QK_A(j+1).
//   warp 9     TMA producer: both Q tiles once, then K and V tiles (128 keys x 128 dims, two SWIZZLE_128B boxes
//              each) into two stages each, released by tcgen05.commit when the MMAs that read them retire.
// Tensor memory (all 512 columns): S_A/P_A [0,128), S_B/P_B [128,256), O_A [256,384), O_B [384,512).
// Shared memory: Q_A, Q_B, 2 x K, 2 x V tiles of 32 KB = 192 KB.
// Under a causal mask tile A sees one key tile less than tile B; CTAs are dispatched heaviest-first.
// Every mbarrier wait is bounded; on a timeout the CTA records status 2, frees tensor memory and leaves.
#include "common.cuh"
#include "tcgen05.cuh"

namespace singe {

namespace {

constexpr int kPrefillThreads = 320;
constexpr int kTile = 128;           // rows of one query tile, and keys per key tile
constexpr int kPair = 2 * kTile;     // query rows per CTA
constexpr int kHalfRow = kTile / 2;  // score columns one softmax thread handles
constexpr int kHeadDim = 128;
constexpr int kHalfTileBytes = kTile * 128;       // one TMA box: 128 rows x 128 bytes
constexpr int kTileBytes = 2 * kHalfTileBytes;    // 32 KB
constexpr int kMaxRankTiles = 1024;               // heaviest-first dispatch: sequences up to 256 Ki tokens
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

__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// 2^x for two values on the FMA pipe with packed f32x2 arithmetic: x = r + f with r the nearest integer and f in
// [-0.5, 0.5]; 2^f by a degree-4 polynomial (relative error ~4e-5, far below bf16 resolution), 2^r by adding r
// to the exponent field.
__device__ __forceinline__ float2 exp2_poly2(float2 x) {
    x.x = fmaxf(x.x, -120.0f);
    x.y = fmaxf(x.y, -120.0f);
    const float2 magic = make_float2(12582912.0f, 12582912.0f);  // 1.5 * 2^23: the low mantissa bits then hold r
    const float2 shifted = __fadd2_rn(x, magic);
    const float2 r = __fadd2_rn(shifted, make_float2(-12582912.0f, -12582912.0f));
    const float2 f = __ffma2_rn(r, make_float2(-1.0f, -1.0f), x);
    float2 p = __ffma2_rn(f, make_float2(0.009618129f, 0.009618129f), make_float2(0.055504109f, 0.055504109f));
    p = __ffma2_rn(p, f, make_float2(0.240226507f, 0.240226507f));
    p = __ffma2_rn(p, f, make_float2(0.693147181f, 0.693147181f));
    p = __ffma2_rn(p, f, make_float2(1.0f, 1.0f));
    p.x = __int_as_float(__float_as_int(p.x) + (__float_as_int(shifted.x) << 23));
    p.y = __int_as_float(__float_as_int(p.y) + (__float_as_int(shifted.y) << 23));
    return p;
}

// Maximum of the 64 raw scores one thread holds (half a row).  MASKED handles tiles where some keys are hidden (the
// diagonal tile and a sequence's last tile); the unmasked form is the steady state: three-input maxima, no compares.
template <bool MASKED>
__device__ __forceinline__ float row_max(const uint32_t (&sc)[kHalfRow], int limit, float sign) {
    float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;  // independent chains for ILP
    if (MASKED) {
#pragma unroll
        for (int i = 0; i < kHalfRow; i += 4) {
            if (i < limit) m0 = fmaxf(m0, __uint_as_float(sc[i]) * sign);
            if (i + 1 < limit) m1 = fmaxf(m1, __uint_as_float(sc[i + 1]) * sign);
            if (i + 2 < limit) m2 = fmaxf(m2, __uint_as_float(sc[i + 2]) * sign);
            if (i + 3 < limit) m3 = fmaxf(m3, __uint_as_float(sc[i + 3]) * sign);
        }
    } else {
#pragma unroll
        for (int i = 0; i < kHalfRow; i += 8) {
            m0 = max3(m0, __uint_as_float(sc[i]), __uint_as_float(sc[i + 1]));
            m1 = max3(m1, __uint_as_float(sc[i + 2]), __uint_as_float(sc[i + 3]));
            m2 = max3(m2, __uint_as_float(sc[i + 4]), __uint_as_float(sc[i + 5]));
            m3 = max3(m3, __uint_as_float(sc[i + 6]), __uint_as_float(sc[i + 7]));
        }
    }
    return fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
}

// P = exp2(s * scale + bias) for the 64 scores one thread holds: bf16 pairs go back to tensor memory over S, the
// (unrounded) values are summed.  Scores are handled as f32x2 pairs; every fourth pair takes its two exponentials
// from the polynomial on the FMA pipe instead of the special-function unit.
template <bool MASKED>
__device__ __forceinline__ float row_exp_store(const uint32_t (&sc)[kHalfRow], uint32_t tmem_s, float scale_log2,
                                               float bias, int limit) {
    float2 sum = make_float2(0.0f, 0.0f);
    const float2 scale2 = make_float2(scale_log2, scale_log2);
    const float2 bias2 = make_float2(bias, bias);
#pragma unroll
    for (int c = 0; c < kHalfRow; c += 32) {
        uint32_t packed[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
            const float2 x = __ffma2_rn(make_float2(__uint_as_float(sc[c + i]), __uint_as_float(sc[c + i + 1])),
                                        scale2, bias2);
            float2 e;
            if ((i & 7) == 6) {
                e = exp2_poly2(x);
            } else {
                e.x = exp2_approx(x.x);
                e.y = exp2_approx(x.y);
            }
            if (MASKED) {
                e.x = (c + i < limit) ? e.x : 0.0f;
                e.y = (c + i + 1 < limit) ? e.y : 0.0f;
            }
            sum = __fadd2_rn(sum, e);
            packed[i >> 1] = pack2<__nv_bfloat16>(e.x, e.y);
        }
        tmem_st_x16(tmem_s + (c >> 1), packed);
    }
    return sum.x + sum.y;
}

__global__ void __launch_bounds__(kPrefillThreads, 1)
    prefill_tcgen05_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap k_map,
                           const __grid_constant__ CUtensorMap v_map, const PrefillParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    const uint32_t q_smem = base;                        // [2 tiles]
    const uint32_t k_smem = base + 2 * kTileBytes;       // [2 stages]
    const uint32_t v_smem = base + 4 * kTileBytes;       // [2 stages]
    const uint32_t bars = base + 6 * kTileBytes;
    const uint32_t bar_q_full = bars;
    const uint32_t bar_k_full = bars + 8;     // [2]
    const uint32_t bar_k_empty = bars + 24;   // [2]
    const uint32_t bar_v_full = bars + 40;    // [2]
    const uint32_t bar_v_empty = bars + 56;   // [2]
    const uint32_t bar_s_full = bars + 72;    // [2 tiles]
    const uint32_t bar_p_full = bars + 88;    // [2 tiles]
    const uint32_t bar_o_full = bars + 104;   // [2 tiles]
    const uint32_t bar_exchange = bars + 120;
    const uint32_t tmem_holder = bars + 128;
    volatile uint32_t *holder_ptr = reinterpret_cast<volatile uint32_t *>(smem_raw + (tmem_holder - raw));
    volatile int *picked = reinterpret_cast<volatile int *>(smem_raw + (tmem_holder + 8 - raw));  // [2]
    float *exchange = reinterpret_cast<float *>(smem_raw + (bars + 160 - raw));  // [2 buffers][2 halves][128 rows]
    int *counts = reinterpret_cast<int *>(smem_raw + (bars + 160 + 4 * kTile * 4 - raw));  // [kMaxRankTiles] dispatch scratch

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const int head = blockIdx.y;

    // ---- which (sequence, 256-row pair) is this CTA?  rank 0 = highest pair index over all sequences ----
    {
        int tmax = 0;
        for (int b = 0; b < p.batch; ++b) {
            tmax = max(tmax, (max(p.lens_q[b], 0) + kPair - 1) / kPair);
        }
        tmax = min(tmax, kMaxRankTiles);
        for (int t = tid; t < tmax; t += kPrefillThreads) {
            int count = 0;
            for (int b = 0; b < p.batch; ++b) {
                count += ((max(p.lens_q[b], 0) + kPair - 1) / kPair) > t ? 1 : 0;
            }
            counts[t] = count;
        }
        __syncthreads();
        if (tid == 0) {
            int rank = blockIdx.x;
            int chosen_pair = -1, chosen_seq = -1;
            for (int t = tmax - 1; t >= 0; --t) {
                if (rank < counts[t]) {
                    chosen_pair = t;
                    break;
                }
                rank -= counts[t];
            }
            if (chosen_pair >= 0) {
                for (int b = 0; b < p.batch; ++b) {
                    if (((max(p.lens_q[b], 0) + kPair - 1) / kPair) > chosen_pair) {
                        if (rank == 0) {
                            chosen_seq = b;
                            break;
                        }
                        --rank;
                    }
                }
            }
            picked[0] = chosen_seq;
            picked[1] = chosen_pair;
        }
        __syncthreads();
    }
    const int seq = picked[0];
    const int pair = picked[1];
    if (seq < 0 || pair < 0) {
        return;  // more CTAs were launched than there are query pairs
    }
    const int len_q = max(p.lens_q[seq], 0);
    const int len_kv = max(p.lens_kv[seq], 0);
    const int offset = p.offsets[seq];
    const int q0 = pair * kPair;  // sequence-local index of the CTA's first query
    const int kv_head = head / (p.heads / p.kv_heads);
    if (offset < 0 || offset + len_q > p.total_q || offset + len_kv > p.total_kv) {
        if (tid == 0) report_status(p.error, kStatusIndexOutOfBounds);
        return;
    }
    // key tiles each query tile needs (0 when the tile has no real row or sees no key)
    int tiles_needed[2];
#pragma unroll
    for (int x = 0; x < 2; ++x) {
        const int first = q0 + x * kTile;
        const int real = min(max(len_q - first, 0), kTile);
        int visible = real > 0 ? len_kv : 0;
        if (p.causal && real > 0) visible = min(visible, first + real);
        tiles_needed[x] = (visible + kTile - 1) / kTile;
    }
    const int key_tiles = max(tiles_needed[0], tiles_needed[1]);

    if (key_tiles == 0) {
        // No key is visible to any row: zeros and LSE -1e20.
        if (warp < 8) {
            const int row = q0 + (warp >> 2) * kTile + (warp & 3) * 32 + lane;
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
        for (int i = 0; i < 16; ++i) {
            // p_full[2] and the exchange barrier take one arrival per softmax warp (eight warps share every tile)
            const bool by_warps = i == 11 || i == 12 || i == 15;
            mbar_init(bars + 8 * i, by_warps ? 8 : 1);
        }
        mbar_init_fence();
    }
    if (warp == 8) {
        tmem_alloc(tmem_holder, 512);
        tmem_relinquish();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *holder_ptr;

    bool failed = false;

    if (warp == 9) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            prefetch_tensor_map(&q_map);
            prefetch_tensor_map(&k_map);
            prefetch_tensor_map(&v_map);
            mbar_expect_tx(bar_q_full, 2 * kTileBytes);
#pragma unroll
            for (int x = 0; x < 2; ++x) {
                tma_load_3d(q_smem + x * kTileBytes, &q_map, bar_q_full, 0, head, offset + q0 + x * kTile);
                tma_load_3d(q_smem + x * kTileBytes + kHalfTileBytes, &q_map, bar_q_full, 64, head,
                            offset + q0 + x * kTile);
            }
        }
        for (int j = 0; j < key_tiles; ++j) {
            const int stage = j & 1;
            const int row0 = offset + j * kTile;
            int ok = 1;
            if (lane == 0 && j >= 2) ok = mbar_wait(bar_k_empty + stage * 8, ((j >> 1) - 1) & 1) ? 1 : 0;
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) {
                failed = true;
                break;
            }
            if (lane == 0) {
                mbar_expect_tx(bar_k_full + stage * 8, kTileBytes);
                tma_load_3d(k_smem + stage * kTileBytes, &k_map, bar_k_full + stage * 8, 0, kv_head, row0);
                tma_load_3d(k_smem + stage * kTileBytes + kHalfTileBytes, &k_map, bar_k_full + stage * 8, 64, kv_head,
                            row0);
            }
            if (lane == 0 && j >= 2) ok = mbar_wait(bar_v_empty + stage * 8, ((j >> 1) - 1) & 1) ? 1 : 0;
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) {
                failed = true;
                break;
            }
            if (lane == 0) {
                mbar_expect_tx(bar_v_full + stage * 8, kTileBytes);
                tma_load_3d(v_smem + stage * kTileBytes, &v_map, bar_v_full + stage * 8, 0, kv_head, row0);
                tma_load_3d(v_smem + stage * kTileBytes + kHalfTileBytes, &v_map, bar_v_full + stage * 8, 64, kv_head,
                            row0);
            }
        }
    } else if (warp == 8) {
        // ---------------- MMA issuer ----------------
        constexpr uint32_t kIdescQK = make_instr_desc(kTile, kTile, true, 0, 0);      // A, B K-major
        constexpr uint32_t kIdescPV = make_instr_desc(kTile, kHeadDim, true, 0, 1);   // B (V) MN-major
        auto wait_all = [&](uint32_t bar, uint32_t parity) -> bool {
            return __all_sync(0xffffffffu, mbar_wait(bar, parity) ? 1 : 0) != 0;
        };
        // S_x = Q_x K(stage)^T
        auto issue_qk = [&](int x, int stage) {
            if (lane == 0) {
                const uint32_t q_tile = q_smem + x * kTileBytes;
                const uint32_t k_tile = k_smem + stage * kTileBytes;
#pragma unroll
                for (int ks = 0; ks < kHeadDim / 16; ++ks) {
                    const uint32_t within = (ks >> 2) * kHalfTileBytes + (ks & 3) * 32;
                    umma_ss(tmem_base + x * kTile, make_smem_desc(q_tile + within, 16, 1024),
                            make_smem_desc(k_tile + within, 16, 1024), kIdescQK, ks > 0 ? 1u : 0u);
                }
                tcgen05_commit(bar_s_full + x * 8);
            }
            __syncwarp();
        };
        // O_x (+)= P_x V(stage): 16 keys per step, P advances 8 packed columns, V two 8-row groups (2 x 1024 bytes);
        // the second 64 dims of V are the next box, 16 KB further (leading byte offset).
        auto issue_pv = [&](int x, int stage, bool accumulate, bool last) {
            if (lane == 0) {
                const uint32_t v_tile = v_smem + stage * kTileBytes;
#pragma unroll
                for (int ks = 0; ks < kTile / 16; ++ks) {
                    umma_ts(tmem_base + 2 * kTile + x * kHeadDim, tmem_base + x * kTile + ks * 8,
                            make_smem_desc(v_tile + ks * 2048, kHalfTileBytes, 1024), kIdescPV,
                            (accumulate || ks > 0) ? 1u : 0u);
                }
                if (last) tcgen05_commit(bar_o_full + x * 8);
            }
            __syncwarp();
        };
        if (!wait_all(bar_q_full, 0) || !wait_all(bar_k_full, 0)) failed = true;
        if (!failed) {
            tcgen05_fence_after();
            if (tiles_needed[0] > 0) issue_qk(0, 0);
            if (tiles_needed[1] > 0) issue_qk(1, 0);
            if (lane == 0) tcgen05_commit(bar_k_empty);
            __syncwarp();
        }
        for (int j = 0; j < key_tiles && !failed; ++j) {
            const int stage = j & 1;
            const int next = (j + 1) & 1;
            const bool more = j + 1 < key_tiles;
            if (!wait_all(bar_v_full + stage * 8, (j >> 1) & 1)) {
                failed = true;
                break;
            }
            if (j < tiles_needed[0]) {
                if (!wait_all(bar_p_full, j & 1)) {
                    failed = true;
                    break;
                }
                tcgen05_fence_after();
                issue_pv(0, stage, j > 0, j == tiles_needed[0] - 1);
            }
            if (more) {
                if (!wait_all(bar_k_full + next * 8, ((j + 1) >> 1) & 1)) {
                    failed = true;
                    break;
                }
                tcgen05_fence_after();
                if (j + 1 < tiles_needed[0]) issue_qk(0, next);
            }
            if (j < tiles_needed[1]) {
                if (!wait_all(bar_p_full + 8, j & 1)) {
                    failed = true;
                    break;
                }
                tcgen05_fence_after();
                issue_pv(1, stage, j > 0, j == tiles_needed[1] - 1);
            }
            if (lane == 0) tcgen05_commit(bar_v_empty + stage * 8);
            __syncwarp();
            if (more) {
                if (j + 1 < tiles_needed[1]) issue_qk(1, next);
                if (lane == 0) tcgen05_commit(bar_k_empty + next * 8);
                __syncwarp();
            }
        }
    } else {
        // ---------------- softmax / correction / epilogue ----------------
        // All eight warps work on the tile whose scores are ready, A then B in turn: a row is shared by two
        // threads, warp w (columns 0-63) and warp w+4 (columns 64-127) of the same tensor-memory lane quarter, so a
        // tile's softmax takes half as long and is done before the other tile's MMAs finish.  The two halves
        // exchange their row maxima through shared memory (an mbarrier with a bounded wait, double-buffered).
        const int quarter = warp & 3;                  // tensor-memory lanes 32*quarter .. +31
        const int half = warp >> 2;                    // which 64 columns of the row
        const int local_row = quarter * 32 + lane;
        const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
        float used_max[2] = {-INFINITY, -INFINITY};   // per tile: the max baked into P, O and row_sum
        float row_sum[2] = {0.0f, 0.0f};               // per tile: this half's share of the row sum
        int turn = 0;                                  // exchanges done so far (selects buffer and barrier phase)
        for (int j = 0; j < key_tiles && !failed; ++j) {
#pragma unroll
            for (int x = 0; x < 2; ++x) {
                if (j >= tiles_needed[x] || failed) continue;
                const int row = q0 + x * kTile + local_row;  // sequence-local query index
                const uint32_t tmem_s = tmem_base + x * kTile + lane_base;
                const uint32_t tmem_o = tmem_base + 2 * kTile + x * kHeadDim + lane_base;
                if (!__all_sync(0xffffffffu, mbar_wait(bar_s_full + x * 8, j & 1) ? 1 : 0)) {
                    failed = true;
                    continue;
                }
                tcgen05_fence_after();
                const int key0 = j * kTile + half * kHalfRow;
                // number of keys of this half-tile the row may see
                int limit = len_kv - key0;
                if (p.causal) limit = min(limit, row + 1 - key0);
                limit = row < len_q ? limit : 0;
                const bool partial = __any_sync(0xffffffffu, limit < kHalfRow);

                uint32_t sc[kHalfRow];
                tmem_ld_x32(tmem_s + half * kHalfRow, *reinterpret_cast<uint32_t(*)[32]>(&sc[0]));
                tmem_ld_x32(tmem_s + half * kHalfRow + 32, *reinterpret_cast<uint32_t(*)[32]>(&sc[32]));
                tmem_wait_ld();

                // pass 1: maximum of this half, then the row maximum through the partner's half
                const float sign = p.scale_log2 < 0.0f ? -1.0f : 1.0f;
                float tile_max = (partial || sign < 0.0f) ? row_max<true>(sc, limit, sign) : row_max<false>(sc, limit, sign);
                tile_max *= fabsf(p.scale_log2);
                float *mine = exchange + ((turn & 1) * 2 + half) * kTile;
                const float *theirs = exchange + ((turn & 1) * 2 + (half ^ 1)) * kTile;
                mine[local_row] = tile_max;
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_exchange);
                if (!__all_sync(0xffffffffu, mbar_wait(bar_exchange, turn & 1) ? 1 : 0)) {
                    failed = true;
                    continue;
                }
                ++turn;
                tile_max = fmaxf(tile_max, theirs[local_row]);
                const float wanted = fmaxf(used_max[x], tile_max);
                // Rescale O only when some row's max grew past the threshold; then every row of the warp re-bases.
                // Both halves see the same row maxima, so they take the same decision.
                const bool grow = wanted > used_max[x] + kRescaleThreshold ||
                                  (used_max[x] == -INFINITY && wanted > -INFINITY);
                if (__any_sync(0xffffffffu, grow)) {
                    const float factor = used_max[x] == -INFINITY ? 0.0f : exp2_approx(used_max[x] - wanted);
                    if (j > 0) {
                        row_sum[x] *= factor;
#pragma unroll 1
                        for (int c = 0; c < kHalfRow; c += 32) {  // this half's 64 columns of O
                            uint32_t r[32];
                            tmem_ld_x32(tmem_o + half * kHalfRow + c, r);
                            tmem_wait_ld();
#pragma unroll
                            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * factor);
                            tmem_st_x32(tmem_o + half * kHalfRow + c, r);
                        }
                        tmem_wait_st();
                    }
                    used_max[x] = wanted;
                }
                // pass 2: P = exp2(s * scale - used_max), row sum, bf16 pairs back into tensor memory
                const float bias = used_max[x] == -INFINITY ? 0.0f : -used_max[x];
                row_sum[x] += partial ? row_exp_store<true>(sc, tmem_s + half * (kHalfRow / 2), p.scale_log2, bias, limit)
                                      : row_exp_store<false>(sc, tmem_s + half * (kHalfRow / 2), p.scale_log2, bias, limit);
                tmem_wait_st();
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(bar_p_full + x * 8);
                }
            }
        }
        // ---- epilogue: the halves add their row sums, then each writes its 64 output columns ----
#pragma unroll
        for (int x = 0; x < 2; ++x) {
            if (tiles_needed[x] == 0 || failed) continue;
            const int row = q0 + x * kTile + local_row;
            const uint32_t tmem_o = tmem_base + 2 * kTile + x * kHeadDim + lane_base;
            float *mine = exchange + ((turn & 1) * 2 + half) * kTile;
            const float *theirs = exchange + ((turn & 1) * 2 + (half ^ 1)) * kTile;
            mine[local_row] = row_sum[x];
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_exchange);
            if (!__all_sync(0xffffffffu, mbar_wait(bar_exchange, turn & 1) ? 1 : 0)) {
                failed = true;
                continue;
            }
            ++turn;
            const float total = row_sum[x] + theirs[local_row];
            if (!__all_sync(0xffffffffu, mbar_wait(bar_o_full + x * 8, 0) ? 1 : 0)) {
                failed = true;
                continue;
            }
            tcgen05_fence_after();
            const bool real = row < len_q;
            const bool empty = total == 0.0f;
            const float inverse = empty ? 0.0f : 1.0f / total;
            const size_t token = static_cast<size_t>(offset) + (real ? row : 0);
            __nv_bfloat16 *dst = p.out + (token * p.heads + head) * kHeadDim + half * kHalfRow;
#pragma unroll 1
            for (int c = 0; c < kHalfRow; c += 32) {
                uint32_t r[32];
                tmem_ld_x32(tmem_o + half * kHalfRow + c, r);
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
            if (real && half == 0) {
                p.lse[token * p.heads + head] =
                    empty ? -1.0e20f : (used_max[x] + log2f(total)) * 0.6931471805599453f;
            }
        }
    }
    if (failed && lane == 0) {
        report_status(p.error, kStatusWaitTimeout);
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 8) {
        tcgen05_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

constexpr int kPrefillSmem = 6 * kTileBytes + 160 + 4 * kTile * 4 + kMaxRankTiles * 4 + 1024;

}  // namespace

bool prefill_fast_path(size_t heads, size_t kv_heads, size_t head_dim, size_t total_query_tokens, const void *query,
                       const void *key, const void *value, const void *out) {
    // The heaviest-first dispatch table holds kMaxRankTiles query pairs per sequence.
    if (total_query_tokens / kPair + 1 > kMaxRankTiles) return false;
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
    // Upper bound on 256-row query pairs: every sequence can add one partial pair.
    const size_t pairs = total_query_tokens / kPair + batch;
    if (pairs > 0x7fffffffull) return SINGE_ERR_LENGTH_EXCEEDS_I32;
    dim3 grid(static_cast<unsigned>(pairs), static_cast<unsigned>(heads));
    prefill_tcgen05_kernel<<<grid, kPrefillThreads, kPrefillSmem, stream>>>(q_map, k_map, v_map, params);
    return launch_status();
}

}  // namespace singe
