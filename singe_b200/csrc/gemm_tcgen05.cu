// bf16 linear-layer GEMM on the tcgen05 tensor core:  out[M, N] = lhs[M, K] . rhs[N, K]^T, f32 accumulate.
//
// Meaning: Linear::forward = x.matmul(W^T) (singe/src/nn/layers/linear/mod.rs:49-70); CPU form bf16 -> f32,
// ascending-k sum, one rounding of the result (singe/src/backend/cpu/binary/matmul.rs:18-43,
// singe-kernel/src/cpu/matmul/blocked.rs:27-95).  Replaces singe_tcgen05_matmul
// (singe/src/backend/cuda/kernel_plan/source/tcgen05.rs:137-266), which is single-stage and cp.async-fed.
//
// Structure: persistent CTAs (one per SM), warp-specialised.
//   warp 0   TMA producer: A tile [a_rows x 64] and B tile [BN x 64] of bf16 per stage, SWIZZLE_128B, ring of
//            `stages` mbarrier pairs.
//   warp 1   MMA issuer: owns tensor memory (2 accumulators of BN columns), issues four
//            tcgen05.mma 128 x BN x 16 per stage, commits the stage back to the producer and, after the last
//            k-block, the accumulator to the epilogue.
//   warps 2-5 epilogue: tcgen05.ld 32 columns at a time, convert, store; then hand the accumulator back, so
//            the MMA of the next tile overlaps this tile's epilogue.
// In the linear-layer form both operands are K-major, so M/N/K tails come for free from TMA's zero fill; stores are
// masked.  The other layouts of MatmulConfig (lhs [K, M], rhs [K, N]; singe-kernel/src/cuda/matmul.rs:190-246) are
// template forms of the same kernels: such an operand is staged in boxes of 64 contiguous M or N elements and read
// by the MMA as an MN-major operand.
// Small M (decode batches) uses narrow BN so that enough CTAs stream the weight matrix to fill HBM, and a
// short A box: rows past the box are stale shared memory, which only reaches output rows that are not stored.
// Tiles are ordered in groups of eight M-tiles so that one wave of CTAs shares A and B tiles through L2.
// Every mbarrier wait is bounded; a wait that runs out sets the device error word and the CTA leaves.
#include <atomic>

#include "common.cuh"
#include "tcgen05.cuh"

namespace singe {

namespace {

constexpr int kGemmThreads = 192;
// The split-K kernel carries six more warps that do nothing but join its last phase: adding up the CTA's rows and
// applying the epilogue is a few hundred dependent instructions, and with one warp per scheduler every one of them
// waits out its own latency.
constexpr int kSplitKThreads = 384;
constexpr int kBlockM = 128;
constexpr int kBlockK = 64;
constexpr int kMaxStages = 16;
constexpr int kGroupM = 8;

struct GemmParams {
    void *out;
    int out_f32;
    int m, n, k;
    long long ldo;
    int a_rows;       // rows of the A box (multiple of 8, <= 128)
    int stages;
    int stage_bytes;  // KPS * (a_rows * 128 + BN * 128)
    int pad_bytes;    // behind the ring: what the MMA's read of 128 A rows may touch past the last stage's short A box
    int tiles_m, tiles_n, k_blocks;  // k_blocks counts stages: KPS 64-wide slices each
    int vector_store;  // 16-byte stores are legal (alignment and stride)
    int gated;         // 1: columns are (gate, up) pairs; the epilogue stores bf16(bf16(silu(gate)) * up), n / 2 wide
    int stable_rhs;    // 1: the caller vouches that rhs (a weight matrix) is not written by work still in flight, so
                       //    its first tiles are fetched before the wait on the preceding kernels
    int prefetch_blocks;  // with stable_rhs: k-blocks beyond the ring whose rhs tiles are pulled into L2 before the wait
    int rhs_kn;        // 1: rhs is stored [K, N] (transpose_rhs == 0): its tiles are staged N-contiguous and the MMA
                       //    reads them as an MN-major operand; 0: [N, K], K-major (a linear layer's weight)
    uint32_t *error;   // sticky device error word (2 = a bounded wait ran out)
    int lhs_km;        // 1: lhs is stored [K, M] (transpose_lhs != 0), staged M-contiguous and read as an MN-major A operand
    WarmRange warm;    // pulled into L2 by the epilogue warps while they have nothing else to do
};

// GatedMlp's activation-then-multiply (singe/src/nn/layers/feed_forward/mod.rs:58-66) on two accumulators, with the
// roundings of the unfused chain: both projections to bf16, silu to bf16, the product to bf16 (by the caller's store).
__device__ __forceinline__ float gated_value(float gate_acc, float up_acc) {
    const float gate = __bfloat162float(__float2bfloat16_rn(gate_acc));
    const float up = __bfloat162float(__float2bfloat16_rn(up_acc));
    const float activated = __bfloat162float(__float2bfloat16_rn(silu_fast(gate)));
    return activated * up;
}

// One 64-wide K slice of the B operand into shared memory (BN x 128 bytes either way).  [N, K] weights: one box of BN
// rows x 64 K-elements.  [K, N] right operands: BN / 64 boxes of 64 K-rows x 64 N-elements, 8 KB apart, which the MMA
// reads MN-major (leading byte offset 8 KB to the next 64 columns, 1 KB to the next eight K-rows, 2 KB per 16-wide k step).
template <int BN, bool KN>
__device__ __forceinline__ void load_b_slice(uint32_t dst, const CUtensorMap *map, uint32_t bar, int k0, int n0) {
    if (!KN) {
        tma_load_2d(dst, map, bar, k0, n0);
    } else {
#pragma unroll
        for (int h = 0; h < BN / 64; ++h) tma_load_2d(dst + h * 8192, map, bar, n0 + h * 64, k0);
    }
}

template <int BN, bool KN>
__device__ __forceinline__ void prefetch_b_slice(const CUtensorMap *map, int k0, int n0) {
    if (!KN) {
        tma_prefetch_2d(map, k0, n0);
    } else {
#pragma unroll
        for (int h = 0; h < BN / 64; ++h) tma_prefetch_2d(map, n0 + h * 64, k0);
    }
}

// How the MMA walks a B slice: the leading byte offset of the shared-memory descriptor and what one 16-wide k step
// adds to its address field (16-byte units): 32 bytes along a K-major row, or sixteen 128-byte K-rows of an MN-major
// tile.  The layout is a template argument of the kernels (KN), so the linear-layer form carries no trace of the other.
template <bool KN>
struct BWalk {
    static constexpr uint32_t kLeadingBytes = KN ? 8192u : 16u;
    static constexpr uint32_t kStep = KN ? 128u : 2u;
};

__device__ __forceinline__ void tile_coordinates(int tile, int tiles_m, int tiles_n, int &tm, int &tn) {
    const int per_group = kGroupM * tiles_n;
    const int group = tile / per_group;
    const int first_m = group * kGroupM;
    const int rows = min(kGroupM, tiles_m - first_m);
    const int within = tile - group * per_group;
    tm = first_m + within % rows;
    tn = within / rows;
}

// KPS = 64-wide K slices per pipeline stage.  Skinny problems stream the weight matrix from HBM; with one
// slice per stage every request touches 128 contiguous bytes of a weight row, which opens a DRAM page for two
// bursts.  Several adjacent slices issued together give the memory controller 512-1024 contiguous bytes per row.
// AT: the left operand is stored [K, M]; its 128 x 64 tile is two boxes of 64 K-rows x 64 M-columns, 8 KB apart, read
// MN-major like a [K, N] right operand.
// MT = 2: a tile is 256 rows, two 128-row MMAs per k step that read the same B slice: 64 KB of operands per 1024 clk
// of tensor-core work instead of 48 KB per 512, which is what one SM can pull out of L2 (the 128 x 256 tile runs at the
// SM's L2 read bandwidth, about 106 GB/s, not at the tensor core's rate).  Both accumulators belong to the one tile
// (columns [0, BN) and [BN, 2 BN)), so the epilogue of a tile no longer overlaps the next tile's MMAs.
template <int BN, int KPS, bool KN, bool AT = false, int MT = 1>
__global__ void __launch_bounds__(kGemmThreads, 1)
    gemm_bf16_kernel(const __grid_constant__ CUtensorMap a_map, const __grid_constant__ CUtensorMap b_map,
                     const GemmParams p) {
    constexpr uint32_t kTmemColumns = 2 * BN < 32 ? 32 : 2 * BN;
    constexpr uint32_t kIdesc = make_instr_desc(kBlockM, BN, true, AT ? 1 : 0, KN ? 1 : 0);  // KN / AT: MN-major reads
    constexpr int kBBytes = BN * 128;

    grid_launch_dependents();
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    // [stages x stage_bytes][over-read pad][barriers]
    const uint32_t bars = base + p.stages * p.stage_bytes + p.pad_bytes;
    const uint32_t bar_full = bars;
    const uint32_t bar_empty = bars + kMaxStages * 8;
    const uint32_t bar_acc_full = bars + 2 * kMaxStages * 8;
    const uint32_t bar_acc_empty = bar_acc_full + 16;
    const uint32_t tmem_holder = bar_acc_empty + 16;
    volatile uint32_t *tmem_holder_ptr =
        reinterpret_cast<volatile uint32_t *>(smem_raw + (tmem_holder - raw));

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int a_bytes = p.a_rows * 128;
    const int total_tiles = p.tiles_m * p.tiles_n;

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(bar_full + s * 8, 1);
            mbar_init(bar_empty + s * 8, 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(bar_acc_full + a * 8, 1);
            mbar_init(bar_acc_empty + a * 8, 4);
        }
        mbar_init_fence();
    }
    if (warp == 1) {
        tmem_alloc(tmem_holder, kTmemColumns);
        tmem_relinquish();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_holder_ptr;

    bool failed = false;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            prefetch_tensor_map(&a_map);
            prefetch_tensor_map(&b_map);
        }
        // A stable weight operand does not depend on the kernels before this one: the B halves of the first tile's
        // first `stages` ring slots are requested now (and a few more k-blocks pulled into L2), so that they cross
        // HBM while the preceding kernel is still running.  Each slot's barrier expects the bytes of both operands;
        // the A halves follow after the wait.
        int preloaded = 0;
        if (p.stable_rhs && blockIdx.x < total_tiles) {
            int tm, tn;
            tile_coordinates(blockIdx.x, p.tiles_m, p.tiles_n, tm, tn);
            preloaded = min(p.stages, p.k_blocks);
            if (lane == 0) {
                for (int kb = 0; kb < preloaded; ++kb) {
                    const uint32_t stage = base + kb * p.stage_bytes;
                    const uint32_t full = bar_full + kb * 8;
                    mbar_expect_tx(full, KPS * (MT * a_bytes + kBBytes));
#pragma unroll
                    for (int sub = 0; sub < KPS; ++sub) {
                        load_b_slice<BN, KN>(stage + KPS * MT * a_bytes + sub * kBBytes, &b_map, full, (kb * KPS + sub) * kBlockK,
                                         tn * BN);
                    }
                }
                const int last = min(p.k_blocks, preloaded + p.prefetch_blocks);
                for (int kb = preloaded; kb < last; ++kb) {
#pragma unroll
                    for (int sub = 0; sub < KPS; ++sub) prefetch_b_slice<BN, KN>(&b_map, (kb * KPS + sub) * kBlockK, tn * BN);
                }
            }
        }
        grid_dependency_wait();  // the A operand comes from the kernel before
        int it = 0;
        for (int tile = blockIdx.x; tile < total_tiles && !failed; tile += gridDim.x) {
            int tm, tn;
            tile_coordinates(tile, p.tiles_m, p.tiles_n, tm, tn);
            for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
                const int s = it % p.stages;
                const uint32_t phase = (it / p.stages) & 1;
                const bool early = it < preloaded;  // slot armed and its B half requested before the wait
                int ok = 1;
                if (lane == 0 && !early) ok = mbar_wait(bar_empty + s * 8, phase ^ 1) ? 1 : 0;
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) {
                    failed = true;
                    break;
                }
                if (lane == 0) {
                    const uint32_t stage = base + s * p.stage_bytes;
                    const uint32_t full = bar_full + s * 8;
                    if (!early) mbar_expect_tx(full, KPS * (MT * a_bytes + kBBytes));
#pragma unroll
                    for (int sub = 0; sub < KPS; ++sub) {
                        // slices past K are zero-filled by TMA and add nothing
#pragma unroll
                        for (int mt = 0; mt < MT; ++mt) {
                            const uint32_t a_at = stage + (sub * MT + mt) * a_bytes;
                            const int row0 = (tm * MT + mt) * kBlockM;
                            if (AT) {
                                tma_load_2d(a_at, &a_map, full, row0, (kb * KPS + sub) * kBlockK);
                                tma_load_2d(a_at + 8192, &a_map, full, row0 + 64, (kb * KPS + sub) * kBlockK);
                            } else {
                                tma_load_2d(a_at, &a_map, full, (kb * KPS + sub) * kBlockK, row0);
                            }
                        }
                    }
                    if (!early) {
#pragma unroll
                        for (int sub = 0; sub < KPS; ++sub) {
                            load_b_slice<BN, KN>(stage + KPS * MT * a_bytes + sub * kBBytes, &b_map, full,
                                             (kb * KPS + sub) * kBlockK, tn * BN);
                        }
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        int it = 0;
        int local = 0;
        for (int tile = blockIdx.x; tile < total_tiles && !failed; tile += gridDim.x, ++local) {
            // MT == 1: two accumulators take turns; MT == 2: both belong to every tile
            const int acc = MT == 2 ? 0 : (local & 1);
            const uint32_t acc_phase = MT == 2 ? (local & 1) : ((local >> 1) & 1);
            if (!__all_sync(0xffffffffu, mbar_wait(bar_acc_empty + acc * 8, acc_phase ^ 1) ? 1 : 0)) {
                failed = true;
                break;
            }
            tcgen05_fence_after();
            const uint32_t tmem_d = tmem_base + acc * BN;
            for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
                const int s = it % p.stages;
                const uint32_t phase = (it / p.stages) & 1;
                if (!__all_sync(0xffffffffu, mbar_wait(bar_full + s * 8, phase) ? 1 : 0)) {
                    failed = true;
                    break;
                }
                tcgen05_fence_after();
                if (lane == 0) {
                    const uint32_t stage = base + s * p.stage_bytes;
#pragma unroll
                    for (int sub = 0; sub < KPS; ++sub) {
                        const uint64_t b_desc =
                            make_smem_desc(stage + KPS * MT * a_bytes + sub * kBBytes, BWalk<KN>::kLeadingBytes, 1024);
#pragma unroll
                        for (int mt = 0; mt < MT; ++mt) {
                            const uint64_t a_desc =
                                make_smem_desc(stage + (sub * MT + mt) * a_bytes, BWalk<AT>::kLeadingBytes, 1024);
#pragma unroll
                            for (int ks = 0; ks < kBlockK / 16; ++ks) {
                                // 16 bf16 of K: 2 descriptor address units along a K-major row, 128 down an MN-major tile
                                umma_ss(tmem_d + mt * BN, a_desc + BWalk<AT>::kStep * ks, b_desc + BWalk<KN>::kStep * ks,
                                        kIdesc, (kb > 0 || sub > 0 || ks > 0) ? 1u : 0u);
                            }
                        }
                    }
                    tcgen05_commit(bar_empty + s * 8);
                }
                __syncwarp();
            }
            if (failed) break;
            if (lane == 0) {
                tcgen05_commit(bar_acc_full + acc * 8);
            }
            __syncwarp();
        }
    } else {
        // ---------------- epilogue ----------------
        if (warp == 2) warm_l2(p.warm, blockIdx.x, gridDim.x, lane);
        grid_dependency_wait();  // nothing is stored while an earlier kernel may still read the output buffer
        const int quarter = warp & 3;  // tensor-memory lanes 32*quarter .. +31
        int local = 0;
        for (int tile = blockIdx.x; tile < total_tiles && !failed; tile += gridDim.x, ++local) {
            int tm, tn;
            tile_coordinates(tile, p.tiles_m, p.tiles_n, tm, tn);
            const int acc = MT == 2 ? 0 : (local & 1);
            const uint32_t acc_phase = MT == 2 ? (local & 1) : ((local >> 1) & 1);
            if (!__all_sync(0xffffffffu, mbar_wait(bar_acc_full + acc * 8, acc_phase) ? 1 : 0)) {
                failed = true;
                break;
            }
            tcgen05_fence_after();
#pragma unroll 1
            for (int mt = 0; mt < MT; ++mt) {
            const int row = (tm * MT + mt) * kBlockM + quarter * 32 + lane;
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + (acc + mt) * BN;
#pragma unroll 1
            for (int c = 0; c < BN; c += 32) {
                uint32_t r[32];
                tmem_ld_x32(taddr + c, r);
                tmem_wait_ld();
                const int col = tn * BN + c;
                if (row < p.m && col < p.n && p.gated) {
                    __nv_bfloat16 *dst =
                        static_cast<__nv_bfloat16 *>(p.out) + static_cast<long long>(row) * p.ldo + col / 2;
                    if (p.vector_store && col + 32 <= p.n) {
#pragma unroll
                        for (int j = 0; j < 32; j += 16) {
                            uint4 packed;
                            uint32_t *words = &packed.x;
#pragma unroll
                            for (int w = 0; w < 4; ++w) {
                                words[w] = pack2<__nv_bfloat16>(
                                    gated_value(__uint_as_float(r[j + 4 * w]), __uint_as_float(r[j + 4 * w + 1])),
                                    gated_value(__uint_as_float(r[j + 4 * w + 2]), __uint_as_float(r[j + 4 * w + 3])));
                            }
                            *reinterpret_cast<uint4 *>(dst + j / 2) = packed;
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; j += 2) {
                            if (col + j + 1 < p.n) {
                                dst[j / 2] = __float2bfloat16_rn(
                                    gated_value(__uint_as_float(r[j]), __uint_as_float(r[j + 1])));
                            }
                        }
                    }
                } else if (row < p.m && col < p.n) {
                    if (p.out_f32) {
                        float *dst = static_cast<float *>(p.out) + static_cast<long long>(row) * p.ldo + col;
                        if (p.vector_store && col + 32 <= p.n) {
#pragma unroll
                            for (int j = 0; j < 32; j += 4) {
                                *reinterpret_cast<uint4 *>(dst + j) = make_uint4(r[j], r[j + 1], r[j + 2], r[j + 3]);
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j) {
                                if (col + j < p.n) dst[j] = __uint_as_float(r[j]);
                            }
                        }
                    } else {
                        __nv_bfloat16 *dst =
                            static_cast<__nv_bfloat16 *>(p.out) + static_cast<long long>(row) * p.ldo + col;
                        if (p.vector_store && col + 32 <= p.n) {
#pragma unroll
                            for (int j = 0; j < 32; j += 8) {
                                uint4 packed;
                                packed.x = pack2<__nv_bfloat16>(__uint_as_float(r[j]), __uint_as_float(r[j + 1]));
                                packed.y = pack2<__nv_bfloat16>(__uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
                                packed.z = pack2<__nv_bfloat16>(__uint_as_float(r[j + 4]), __uint_as_float(r[j + 5]));
                                packed.w = pack2<__nv_bfloat16>(__uint_as_float(r[j + 6]), __uint_as_float(r[j + 7]));
                                *reinterpret_cast<uint4 *>(dst + j) = packed;
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j) {
                                if (col + j < p.n) dst[j] = __float2bfloat16_rn(__uint_as_float(r[j]));
                            }
                        }
                    }
                }
            }
            }  // mt
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(bar_acc_empty + acc * 8);
            }
        }
    }
    if (failed && lane == 0) {
        report_status(p.error, kStatusWaitTimeout);
    }
    if (failed) linger_after_timeout();
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after();
        tmem_dealloc(tmem_base, kTmemColumns);
    }
}

// ---- split-K for one-M-tile problems whose N gives too few tiles to fill the machine ----
// A thread-block cluster of `splits` CTAs owns one N tile; CTA r of the cluster streams K slice r (its own TMA ring,
// its own accumulator in tensor memory) and pushes each row of its f32 partial tile into the shared memory of the
// cluster CTA that owns the row (distributed shared memory stores); after one cluster barrier every CTA sums its
// rows' partials out of its own shared memory, in split order (so the result does not depend on timing), and stores
// them.  No workspace in global memory, no atomics, nothing to reset between launches.  A timeline of the earlier
// form (partials parked locally, owners pulling them with remote loads, a second barrier before leaving) showed
// 2.2 - 2.6 us in the pull and 0.8 us in the closing barrier of a 10 us kernel.
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t value;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(value));
    return value;
}

__device__ __forceinline__ uint32_t cluster_size() {
    uint32_t value;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(value));
    return value;
}

// Every thread of every CTA of the cluster takes part; shared-memory writes before it are visible cluster-wide after.
__device__ __forceinline__ void cluster_barrier() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

template <int BN, int KPS, bool KN>
__global__ void __launch_bounds__(kSplitKThreads, 1)
    gemm_splitk_kernel(const __grid_constant__ CUtensorMap a_map, const __grid_constant__ CUtensorMap b_map,
                       const GemmParams p) {
    constexpr uint32_t kTmemColumns = BN < 32 ? 32 : BN;
    constexpr uint32_t kIdesc = make_instr_desc(kBlockM, BN, true, 0, KN ? 1 : 0);  // KN: B read MN-major
    constexpr int kBBytes = BN * 128;
    constexpr int kQuads = BN / 4;  // float4 groups per row

    grid_launch_dependents();
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    const uint32_t rank = cluster_rank();
    const uint32_t splits = cluster_size();
    const int rows_per_cta = (p.m + static_cast<int>(splits) - 1) / static_cast<int>(splits);
    // [ring: stages x stage_bytes, its start reused for the parked partial tile][over-read pad]
    // [receive area: splits x rows_per_cta x BN floats][barriers]
    const uint32_t slot_bytes = static_cast<uint32_t>(rows_per_cta) * BN * 4;  // one CTA's rows of one split's partial
    const uint32_t recv = base + max(static_cast<uint32_t>(p.stages * p.stage_bytes), splits * slot_bytes) + p.pad_bytes;
    const uint32_t bars = recv + splits * slot_bytes;
    const uint32_t bar_full = bars;
    const uint32_t bar_empty = bars + kMaxStages * 8;
    const uint32_t bar_acc_full = bars + 2 * kMaxStages * 8;
    const uint32_t bar_recv = bar_acc_full + 8;
    const uint32_t tmem_holder = bar_acc_full + 16;
    volatile uint32_t *tmem_holder_ptr = reinterpret_cast<volatile uint32_t *>(smem_raw + (tmem_holder - raw));

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int a_bytes = p.a_rows * 128;
    const int tn = blockIdx.x / splits;
    const int per_split = (p.k_blocks + splits - 1) / splits;
    const int kb_first = rank * per_split;
    const int kb_last = min(kb_first + per_split, p.k_blocks);  // may leave this CTA without work: its partial is zero
    const bool has_work = kb_first < kb_last;

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(bar_full + s * 8, 1);
            mbar_init(bar_empty + s * 8, 1);
        }
        mbar_init(bar_acc_full, 1);
        mbar_init(bar_recv, 1);
        mbar_init_fence();
    }
    if (warp == 1) {
        tmem_alloc(tmem_holder, kTmemColumns);
        tmem_relinquish();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_holder_ptr;
    cluster_barrier();  // every CTA's receive barrier exists before anyone may complete bytes on it

    bool failed = false;
    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            prefetch_tensor_map(&a_map);
            prefetch_tensor_map(&b_map);
        }
        // Stable weights: the B halves of this CTA's first ring slots are requested before the wait (see
        // gemm_bf16_kernel), a few more k-blocks are pulled into L2.
        int preloaded = 0;
        if (p.stable_rhs && has_work) {
            preloaded = min(p.stages, kb_last - kb_first);
            if (lane == 0) {
                for (int i = 0; i < preloaded; ++i) {
                    const int kb = kb_first + i;
                    const uint32_t stage = base + i * p.stage_bytes;
                    const uint32_t full = bar_full + i * 8;
                    mbar_expect_tx(full, KPS * (a_bytes + kBBytes));
#pragma unroll
                    for (int sub = 0; sub < KPS; ++sub) {
                        load_b_slice<BN, KN>(stage + KPS * a_bytes + sub * kBBytes, &b_map, full, (kb * KPS + sub) * kBlockK,
                                         tn * BN);
                    }
                }
                const int last = min(kb_last, kb_first + preloaded + p.prefetch_blocks);
                for (int kb = kb_first + preloaded; kb < last; ++kb) {
#pragma unroll
                    for (int sub = 0; sub < KPS; ++sub) prefetch_b_slice<BN, KN>(&b_map, (kb * KPS + sub) * kBlockK, tn * BN);
                }
            }
        }
        grid_dependency_wait();  // the A operand comes from the kernel before
        int it = 0;
        for (int kb = kb_first; kb < kb_last; ++kb, ++it) {
            const int s = it % p.stages;
            const uint32_t phase = (it / p.stages) & 1;
            const bool early = it < preloaded;
            int ok = 1;
            if (lane == 0 && !early) ok = mbar_wait(bar_empty + s * 8, phase ^ 1) ? 1 : 0;
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) {
                failed = true;
                break;
            }
            if (lane == 0) {
                const uint32_t stage = base + s * p.stage_bytes;
                const uint32_t full = bar_full + s * 8;
                if (!early) mbar_expect_tx(full, KPS * (a_bytes + kBBytes));
#pragma unroll
                for (int sub = 0; sub < KPS; ++sub) {
                    tma_load_2d(stage + sub * a_bytes, &a_map, full, (kb * KPS + sub) * kBlockK, 0);
                }
                if (!early) {
#pragma unroll
                    for (int sub = 0; sub < KPS; ++sub) {
                        load_b_slice<BN, KN>(stage + KPS * a_bytes + sub * kBBytes, &b_map, full, (kb * KPS + sub) * kBlockK,
                                         tn * BN);
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        int it = 0;
        for (int kb = kb_first; kb < kb_last; ++kb, ++it) {
            const int s = it % p.stages;
            const uint32_t phase = (it / p.stages) & 1;
            if (!__all_sync(0xffffffffu, mbar_wait(bar_full + s * 8, phase) ? 1 : 0)) {
                failed = true;
                break;
            }
            tcgen05_fence_after();
            if (lane == 0) {
                const uint32_t stage = base + s * p.stage_bytes;
#pragma unroll
                for (int sub = 0; sub < KPS; ++sub) {
                    const uint64_t a_desc = make_smem_desc(stage + sub * a_bytes, 16, 1024);
                    const uint64_t b_desc =
                        make_smem_desc(stage + KPS * a_bytes + sub * kBBytes, BWalk<KN>::kLeadingBytes, 1024);
#pragma unroll
                    for (int ks = 0; ks < kBlockK / 16; ++ks) {
                        umma_ss(tmem_base, a_desc + 2 * ks, b_desc + BWalk<KN>::kStep * ks, kIdesc,
                                (kb > kb_first || sub > 0 || ks > 0) ? 1u : 0u);
                    }
                }
                tcgen05_commit(bar_empty + s * 8);
            }
            __syncwarp();
        }
        if (!failed && has_work) {
            if (lane == 0) tcgen05_commit(bar_acc_full);
            __syncwarp();
        }
    } else if (warp < 6) {
        // ---------------- hand the partial tile to the CTAs that own its rows ----------------
        // Row i of the tile belongs to cluster CTA i % splits.  The four warps park the CTA's f32 partial tile in its
        // own shared memory grouped by owner ([owner][row / splits][BN], 16-byte groups XOR-swizzled by the row so the
        // one-row-per-thread writes spread over the banks), then one thread sends each other owner its group with a
        // single bulk copy into that CTA's receive area (slot = this CTA's rank), completing bytes on the owner's
        // receive barrier.  An owner waits for the bytes of all live splits and sums its rows out of its own shared
        // memory: no thread ever waits for a remote load.  (Stores of one row per thread straight into the owners'
        // shared memory took 1.6 us for 24 KB per CTA: 4096 separate 16-byte transfers.)
        if (warp == 2) warm_l2(p.warm, blockIdx.x, gridDim.x, lane);
        grid_dependency_wait();  // these warps store the output: not while an earlier kernel may still read it
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;
        const int live = min(static_cast<int>(splits), (p.k_blocks + per_split - 1) / per_split);
        if (has_work && !__all_sync(0xffffffffu, mbar_wait(bar_acc_full, 0) ? 1 : 0)) failed = true;
        tcgen05_fence_after();
        if (has_work && !failed) {
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
            const int owner = row % static_cast<int>(splits);
            const int local_row = row / static_cast<int>(splits);
            float *mine = reinterpret_cast<float *>(smem_raw + (base - raw)) +
                          (static_cast<size_t>(owner) * rows_per_cta + local_row) * BN;
#pragma unroll 1
            for (int c = 0; c < BN; c += 32) {
                uint32_t r[32];
                tmem_ld_x32(taddr + c, r);
                tmem_wait_ld();
                if (row < p.m) {
#pragma unroll
                    for (int j = 0; j < 32; j += 4) {
                        const int quad = ((c + j) >> 2) ^ (row & (kQuads - 1));
                        *reinterpret_cast<float4 *>(mine + quad * 4) =
                            make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]),
                                        __uint_as_float(r[j + 3]));
                    }
                }
            }
            fence_proxy_async_shared();  // the bulk copies below read what these threads wrote
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");  // the four epilogue warps: the whole tile is parked
        if (threadIdx.x == 64) {
            // bytes this CTA will receive: one slot from every other live split
            const int senders = live - (static_cast<int>(rank) < live ? 1 : 0);
            mbar_expect_tx(bar_recv, static_cast<uint32_t>(senders) * slot_bytes);
            if (has_work && !failed) {
                for (uint32_t o = 0; o < splits; ++o) {
                    if (o == rank) continue;
                    uint32_t remote_slot, remote_bar;
                    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;"
                                 : "=r"(remote_slot)
                                 : "r"(recv + rank * slot_bytes), "r"(o));
                    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote_bar) : "r"(bar_recv), "r"(o));
                    asm volatile(
                        "cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                        ::"r"(remote_slot), "r"(base + o * slot_bytes), "r"(slot_bytes), "r"(remote_bar)
                        : "memory");
                }
            }
        }
    }
    // Every warp helps with the reduction (the producer and MMA warps have nothing left to do): all of them wait for
    // the bytes addressed to this CTA.
    if (!__all_sync(0xffffffffu, mbar_wait(bar_recv, 0) ? 1 : 0)) failed = true;
    if (failed && lane == 0) {
        report_status(p.error, kStatusWaitTimeout);
    }
    if (failed) linger_after_timeout();
    // Arrive: "everything addressed to this CTA has landed".  When all CTAs have said so, every bulk copy of the
    // cluster has finished reading its source, and a CTA may leave (the matching wait is at the end).
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    {
        // ---------------- reduce: CTA r owns rows r, r + splits, ... of the tile ----------------
        if (warp < 2 || warp >= 6) grid_dependency_wait();  // (warps 2-5 did before they parked the tile)
        const int t = threadIdx.x;
        const int my_rows = (p.m - static_cast<int>(rank) + static_cast<int>(splits) - 1) / static_cast<int>(splits);
        const int live = min(static_cast<int>(splits), (p.k_blocks + per_split - 1) / per_split);
        const float *received = reinterpret_cast<const float *>(smem_raw + (recv - raw));
        const float *parked = reinterpret_cast<const float *>(smem_raw + (base - raw));
        const int slot_floats = rows_per_cta * BN;
        // One warp per scheduler runs here, so nothing hides an instruction's latency but the warp's own independent
        // work: the shared-memory reads of a batch of items are issued together before any of them is summed.
        constexpr int kBatch = 2;
        const int items = my_rows * kQuads;
        for (int first = t; first < items; first += kSplitKThreads * kBatch) {
            float4 part[kBatch][8];
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {
                const int index = first + u * kSplitKThreads;
                const int local_row = index / kQuads;
                const int quad = index % kQuads;
                const int row = static_cast<int>(rank) + local_row * static_cast<int>(splits);
                const int at = local_row * BN + ((quad ^ (row & (kQuads - 1))) << 2);
#pragma unroll
                for (int s = 0; s < 8; ++s) {
                    if (index < items && s < live) {
                        // this CTA's own partial never left its parked tile (group `rank` there)
                        const float *from = s == static_cast<int>(rank) ? parked + rank * slot_floats
                                                                         : received + s * slot_floats;
                        part[u][s] = *reinterpret_cast<const float4 *>(from + at);
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {
                const int index = first + u * kSplitKThreads;
                if (index >= items) continue;
                const int local_row = index / kQuads;
                const int row = static_cast<int>(rank) + local_row * static_cast<int>(splits);
                const int quad = index % kQuads;
                const int col = tn * BN + quad * 4;
                if (col >= p.n) continue;
                float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                if (live > 0) sum = part[u][0];
#pragma unroll
                for (int s = 1; s < 8; ++s) {  // split order: the result does not depend on timing
                    if (s < live) {
                        sum.x += part[u][s].x;
                        sum.y += part[u][s].y;
                        sum.z += part[u][s].z;
                        sum.w += part[u][s].w;
                    }
                }
                const float values[4] = {sum.x, sum.y, sum.z, sum.w};
                if (p.gated) {
                    __nv_bfloat16 *dst =
                        static_cast<__nv_bfloat16 *>(p.out) + static_cast<long long>(row) * p.ldo + col / 2;
                    if (col + 4 <= p.n) {
                        *reinterpret_cast<uint32_t *>(dst) =
                            pack2<__nv_bfloat16>(gated_value(sum.x, sum.y), gated_value(sum.z, sum.w));
                    } else if (col + 2 <= p.n) {
                        dst[0] = __float2bfloat16_rn(gated_value(sum.x, sum.y));
                    }
                } else if (p.out_f32) {
                    float *dst = static_cast<float *>(p.out) + static_cast<long long>(row) * p.ldo + col;
                    if (p.vector_store && col + 4 <= p.n) {
                        *reinterpret_cast<float4 *>(dst) = sum;
                    } else {
                        for (int j = 0; j < 4; ++j) {
                            if (col + j < p.n) dst[j] = values[j];
                        }
                    }
                } else {
                    __nv_bfloat16 *dst =
                        static_cast<__nv_bfloat16 *>(p.out) + static_cast<long long>(row) * p.ldo + col;
                    if (p.vector_store && col + 4 <= p.n) {
                        *reinterpret_cast<uint2 *>(dst) =
                            make_uint2(pack2<__nv_bfloat16>(sum.x, sum.y), pack2<__nv_bfloat16>(sum.z, sum.w));
                    } else {
                        for (int j = 0; j < 4; ++j) {
                            if (col + j < p.n) dst[j] = __float2bfloat16_rn(values[j]);
                        }
                    }
                }
            }
        }
    }
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");  // see the arrive above
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after();
        tmem_dealloc(tmem_base, kTmemColumns);
    }
}

// Explicit tuning (the reference's TuningChoice::Explicit(MatmulTuning), singe-kernel/src/cuda/matmul.rs:58-77):
// 0 = choose from the problem shape.  Atomics: calls on several host threads may race with a setter.
std::atomic<int> g_tuning_block_n{0};
std::atomic<int> g_tuning_slices{0};
std::atomic<int> g_tuning_splits{0};       // 0 = choose, 1 = never split K
std::atomic<int> g_tuning_shared_kb{0};    // 0 = choose; otherwise the dynamic shared memory a CTA may take, in KB
std::atomic<int> g_tuning_prefetch_kb{-1};  // -1 = choose; KB of stable weights per CTA pulled into L2 before the wait

// Dynamic shared memory a GEMM CTA may use.  One-M-tile problems with stable weights are the decode step's linears:
// kept to half an SM so that the CTAs of the next linear can become resident beside them and fetch their own first
// weight tiles while this one still runs; everything else takes the whole SM.
int shared_limit(const GemmParams &params) {
    const int forced = g_tuning_shared_kb.load(std::memory_order_relaxed);
    if (forced > 0) return forced * 1024 > 227 * 1024 ? 227 * 1024 : forced * 1024;
    return 227 * 1024;
}

// The MMA reads 128 rows of A from every stage although a short box fills only a_rows of them; what it reads past the
// box lies inside the stage while the B tiles behind the last A tile are at least as large as the overhang.
int over_read_pad(int a_rows, int stage_b_bytes) {
    const int overhang = (kBlockM - a_rows) * 128 - stage_b_bytes;
    return overhang > 0 ? (overhang + 1023) / 1024 * 1024 : 0;
}

int prefetch_blocks_for(const GemmParams &params, int block_b_bytes) {
    if (!params.stable_rhs) return 0;
    const int forced = g_tuning_prefetch_kb.load(std::memory_order_relaxed);
    const int kb = forced >= 0 ? forced : 0;
    return kb * 1024 / block_b_bytes;
}

template <int BN, int KPS>
int launch_gemm_splitk(cudaStream_t stream, GemmParams params, const void *lhs, const void *rhs,
                       size_t lhs_row_stride, size_t rhs_row_stride, int splits) {
    const int kSmemLimit = shared_limit(params);
    const int b_bytes = BN * 128;
    params.stage_bytes = KPS * (params.a_rows * 128 + b_bytes);
    params.k_blocks = (params.k + kBlockK * KPS - 1) / (kBlockK * KPS);
    params.prefetch_blocks = prefetch_blocks_for(params, KPS * b_bytes);
    const int per_split = (params.k_blocks + splits - 1) / splits;
    params.pad_bytes = over_read_pad(params.a_rows, KPS * b_bytes);
    const int receive = splits * ((params.m + splits - 1) / splits) * BN * 4;  // every split's partial of the CTA's rows
    const int fixed = params.pad_bytes + receive + 2 * kMaxStages * 8 + 64 + 1024;
    // (the ring is at least as large as the parked tile, which reuses it: checked below)
    int stages = (kSmemLimit - fixed) / params.stage_bytes;
    if (stages > kMaxStages) stages = kMaxStages;
    if (stages > per_split + 1 && per_split + 1 >= 2) stages = per_split + 1;
    if (stages < 2) stages = 2;  // the limit is a preference; two stages is the least the pipeline runs with
    params.stages = stages;
    params.tiles_n = (params.n + BN - 1) / BN;
    const int ring = stages * params.stage_bytes > receive ? stages * params.stage_bytes : receive;
    const int smem = ring + fixed;
    if (smem > 227 * 1024) return SINGE_ERR_UNSUPPORTED_CONFIGURATION;
    // [K, N] right operands are staged in boxes of 64 columns: those kernels exist from 64-wide tiles up
    constexpr bool kHasKN = BN >= 64;
    if (params.rhs_kn && !kHasKN) return SINGE_ERR_UNSUPPORTED_CONFIGURATION;
    static int configured[kMaxDevices] = {0};
    static int configured_kn[kMaxDevices] = {0};
    if (params.rhs_kn) {
        SINGE_CUDA_TRY(ensure_dynamic_shared(gemm_splitk_kernel<BN, KPS, kHasKN>, smem, configured_kn));
    } else {
        SINGE_CUDA_TRY(ensure_dynamic_shared(gemm_splitk_kernel<BN, KPS, false>, smem, configured));
    }

    CUtensorMap a_map, b_map;
    {
        const uint64_t dims[2] = {static_cast<uint64_t>(params.k), static_cast<uint64_t>(params.m)};
        const uint64_t strides[1] = {static_cast<uint64_t>(lhs_row_stride) * 2};
        const uint32_t box[2] = {kBlockK, static_cast<uint32_t>(params.a_rows)};
        SINGE_TRY(encode_tensor_map(&a_map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, lhs, dims, strides, box,
                                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B));
    }
    if (params.rhs_kn) {
        const uint64_t dims[2] = {static_cast<uint64_t>(params.n), static_cast<uint64_t>(params.k)};
        const uint64_t strides[1] = {static_cast<uint64_t>(rhs_row_stride) * 2};
        const uint32_t box[2] = {64, kBlockK};
        SINGE_TRY(encode_tensor_map(&b_map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rhs, dims, strides, box,
                                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B));
    } else {
        const uint64_t dims[2] = {static_cast<uint64_t>(params.k), static_cast<uint64_t>(params.n)};
        const uint64_t strides[1] = {static_cast<uint64_t>(rhs_row_stride) * 2};
        const uint32_t box[2] = {kBlockK, static_cast<uint32_t>(BN)};
        SINGE_TRY(encode_tensor_map(&b_map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rhs, dims, strides, box,
                                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B));
    }
    const dim3 grid(static_cast<unsigned>(params.tiles_n * splits));
    if (params.rhs_kn) {
        SINGE_CUDA_TRY(launch_dependent(gemm_splitk_kernel<BN, KPS, kHasKN>, grid, dim3(kSplitKThreads), smem, stream,
                                        kLaunchGemm, static_cast<unsigned>(splits), a_map, b_map, params));
    } else {
        SINGE_CUDA_TRY(launch_dependent(gemm_splitk_kernel<BN, KPS, false>, grid, dim3(kSplitKThreads), smem, stream,
                                        kLaunchGemm, static_cast<unsigned>(splits), a_map, b_map, params));
    }
    return launch_status();
}

template <int BN, int KPS, bool AT = false, int MT = 1>
int launch_gemm(cudaStream_t stream, GemmParams params, const void *lhs, const void *rhs, size_t lhs_row_stride,
                size_t rhs_row_stride) {
    const int kSmemLimit = shared_limit(params);
    const int b_bytes = BN * 128;
    if (MT == 2) params.tiles_m = (params.m + 2 * kBlockM - 1) / (2 * kBlockM);  // 256-row tiles
    params.stage_bytes = KPS * (MT * params.a_rows * 128 + b_bytes);
    params.k_blocks = (params.k + kBlockK * KPS - 1) / (kBlockK * KPS);
    params.prefetch_blocks = prefetch_blocks_for(params, KPS * b_bytes);
    params.pad_bytes = over_read_pad(params.a_rows, KPS * b_bytes);
    const int fixed = params.pad_bytes + 2 * kMaxStages * 8 + 64 + 1024;
    int stages = (kSmemLimit - fixed) / params.stage_bytes;
    if (stages > kMaxStages) stages = kMaxStages;
    if (stages > params.k_blocks + 1 && params.k_blocks + 1 >= 2) stages = params.k_blocks + 1;
    if (stages < 2) stages = 2;  // the limit is a preference; two stages is the least the pipeline runs with
    params.stages = stages;
    params.tiles_n = (params.n + BN - 1) / BN;
    const int smem = stages * params.stage_bytes + fixed;
    if (smem > 227 * 1024) return SINGE_ERR_UNSUPPORTED_CONFIGURATION;
    constexpr bool kHasKN = BN >= 64;
    if (params.rhs_kn && !kHasKN) return SINGE_ERR_UNSUPPORTED_CONFIGURATION;
    static int configured[kMaxDevices] = {0};
    static int configured_kn[kMaxDevices] = {0};
    if (params.rhs_kn) {
        SINGE_CUDA_TRY(ensure_dynamic_shared(gemm_bf16_kernel<BN, KPS, kHasKN, AT, MT>, smem, configured_kn));
    } else {
        SINGE_CUDA_TRY(ensure_dynamic_shared(gemm_bf16_kernel<BN, KPS, false, AT, MT>, smem, configured));
    }

    CUtensorMap a_map, b_map;
    if (AT) {
        const uint64_t dims[2] = {static_cast<uint64_t>(params.m), static_cast<uint64_t>(params.k)};
        const uint64_t strides[1] = {static_cast<uint64_t>(lhs_row_stride) * 2};
        const uint32_t box[2] = {64, kBlockK};
        SINGE_TRY(encode_tensor_map(&a_map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, lhs, dims, strides, box,
                                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B));
    } else {
        const uint64_t dims[2] = {static_cast<uint64_t>(params.k), static_cast<uint64_t>(params.m)};
        const uint64_t strides[1] = {static_cast<uint64_t>(lhs_row_stride) * 2};
        const uint32_t box[2] = {kBlockK, static_cast<uint32_t>(params.a_rows)};
        SINGE_TRY(encode_tensor_map(&a_map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, lhs, dims, strides, box,
                                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B));
    }
    if (params.rhs_kn) {
        const uint64_t dims[2] = {static_cast<uint64_t>(params.n), static_cast<uint64_t>(params.k)};
        const uint64_t strides[1] = {static_cast<uint64_t>(rhs_row_stride) * 2};
        const uint32_t box[2] = {64, kBlockK};
        SINGE_TRY(encode_tensor_map(&b_map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rhs, dims, strides, box,
                                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B));
    } else {
        const uint64_t dims[2] = {static_cast<uint64_t>(params.k), static_cast<uint64_t>(params.n)};
        const uint64_t strides[1] = {static_cast<uint64_t>(rhs_row_stride) * 2};
        const uint32_t box[2] = {kBlockK, static_cast<uint32_t>(BN)};
        SINGE_TRY(encode_tensor_map(&b_map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rhs, dims, strides, box,
                                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B));
    }
    const int total = params.tiles_m * params.tiles_n;
    const int grid = total < device_sm_count() ? total : device_sm_count();
    if (params.rhs_kn) {
        SINGE_CUDA_TRY(launch_dependent(gemm_bf16_kernel<BN, KPS, kHasKN, AT, MT>, dim3(grid), dim3(kGemmThreads), smem,
                                        stream, kLaunchGemm, 1, a_map, b_map, params));
    } else {
        SINGE_CUDA_TRY(launch_dependent(gemm_bf16_kernel<BN, KPS, false, AT, MT>, dim3(grid), dim3(kGemmThreads), smem,
                                        stream, kLaunchGemm, 1, a_map, b_map, params));
    }
    return launch_status();
}

}  // namespace

// validate_matmul (singe-kernel/src/cuda/matmul.rs:2977-3020), then the layout gate of the tensor-core path.
int gemm_bf16(cudaStream_t stream, void *out, bool out_f32, const void *lhs, const void *rhs, size_t rows,
              size_t columns, size_t reduction, size_t lhs_row_stride, size_t rhs_row_stride,
              size_t output_row_stride, int transpose_lhs, int transpose_rhs, bool gated, unsigned hints) {
    const size_t lhs_min = transpose_lhs ? rows : reduction;
    const size_t rhs_min = transpose_rhs ? reduction : columns;
    if (rows == 0 || columns == 0 || reduction == 0 || lhs_row_stride < lhs_min || rhs_row_stride < rhs_min ||
        output_row_stride < (gated ? columns / 2 : columns) || (gated && (columns % 2 != 0 || out_f32))) {
        return SINGE_ERR_INVALID_LENGTH;
    }
    if (!fits_i32(rows) || !fits_i32(columns) || !fits_i32(reduction) || !fits_i32(lhs_row_stride) ||
        !fits_i32(rhs_row_stride) || !fits_i32(output_row_stride)) {
        return SINGE_ERR_LENGTH_EXCEEDS_I32;
    }
    if (out == nullptr || lhs == nullptr || rhs == nullptr) {
        return SINGE_ERR_NULL_POINTER;
    }
    // Tensor-core path: linear-layer layout, 16-byte aligned rows for TMA.
    const bool aligned = ((reinterpret_cast<uintptr_t>(lhs) | reinterpret_cast<uintptr_t>(rhs)) & 15u) == 0 &&
                         lhs_row_stride % 8 == 0 && rhs_row_stride % 8 == 0;
    // lhs may be [M, K] or [K, M] (transpose_lhs != 0); rhs [N, K] (a linear layer's weight, transpose_rhs != 0) or
    // [K, N].  The gated epilogue belongs to the linear-layer form.
    if (!aligned || (gated && (!transpose_rhs || transpose_lhs))) {
        return SINGE_ERR_UNSUPPORTED_CONFIGURATION;
    }
    GemmParams params;
    params.error = device_error_word();
    params.out = out;
    params.out_f32 = out_f32 ? 1 : 0;
    params.gated = gated ? 1 : 0;
    params.stable_rhs = (hints & SINGE_HINT_STABLE_WEIGHTS) != 0 ? 1 : 0;
    params.warm = take_pending_warm();
    params.rhs_kn = transpose_rhs ? 0 : 1;
    params.lhs_km = transpose_lhs ? 1 : 0;
    params.prefetch_blocks = 0;
    params.m = static_cast<int>(rows);
    params.n = static_cast<int>(columns);
    params.k = static_cast<int>(reduction);
    params.ldo = static_cast<long long>(output_row_stride);
    params.tiles_m = (params.m + kBlockM - 1) / kBlockM;
    params.k_blocks = (params.k + kBlockK - 1) / kBlockK;
    int a_rows = kBlockM;
    if (params.m < kBlockM && !params.lhs_km) {
        a_rows = (params.m + 7) / 8 * 8;
    }
    params.a_rows = a_rows;
    const size_t element = out_f32 ? 4 : 2;
    params.vector_store =
        ((reinterpret_cast<uintptr_t>(out) & 15u) == 0 && (output_row_stride * element) % 16 == 0) ? 1 : 0;
    // Widest tile that still gives every SM a tile; narrow tiles for skinny (HBM-bound) problems, which also take
    // several K slices per stage so that each weight row is requested in long contiguous runs.
    const int sms = device_sm_count();
    auto tiles = [&](int bn) { return params.tiles_m * ((params.n + bn - 1) / bn); };
    int bn = 32;
    int slices = 1;
    if (params.m > kBlockM) {
        if (tiles(256) >= sms) bn = 256;
        else if (tiles(128) >= sms) bn = 128;
        else if (tiles(64) >= sms) bn = 64;
    } else {
        // One M tile: the weight matrix is streamed once.  Measured on B200 (M = 1..128, N = 4096..28672,
        // K = 4096/14336): 128-wide tiles with 2 slices win once they give two thirds of the SMs a tile,
        // otherwise the narrowest tile that does, with as many slices per stage as two stages allow.
        const int enough = (sms * 2) / 3;
        if (tiles(128) >= enough) {
            bn = 128;
            slices = 2;
        } else {
            bn = tiles(64) >= enough ? 64 : 32;
            const int slice_bytes = (params.a_rows + bn) * 128;
            slices = 8;
            while (slices > 1 && slices * slice_bytes * 2 > 200 * 1024) slices >>= 1;
        }
    }
    // One M tile and too few N tiles for the machine: split K over a cluster instead of narrowing the tile.  The
    // tile stays 128 wide with 2 slices per stage (the best streaming shape measured).  Measured on B200 (M = 16..128,
    // N = 768..6144, K = 512..14336): the best cluster is the largest of 2 / 4 whose CTAs still fit the machine in one
    // wave; 8 pays only when even 4 leave two thirds of the SMs idle (then with 64-wide tiles), and a split needs at
    // least three pipeline stages of K to amortise its fill and the reduction.
    int splits = 1;
    const int forced_splits = g_tuning_splits.load(std::memory_order_relaxed);
    const int forced_block_n = g_tuning_block_n.load(std::memory_order_relaxed);
    const int forced_slices = g_tuning_slices.load(std::memory_order_relaxed);
    if (params.m <= kBlockM && tiles(128) < (sms * 2) / 3 && forced_splits != 1) {
        int wide = 128;
        int wanted = 1;
        while (wanted < 4 && tiles(wide) * wanted * 2 <= sms) wanted <<= 1;
        if (wanted == 4 && tiles(wide) * 4 <= sms / 3) {
            wanted = 8;
            wide = 64;
        }
        const int stage_k = kBlockK * 2;
        const int k_stages = (params.k + stage_k - 1) / stage_k;
        while (wanted > 1 && k_stages / wanted < 3) wanted >>= 1;
        if (wanted < 8) wide = 128;
        if (wanted > 1) {
            splits = wanted;
            bn = wide;
            slices = 2;
        }
    }
    if (forced_splits != 0) splits = forced_splits;
    if (forced_block_n != 0) bn = forced_block_n;
    if (params.rhs_kn && bn < 64) {
        // [K, N] tiles are staged in boxes of 64 columns
        bn = 64;
        slices = slices > 4 ? 4 : slices;
    }
    {
        // two stages must fit the shared-memory limit of the call
        const int room = shared_limit(params) - 20 * 1024;
        while (slices > 1 && slices * (params.a_rows + bn) * 128 * 2 > room) slices >>= 1;
    }
    if (forced_slices != 0) slices = forced_slices;
    if (params.lhs_km) {
        // A [K, M] left operand (no caller on the decode path has one) runs the persistent kernel, whole 128-row tiles
        const int wide = (params.m > kBlockM && tiles(256) >= sms) ? 256 : (params.n > 64 ? 128 : 64);
        if (wide == 256) return launch_gemm<256, 1, true>(stream, params, lhs, rhs, lhs_row_stride, rhs_row_stride);
        if (wide == 128) return launch_gemm<128, 1, true>(stream, params, lhs, rhs, lhs_row_stride, rhs_row_stride);
        return launch_gemm<64, 1, true>(stream, params, lhs, rhs, lhs_row_stride, rhs_row_stride);
    }
    if (splits > 1) {
        if (params.m > kBlockM || (splits != 2 && splits != 4 && splits != 8)) return SINGE_ERR_UNSUPPORTED_CONFIGURATION;
#define SINGE_SPLITK_CASE(BN_, KPS_)                                                                             \
    if (bn == BN_ && slices == KPS_)                                                                             \
        return launch_gemm_splitk<BN_, KPS_>(stream, params, lhs, rhs, lhs_row_stride, rhs_row_stride, splits);
        SINGE_SPLITK_CASE(128, 2)
        SINGE_SPLITK_CASE(128, 1)
        SINGE_SPLITK_CASE(64, 1)
        SINGE_SPLITK_CASE(64, 2)
        SINGE_SPLITK_CASE(64, 4)
        SINGE_SPLITK_CASE(32, 8)
#undef SINGE_SPLITK_CASE
        return SINGE_ERR_UNSUPPORTED_CONFIGURATION;
    }
    // Many 256 x 256 tiles: the form with two M sub-tiles per CTA, which halves the A-and-B bytes an SM pulls per flop.
    if (bn == 256 && slices == 1 && params.m >= 2 * kBlockM &&
        ((params.m + 2 * kBlockM - 1) / (2 * kBlockM)) * ((params.n + 255) / 256) >= sms) {
        return launch_gemm<256, 1, false, 2>(stream, params, lhs, rhs, lhs_row_stride, rhs_row_stride);
    }
#define SINGE_GEMM_CASE(BN_, KPS_)                                                                    \
    if (bn == BN_ && slices == KPS_)                                                                  \
        return launch_gemm<BN_, KPS_>(stream, params, lhs, rhs, lhs_row_stride, rhs_row_stride);
    SINGE_GEMM_CASE(256, 1)
    SINGE_GEMM_CASE(128, 1)
    SINGE_GEMM_CASE(128, 2)
    SINGE_GEMM_CASE(64, 1)
    SINGE_GEMM_CASE(64, 2)
    SINGE_GEMM_CASE(64, 4)
    SINGE_GEMM_CASE(64, 8)
    SINGE_GEMM_CASE(32, 1)
    SINGE_GEMM_CASE(32, 2)
    SINGE_GEMM_CASE(32, 4)
    SINGE_GEMM_CASE(32, 8)
#undef SINGE_GEMM_CASE
    return SINGE_ERR_UNSUPPORTED_CONFIGURATION;
}

}  // namespace singe

extern "C" {

int singe_matmul_bf16_bf16(singe_stream_t stream, void *out, const void *lhs, const void *rhs, size_t rows,
                           size_t columns, size_t reduction, size_t lhs_row_stride, size_t rhs_row_stride,
                           size_t output_row_stride, int transpose_lhs, int transpose_rhs) {
    return singe::gemm_bf16(static_cast<cudaStream_t>(stream), out, false, lhs, rhs, rows, columns, reduction,
                            lhs_row_stride, rhs_row_stride, output_row_stride, transpose_lhs, transpose_rhs, false, 0u);
}

// out[M, N/2] = bf16(bf16(silu(g)) * u) with g = bf16(lhs . rhs[2j]^T), u = bf16(lhs . rhs[2j+1]^T): the gate and up
// projections of a gated MLP in one GEMM whose weight rows interleave gate and up, with the activation in the
// epilogue.  Same roundings as singe_matmul_bf16_bf16 followed by singe_silu_mul_bf16.
int singe_matmul_bf16_swiglu_bf16(singe_stream_t stream, void *out, const void *lhs, const void *rhs, size_t rows,
                                  size_t columns, size_t reduction, size_t lhs_row_stride, size_t rhs_row_stride,
                                  size_t output_row_stride) {
    return singe::gemm_bf16(static_cast<cudaStream_t>(stream), out, false, lhs, rhs, rows, columns, reduction,
                            lhs_row_stride, rhs_row_stride, output_row_stride, 0, 1, true, 0u);
}

int singe_matmul_bf16_f32(singe_stream_t stream, float *out, const void *lhs, const void *rhs, size_t rows,
                          size_t columns, size_t reduction, size_t lhs_row_stride, size_t rhs_row_stride,
                          size_t output_row_stride, int transpose_lhs, int transpose_rhs) {
    return singe::gemm_bf16(static_cast<cudaStream_t>(stream), out, true, lhs, rhs, rows, columns, reduction,
                            lhs_row_stride, rhs_row_stride, output_row_stride, transpose_lhs, transpose_rhs, false, 0u);
}

// Linear::forward with the weight matrix as a parameter of the layer: out[M, N] = x[M, K] . weight[N, K]^T.  `hints`
// may carry SINGE_HINT_STABLE_WEIGHTS; `gated` != 0 selects the SwiGLU epilogue of singe_matmul_bf16_swiglu_bf16.
int singe_linear_bf16(singe_stream_t stream, void *out, const void *x, const void *weight, size_t rows,
                      size_t columns, size_t reduction, size_t x_row_stride, size_t weight_row_stride,
                      size_t output_row_stride, int gated, unsigned hints) {
    return singe::gemm_bf16(static_cast<cudaStream_t>(stream), out, false, x, weight, rows, columns, reduction,
                            x_row_stride, weight_row_stride, output_row_stride, 0, 1, gated != 0, hints);
}

// Overrides the tile choice of the GEMM entry points for this process: block_n in {32, 64, 128, 256} and
// k_slices_per_stage in {1, 2, 4, 8}; 0 restores the shape-based choice.  Mirrors TuningChoice::Explicit
// (singe-kernel/src/cuda/matmul.rs:58-77).  Unsupported pairs make the next call return
// SINGE_ERR_UNSUPPORTED_CONFIGURATION.
int singe_matmul_set_tuning(int block_n, int k_slices_per_stage) {
    singe::g_tuning_block_n.store(block_n);
    singe::g_tuning_slices.store(k_slices_per_stage);
    return SINGE_OK;
}

// K splits (the cluster size) for one-M-tile problems: 0 = choose from the shape, 1 = never split, 2/4/8 = as given.
int singe_matmul_set_splits(int k_splits) {
    if (k_splits != 0 && k_splits != 1 && k_splits != 2 && k_splits != 4 && k_splits != 8) {
        return SINGE_ERR_INVALID_ARGUMENT;
    }
    singe::g_tuning_splits.store(k_splits);
    return SINGE_OK;
}

// Shared memory a GEMM CTA may take (KB, 0 = choose) and the amount of stable weights a CTA pulls into L2 ahead of
// its dependency wait (KB, negative = choose).
int singe_matmul_set_staging(int shared_kb, int prefetch_kb) {
    if (shared_kb < 0 || shared_kb > 227) return SINGE_ERR_INVALID_ARGUMENT;
    singe::g_tuning_shared_kb.store(shared_kb);
    singe::g_tuning_prefetch_kb.store(prefetch_kb < 0 ? -1 : prefetch_kb);
    return SINGE_OK;
}

}  // extern "C"
