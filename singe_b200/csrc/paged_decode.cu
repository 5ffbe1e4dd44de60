// Paged-KV flash-decode with split-K and a log-sum-exp combine, for bf16/f16 caches laid out
// [pages, 16, kv_heads, head_dim] with head_dim 64 or 128 and up to 8 query heads per KV head.
//
// Meaning: paged_kv_decode_attention (singe-kernel/src/cpu/attention.rs:1172-1246) with the split
// partials of the reference's split-K decode (singe-kernel/src/cuda/attention/mod.rs:2456-2509) and
// the combine of splitk_reduce_f32 (singe-kernel/src/cpu/attention.rs:2157-2193).
//
// Structure (HBM-bound; 2 * kv_heads * head_dim * 2 bytes per cached token must cross HBM once):
//   grid  = (kv_heads, max_splits, batch); one CTA owns up to `split_tokens` keys of one (sequence,
//           KV head) and ALL query heads of that KV head, so K and V are read once for the group.
//   warp 4 (producer): reads the block table 32 entries at a time and issues one TMA tile load per
//           (page, 64-wide half of the head) -- 16 rows x 128 bytes, SWIZZLE_128B -- for K and V into a
//           ring of eight stages, one mbarrier pair per stage; three CTAs share an SM so that one CTA's start-up
//           (length, block table, first TMA round trip) and final merge overlap the others' streaming.
//   warps 0-3 (consumers): page i belongs to warp i % 4.  S = Q K^T and O += P V run as m16n8k16
//           tensor-core tiles fed by ldmatrix from the swizzled stage (conflict-free), softmax runs in
//           f32 with warp-shuffle row reductions in the exp2 domain.
//   The four warps' (max, sum, O) states are merged through shared memory; the CTA writes either the
//   final row (the sequence fits one split) or a normalised partial + natural-log LSE.
//   decode_combine_kernel folds the partials of sequences that needed more than one split.
// One body, four kernels: the plain drop-in kernel; the decode-step kernel (reads ahead of the dependency wait,
// rotates its queries, may fold its row itself); the fused decode-step kernel (also rotates and stores the step's new
// K/V row); and the ragged kernel of the Tensor surface (FlashInfer page lists, optional score cap and sliding window).
// Every mbarrier wait is bounded; a wait that runs out sets status code 2 and the CTA leaves.
#include "common.cuh"

namespace singe {

namespace {

constexpr int kDecodeWarps = 4;
constexpr int kDecodeThreads = (kDecodeWarps + 1) * 32;
// A multiple of the consumer-warp count, so every use of a stage belongs to the same warp: a warp then
// waits for phase n+1 of a stage's barrier only after it consumed phase n, and a parity wait can never
// alias a phase that is two behind (TMA tiles may complete out of order).
constexpr int kDecodeStages = 8;
static_assert(kDecodeStages % kDecodeWarps == 0, "stage ownership must be fixed per consumer warp");
constexpr int kPageTokens = 16;
constexpr int kHalfBytes = kPageTokens * 128;  // one TMA box: 16 rows x 128 bytes

struct DecodeParams {
    void *out;            // [batch, heads, head_dim] in the cache dtype, or nullptr (partials only)
    float *attn_partial;  // [batch, heads, max_splits, head_dim]
    float *lse_partial;   // [batch, heads, max_splits]
    const void *query;    // [batch, heads, head_dim]
    const int32_t *lens;
    const uint32_t *table;
    int batch;
    int heads;
    int kv_heads;
    int group;
    int physical_blocks;
    int table_stride;
    int split_tokens;  // multiple of 16
    int max_splits;
    int partials_only;  // 1: every split slot is written, nothing goes to `out`
    float scale_log2;   // scale * log2(e)
    uint32_t *status;
};

// What only a decode step passes (the EXTRAS forms of the kernel).  It is a kernel argument of its own: the plain and
// ragged kernels do not carry it, and measurably so -- with these fields inside DecodeParams the plain kernel's
// registers were allotted differently and config 2 took 0.6 us longer.
struct StepExtras {
    int stable_paging;  // 1: lengths, block table and every cached row but each sequence's last key position are not
                        //    written by work still in flight (SINGE_HINT_STABLE_PAGING): they are read ahead of the
                        //    wait on the preceding kernels
    int early_release;  // 1: the grid fits the machine in one wave, so the next kernel may become resident at once
    int prefetch_pages; // with stable_paging: pages beyond the ring pulled into L2 ahead of the wait
    WarmRange warm;     // pulled into L2 beside the kernel's own work (classic form only)
    // Fused step form (FUSED): the kernel reads the step's un-rotated projections itself, rotates Q and the new K row,
    // writes the new K/V rows into the cache and attends over the cached keys plus the new one.
    const void *qkv;          // [batch, qkv_stride]: heads*D query | kv_heads*D key | kv_heads*D value projections
    long long qkv_stride;     // elements
    void *key_rows;           // the caches as plain pointers, for the one row this step adds per sequence and KV head
    void *value_rows;
    const void *write_pages;  // [batch] int32 / int64 (rope_index_width)
    const void *write_slots;
    uint32_t *tickets;  // [batch, kv_heads], zero between launches, or nullptr.  With tickets the split that finishes
                        // a row last folds the row's partials itself and no combine kernel follows (classic form)
    // Rotation of the queries inside the kernel (rope_cos == nullptr: the queries arrive rotated)
    const void *rope_cos;        // [capacity, head_dim / 2] in the cache dtype
    const void *rope_sin;
    const void *rope_positions;  // [batch] position of each sequence's query token, int32 or int64
    int rope_index_width;        // 4 or 8
    int rope_capacity;
    const void *query_gain;      // per-head RMSNorm before the rotation: gain [head_dim] or nullptr
    int query_norm;              // 1: normalise
    float query_norm_eps;
};

__device__ __forceinline__ float fast_tanh(float x) {
    float y;
    asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Rotates (and first, if asked, RMS-normalises) the query fragments a lane holds, in registers.  A lane of row
// `row` (a query head of the group) and quad q holds, for every 16-wide k step ks, the elements ks*16 + 2q, +1
// (qa[ks][0]) and ks*16 + 8 + 2q, +1 (qa[ks][1]): an element of the head's first half and its partner half a head
// further on sit in the same slot of steps ks and ks + KSTEPS/2, so the half-split rotation needs no exchange.
// Rounding follows the tensor-op chain of the separate kernel (singe_rotary_cache_write_bf16): every product and every
// sum is rounded to the cache dtype, so attention over queries rotated here equals attention over queries rotated there.
// Replaces the query stage of singe_rotary_paged_attention
// (singe/src/backend/cuda/kernel_plan/source/paged_attention.rs:881-977, QueryRotation).
template <typename T, int HD>
__device__ __forceinline__ void rotate_query_fragments(uint32_t (&qa)[HD / 16][2], const DecodeParams &p,
                                                       const StepExtras &x, int b, int row,
                                                       int quad, bool may_normalise = true) {
    constexpr int KSTEPS = HD / 16;
    constexpr int HALF_STEPS = KSTEPS / 2;
    long long position = x.rope_index_width == 8 ? static_cast<const long long *>(x.rope_positions)[b]
                                                 : static_cast<long long>(static_cast<const int *>(x.rope_positions)[b]);
    if (position < 0) position += x.rope_capacity;
    if (position < 0 || position >= x.rope_capacity) {
        report_status(p.status, kStatusIndexOutOfBounds);
        position = 0;
    }
    auto low = [](uint32_t word) {
        T value;
        *reinterpret_cast<uint16_t *>(&value) = static_cast<uint16_t>(word & 0xffffu);
        return to_float<T>(value);
    };
    auto high = [](uint32_t word) {
        T value;
        *reinterpret_cast<uint16_t *>(&value) = static_cast<uint16_t>(word >> 16);
        return to_float<T>(value);
    };
    auto rounded = [](float value) { return to_float<T>(from_float<T>(value)); };
    if (x.query_norm && may_normalise) {
        float squares = 0.0f;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
            for (int j = 0; j < 2; ++j) squares += low(qa[ks][j]) * low(qa[ks][j]) + high(qa[ks][j]) * high(qa[ks][j]);
        }
        squares += __shfl_xor_sync(0xffffffffu, squares, 1);
        squares += __shfl_xor_sync(0xffffffffu, squares, 2);
        const float scale = 1.0f / sqrtf(squares / static_cast<float>(HD) + x.query_norm_eps);
        const uint32_t *gain = static_cast<const uint32_t *>(x.query_gain);
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const uint32_t g = gain != nullptr ? gain[ks * 8 + j * 4 + quad] : 0u;
                const float g_low = gain != nullptr ? low(g) : 1.0f;
                const float g_high = gain != nullptr ? high(g) : 1.0f;
                qa[ks][j] = pack2<T>(low(qa[ks][j]) * scale * g_low, high(qa[ks][j]) * scale * g_high);
            }
        }
    }
    const uint32_t *cos_row = static_cast<const uint32_t *>(x.rope_cos) + position * (HD / 4);
    const uint32_t *sin_row = static_cast<const uint32_t *>(x.rope_sin) + position * (HD / 4);
    (void)row;
#pragma unroll
    for (int ks = 0; ks < HALF_STEPS; ++ks) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const uint32_t c = cos_row[ks * 8 + j * 4 + quad];   // pairs ks*16 + 8j + 2q, +1
            const uint32_t s = sin_row[ks * 8 + j * 4 + quad];
            const uint32_t first = qa[ks][j], second = qa[ks + HALF_STEPS][j];
            const float f0 = low(first), f1 = high(first), s0 = low(second), s1 = high(second);
            qa[ks][j] = pack2<T>(rounded(f0 * low(c)) - rounded(s0 * low(s)), rounded(f1 * high(c)) - rounded(s1 * high(s)));
            qa[ks + HALF_STEPS][j] =
                pack2<T>(rounded(s0 * low(c)) + rounded(f0 * low(s)), rounded(s1 * high(c)) + rounded(f1 * high(s)));
        }
    }
}

template <int HD>
constexpr int decode_stage_bytes() {
    return 2 * (HD / 64) * kHalfBytes;
}

template <int HD>
constexpr int decode_smem_bytes() {
    // stages (a warp's first stage doubles as its merge buffer: 8 rows x HD f32 fit one stage) + max/sum of
    // 4 warps x 8 rows + barriers + alignment slack
    return kDecodeStages * decode_stage_bytes<HD>() + 2 * kDecodeWarps * 8 * 4 + 2 * kDecodeStages * 8 + 1024;
}

// RAGGED selects the Tensor-surface form: the pages of sequence b start at ragged.first[b] in ragged.pages (32- or 64-bit
// entries), p.lens and ragged.control were written by the planning kernel of the same call (control[0] != 0: "not a plain
// decode batch, the general kernel runs instead"; control[1] = tokens per split), and finished rows also get their
// base-2 LSE in ragged.lse_out.  The classic form carries none of this code and never reads `ragged`.
// FUSED (classic form only) is the whole attention part of a decode step in one launch: lens[b] counts the keys
// INCLUDING the token this step adds; the CTA whose split holds that last position takes the token's K and V
// projections straight from the qkv buffer (they never come out of the cache in this step), rotates K, writes both
// rows into the cache for later steps and folds the new key into its online softmax as one more key; every CTA
// rotates its own queries.  No rotary / cache-write kernel precedes the launch, so nothing this kernel streams from
// the cache is written by the kernel before it, and with stable paging every page may be requested ahead of the wait.
// EXTRAS compiles in what only a decode step asks for (reads ahead of the dependency wait, the early release of a
// one-wave grid, L2 warming, the rotation of the queries, the in-kernel fold); without it the classic form is the plain
// drop-in kernel and carries none of their registers or branches (they cost it 2 us of 58 on the bench workload).
// OPTIONS (ragged form): tanh-capped scores and / or a sliding window's partly hidden first page.
template <typename T, int HD, bool RAGGED, bool FUSED = false, bool EXTRAS = false, bool OPTIONS = false>
__device__ __forceinline__ void paged_decode_body(const CUtensorMap &k_map, const CUtensorMap &v_map,
                                                  const DecodeParams &p, const StepExtras &x,
                                                  const RaggedDecode &ragged) {
    static_assert(!(RAGGED && FUSED), "the fused step form is a classic-form kernel");
    static_assert(!FUSED || EXTRAS, "the fused step form is a decode-step kernel");
    static_assert(!(RAGGED && EXTRAS) && !(OPTIONS && !RAGGED), "extras: classic form; options: ragged form");
    constexpr int NHALF = HD / 64;
    constexpr int KSTEPS = HD / 16;
    constexpr int NTILES = HD / 8;
    constexpr int STAGE = decode_stage_bytes<HD>();

    // The queries (and, in a decode step, the newest K/V rows) come from the kernel before.  No global write of this
    // kernel -- outputs, split partials -- may move above a thread's wait: an earlier kernel may still read them.
    const bool stable = EXTRAS && x.stable_paging != 0;
    if (EXTRAS && threadIdx.x < 32) {
        warm_l2(x.warm, (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x,
                gridDim.x * gridDim.y * gridDim.z, threadIdx.x);
    }
    if (!stable) grid_dependency_wait();
    if (EXTRAS && x.early_release) grid_launch_dependents();
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *aligned = smem_raw + (base - raw);
    static_assert(8 * HD * 4 <= STAGE, "a warp's merge rows must fit its first stage");
    float *merge_m = reinterpret_cast<float *>(aligned + kDecodeStages * STAGE);  // [4][8]
    float *merge_l = merge_m + kDecodeWarps * 8;                                   // [4][8]
    const uint32_t bar_full = base + kDecodeStages * STAGE + 2 * kDecodeWarps * 8 * 4;
    const uint32_t bar_empty = bar_full + kDecodeStages * 8;

    if (RAGGED && ragged.control[0] != 0) return;
    const int g = blockIdx.x;
    const int split = blockIdx.y;
    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const T *query = static_cast<const T *>(p.query);

    const int b = blockIdx.z;

    // The length and (classic form) this split's slice of the block-table row are read together, the table slice
    // before the length says how much of it is live: one dependent round trip fewer before the first K/V boxes.
    // The ragged form's page list hangs off two more device values and is read below.
    int len = p.lens[b];
    uint32_t early_page = 0u;
    if (!RAGGED && warp == kDecodeWarps) {
        const int at = split * (p.split_tokens / kPageTokens) + lane;
        if (lane < p.split_tokens / kPageTokens && at < p.table_stride) {
            early_page = p.table[static_cast<size_t>(b) * p.table_stride + at];
        }
    }
    // A grid covers the longest possible sequence, so under mixed lengths many CTAs of split >= 1 have nothing to
    // do (40 % on config 2): those leave as soon as the length is here.
    const int bound = RAGGED ? 0x7ffffff0 : p.table_stride * kPageTokens;
    len = len < 0 ? 0 : (len > bound ? bound : len);
    const int piece = RAGGED ? ragged.control[1] : p.split_tokens;
    const int hidden_keys = (OPTIONS && ragged.hidden != nullptr) ? ragged.hidden[b] : 0;
    if (split > 0 && static_cast<long long>(split) * piece >= len && !p.partials_only) return;
    uint32_t qa[KSTEPS][2];
    if (warp < kDecodeWarps && !stable) {
        const int row = lane >> 2;
        const int quad = lane & 3;
        const size_t head = static_cast<size_t>(b) * p.heads + g * p.group + row;
        const uint32_t *q32 =
            FUSED ? reinterpret_cast<const uint32_t *>(static_cast<const T *>(x.qkv) + static_cast<size_t>(b) * x.qkv_stride +
                                                       static_cast<size_t>(g * p.group + row) * HD)
                  : reinterpret_cast<const uint32_t *>(query + head * HD);
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
            qa[ks][0] = row < p.group ? q32[ks * 8 + quad] : 0u;
            qa[ks][1] = row < p.group ? q32[ks * 8 + 4 + quad] : 0u;
        }
        if (EXTRAS && x.rope_cos != nullptr) rotate_query_fragments<T, HD>(qa, p, x, b, row, quad);
    }
    // The barriers are set up while the query reads are in flight.
    if (tid == 0) {
        for (int s = 0; s < kDecodeStages; ++s) {
            mbar_init(bar_full + s * 8, 1);
            mbar_init(bar_empty + s * 8, 1);
        }
        mbar_init_fence();
    }

    const int n_splits = (len + piece - 1) / piece;

    if (split >= n_splits) {
        // Nothing to attend.  Split 0 of an empty sequence still owns the row: zeros, as the reference writes.
        if (stable) grid_dependency_wait();
        const bool owns_row = split == 0 && !p.partials_only;
        if (owns_row || p.partials_only) {
            for (int r = 0; r < p.group; ++r) {
                const size_t row = static_cast<size_t>(b) * p.heads + g * p.group + r;
                for (int d = tid; d < HD; d += kDecodeThreads) {
                    if (owns_row) {
                        static_cast<T *>(p.out)[row * HD + d] = from_float<T>(0.0f);
                        if (RAGGED && d == 0) ragged.lse_out[row] = -INFINITY;
                    } else {
                        p.attn_partial[(row * p.max_splits + split) * HD + d] = 0.0f;
                    }
                }
                if (p.partials_only && tid == 0) {
                    p.lse_partial[row * p.max_splits + split] = -INFINITY;
                }
            }
        }
        return;
    }

    const int tok_begin = split * piece;
    // FUSED: the sequence's last key is not in the cache yet; the split that holds its position adds it from registers
    const bool adds_new = FUSED && (len - 1) / piece == split;
    const int tok_end = min(adds_new ? len - 1 : len, tok_begin + piece);
    const int npages = tok_end > tok_begin ? (tok_end - tok_begin + kPageTokens - 1) / kPageTokens : 0;
    const int first_page = tok_begin / kPageTokens;
    __syncthreads();

    bool failed = false;

    if (warp == kDecodeWarps) {
        // ---------------- producer ----------------
        if (lane == 0) {
            prefetch_tensor_map(&k_map);
            prefetch_tensor_map(&v_map);
        }
        const uint32_t *table = p.table + static_cast<size_t>(b) * p.table_stride + first_page;
        const long long ragged_at = RAGGED ? ragged.first[b] + first_page : 0;
        // Stable paging: the ring's first pages are requested ahead of the wait, up to (not including) the page that
        // holds the sequence's last key position, which the preceding kernel may still be writing.  `ahead` pages
        // are in flight when the wait returns; the loop below starts behind them.
        int ahead = 0;
        if (stable) {
            // relative index of the page still in flux (FUSED: none, this kernel writes the new row itself)
            const int newest = FUSED ? npages : (len - 1) / kPageTokens - first_page;
            ahead = min(min(npages, kDecodeStages), newest);
            if (ahead < 0) ahead = 0;
            uint32_t page = 0u;
            if (lane < ahead) page = early_page;  // kDecodeStages <= 32: the early read covers them
            if (lane < ahead && page >= static_cast<uint32_t>(p.physical_blocks)) {
                report_status(p.status, kStatusIndexOutOfBounds);
                page = 0u;
            }
            for (int j = 0; j < ahead; ++j) {
                const uint32_t pg = __shfl_sync(0xffffffffu, page, j);
                const uint32_t full = bar_full + j * 8;
                const uint32_t stage = base + j * STAGE;
                if (lane == 0) mbar_expect_tx(full, STAGE);
                __syncwarp();
                if (lane < 2 * NHALF) {
                    const int hf = lane % NHALF;
                    const CUtensorMap *map = lane < NHALF ? &k_map : &v_map;
                    tma_load_4d(stage + lane * kHalfBytes, map, full, hf * 64, g, 0, static_cast<int32_t>(pg));
                }
            }
            const int far = min(min(npages, newest), ahead + x.prefetch_pages);
            for (int i = ahead + (lane >> 2); i < far; i += 8) {
                const uint32_t pg = table[i];
                if (pg < static_cast<uint32_t>(p.physical_blocks)) {
                    const int which = lane & 3;  // K low, K high, V low, V high (head_dim 64: K, V only)
                    if (which < 2 * NHALF) {
                        tma_prefetch_4d(which < NHALF ? &k_map : &v_map, (which % NHALF) * 64, g, 0,
                                        static_cast<int32_t>(pg));
                    }
                }
            }
            grid_dependency_wait();
        }
        for (int chunk = 0; chunk < npages && !failed; chunk += 32) {
            const int mine = chunk + lane;
            uint32_t page = 0u;
            if (!RAGGED && mine < npages) page = chunk == 0 ? early_page : table[mine];
            if (RAGGED && mine < npages) {
                if (ragged.index_width == 8) {
                    const long long wide = static_cast<const long long *>(ragged.pages)[ragged_at + mine];
                    page = (wide < 0 || wide > 0x7fffffffll) ? 0xffffffffu : static_cast<uint32_t>(wide);
                } else {
                    const int narrow = static_cast<const int *>(ragged.pages)[ragged_at + mine];
                    page = narrow < 0 ? 0xffffffffu : static_cast<uint32_t>(narrow);
                }
            }
            if (page >= static_cast<uint32_t>(p.physical_blocks)) {
                report_status(p.status, kStatusIndexOutOfBounds);
                page = 0u;
            }
            const int count = min(32, npages - chunk);
            for (int j = 0; j < count; ++j) {
                const uint32_t pg = __shfl_sync(0xffffffffu, page, j);
                const int i = chunk + j;
                if (i < ahead) continue;  // already in flight
                const int s = i % kDecodeStages;
                const int use = i / kDecodeStages;
                if (use > 0) {
                    // Lane 0 alone issues the loads, so it alone waits; the verdict is made warp-uniform.
                    int ok = 1;
                    if (lane == 0) {
                        ok = mbar_wait(bar_empty + s * 8, (use - 1) & 1) ? 1 : 0;
                    }
                    ok = __shfl_sync(0xffffffffu, ok, 0);
                    if (!ok) {
                        failed = true;
                        break;
                    }
                }
                // One box per lane: lanes 0 .. 2*NHALF-1 issue the K halves and the V halves of the page in a single
                // warp-wide instruction instead of one thread issuing them back to back.
                {
                    const uint32_t full = bar_full + s * 8;
                    const uint32_t stage = base + s * STAGE;
                    if (lane == 0) mbar_expect_tx(full, STAGE);
                    __syncwarp();
                    if (lane < 2 * NHALF) {
                        const int hf = lane % NHALF;
                        const CUtensorMap *map = lane < NHALF ? &k_map : &v_map;
                        tma_load_4d(stage + lane * kHalfBytes, map, full, hf * 64, g, 0, static_cast<int32_t>(pg));
                    }
                }
            }
        }
        if (failed && lane == 0) {
            report_status(p.status, kStatusWaitTimeout);
        }
        if (failed) linger_after_timeout();
    } else {
        // ---------------- consumers ----------------
        const int row = lane >> 2;   // query head within the group (rows >= group are zero padding)
        const int quad = lane & 3;
        if (stable) {
            grid_dependency_wait();
            const size_t head = static_cast<size_t>(b) * p.heads + g * p.group + row;
            const uint32_t *q32 =
                FUSED ? reinterpret_cast<const uint32_t *>(static_cast<const T *>(x.qkv) +
                                                           static_cast<size_t>(b) * x.qkv_stride +
                                                           static_cast<size_t>(g * p.group + row) * HD)
                      : reinterpret_cast<const uint32_t *>(query + head * HD);
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ++ks) {
                qa[ks][0] = row < p.group ? q32[ks * 8 + quad] : 0u;
                qa[ks][1] = row < p.group ? q32[ks * 8 + 4 + quad] : 0u;
            }
            if (x.rope_cos != nullptr) rotate_query_fragments<T, HD>(qa, p, x, b, row, quad);
        }
        float o[NTILES][4];
#pragma unroll
        for (int nt = 0; nt < NTILES; ++nt) {
            o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.0f;
        }
        float run_max = -INFINITY;
        float run_sum = 0.0f;

        // Per-lane constants of the ldmatrix addresses (see the layout note at the top of the file).
        const int mat = lane >> 3;
        const int k_tok = ((mat >> 1) << 3) + (lane & 7);
        const int k_sel = mat & 1;
        const int v_tok = ((mat & 1) << 3) + (lane & 7);
        const int v_sel = mat >> 1;

        for (int i = warp; i < npages; i += kDecodeWarps) {
            const int s = i % kDecodeStages;
            const int use = i / kDecodeStages;
            // Every lane observes the phase itself (it reads the TMA-written tile); the verdict is warp-uniform.
            if (!__all_sync(0xffffffffu, mbar_wait(bar_full + s * 8, use & 1) ? 1 : 0)) {
                failed = true;
                break;
            }
            const uint32_t stage_k = base + s * STAGE;
            const uint32_t stage_v = stage_k + NHALF * kHalfBytes;

            float s0[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            float s1[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ++ks) {
                const int hf = ks >> 2;
                const int c = ((ks & 3) << 1) + k_sel;
                uint32_t r0, r1, r2, r3;
                ldmatrix_x4(stage_k + hf * kHalfBytes + k_tok * 128 + ((c ^ (k_tok & 7)) << 4), r0, r1, r2, r3);
                mma_m16n8k16<T>(s0, qa[ks][0], 0u, qa[ks][1], 0u, r0, r1);
                mma_m16n8k16<T>(s1, qa[ks][0], 0u, qa[ks][1], 0u, r2, r3);
            }
            // Row `row` of this lane: keys t0, t0+1 (tile 0) and t0+8, t0+9 (tile 1).
            const int t0 = tok_begin + i * kPageTokens + quad * 2;
            if (OPTIONS && ragged.softcap > 0.0f) {
                // AttentionOptions::softcap: cap * tanh(scaled score / cap), then into the base-2 domain
                const float inward = p.scale_log2 * 0.6931471805599453f / ragged.softcap;
                const float outward = ragged.softcap * 1.4426950408889634f;
                s0[0] = outward * fast_tanh(s0[0] * inward) / p.scale_log2;
                s0[1] = outward * fast_tanh(s0[1] * inward) / p.scale_log2;
                s1[0] = outward * fast_tanh(s1[0] * inward) / p.scale_log2;
                s1[1] = outward * fast_tanh(s1[1] * inward) / p.scale_log2;
            }
            // visible keys: below the sequence's end and (sliding window) not among the hidden ones of its first page
            // (the lower bound exists only in the OPTIONS form: the other kernels keep their single compare per key)
            float x00 = (t0 < tok_end && (!OPTIONS || t0 >= hidden_keys)) ? s0[0] * p.scale_log2 : -INFINITY;
            float x01 = (t0 + 1 < tok_end && (!OPTIONS || t0 + 1 >= hidden_keys)) ? s0[1] * p.scale_log2 : -INFINITY;
            float x10 = (t0 + 8 < tok_end && (!OPTIONS || t0 + 8 >= hidden_keys)) ? s1[0] * p.scale_log2 : -INFINITY;
            float x11 = (t0 + 9 < tok_end && (!OPTIONS || t0 + 9 >= hidden_keys)) ? s1[1] * p.scale_log2 : -INFINITY;
            float tile_max = fmaxf(fmaxf(x00, x01), fmaxf(x10, x11));
            tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 1));
            tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 2));
            const float next_max = fmaxf(run_max, tile_max);
            const float correction = fast_exp2(run_max - next_max);
            run_max = next_max;
            x00 = fast_exp2(x00 - next_max);
            x01 = fast_exp2(x01 - next_max);
            x10 = fast_exp2(x10 - next_max);
            x11 = fast_exp2(x11 - next_max);
            run_sum = run_sum * correction + (x00 + x01) + (x10 + x11);
#pragma unroll
            for (int nt = 0; nt < NTILES; ++nt) {
                o[nt][0] *= correction;
                o[nt][1] *= correction;
            }
            const uint32_t pa0 = pack2<T>(x00, x01);
            const uint32_t pa2 = pack2<T>(x10, x11);
#pragma unroll
            for (int j = 0; j < NTILES / 2; ++j) {
                const int cg = 2 * j + v_sel;
                const int hf = cg >> 3;
                const int c = cg & 7;
                uint32_t r0, r1, r2, r3;
                ldmatrix_x4_trans(stage_v + hf * kHalfBytes + v_tok * 128 + ((c ^ (v_tok & 7)) << 4), r0, r1, r2, r3);
                mma_m16n8k16<T>(o[2 * j], pa0, 0u, pa2, 0u, r0, r1);
                mma_m16n8k16<T>(o[2 * j + 1], pa0, 0u, pa2, 0u, r2, r3);
            }
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(bar_empty + s * 8);
            }
        }
        if (failed && lane == 0) {
            report_status(p.status, kStatusWaitTimeout);
        }
        if (FUSED && adds_new && warp == 0) {
            // ---- the key and value this step adds: rotate K, put both rows into the cache, attend the new key ----
            const T *projections = static_cast<const T *>(x.qkv) + static_cast<size_t>(b) * x.qkv_stride;
            const uint32_t *k32 = reinterpret_cast<const uint32_t *>(projections + static_cast<size_t>(p.heads + g) * HD);
            const uint32_t *v32 =
                reinterpret_cast<const uint32_t *>(projections + static_cast<size_t>(p.heads + p.kv_heads + g) * HD);
            long long page = x.rope_index_width == 8 ? static_cast<const long long *>(x.write_pages)[b]
                                                     : static_cast<long long>(static_cast<const int *>(x.write_pages)[b]);
            long long slot = x.rope_index_width == 8 ? static_cast<const long long *>(x.write_slots)[b]
                                                     : static_cast<long long>(static_cast<const int *>(x.write_slots)[b]);
            if (page < 0) page += p.physical_blocks;
            if (slot < 0) slot += kPageTokens;
            const bool slot_ok = page >= 0 && page < p.physical_blocks && slot >= 0 && slot < kPageTokens;
            if (!slot_ok && lane == 0) report_status(p.status, kStatusIndexOutOfBounds);
            const size_t cache_row = ((static_cast<size_t>(slot_ok ? page : 0) * kPageTokens + (slot_ok ? slot : 0)) *
                                          p.kv_heads + g) * HD;
            uint32_t *k_out = reinterpret_cast<uint32_t *>(static_cast<T *>(x.key_rows) + cache_row);
            uint32_t *v_out = reinterpret_cast<uint32_t *>(static_cast<T *>(x.value_rows) + cache_row);
            uint32_t kf[KSTEPS][2];
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ++ks) {
                kf[ks][0] = k32[ks * 8 + quad];
                kf[ks][1] = k32[ks * 8 + 4 + quad];
            }
            rotate_query_fragments<T, HD>(kf, p, x, b, row, quad, false);   // the same rotation, without the query's norm
            auto low = [](uint32_t word) {
                T value;
                *reinterpret_cast<uint16_t *>(&value) = static_cast<uint16_t>(word & 0xffffu);
                return to_float<T>(value);
            };
            auto high = [](uint32_t word) {
                T value;
                *reinterpret_cast<uint16_t *>(&value) = static_cast<uint16_t>(word >> 16);
                return to_float<T>(value);
            };
            float dot = 0.0f;
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    dot = fmaf(low(qa[ks][j]), low(kf[ks][j]), dot);
                    dot = fmaf(high(qa[ks][j]), high(kf[ks][j]), dot);
                    if (row == 0 && slot_ok) k_out[ks * 8 + j * 4 + quad] = kf[ks][j];   // lanes 0-3 hold the whole row
                }
            }
            dot += __shfl_xor_sync(0xffffffffu, dot, 1);
            dot += __shfl_xor_sync(0xffffffffu, dot, 2);
            if (slot_ok && lane < HD / 2) v_out[lane] = v32[lane];   // HD / 2 words
            if (HD / 2 > 32 && slot_ok) v_out[lane + 32] = v32[lane + 32];
            const float x = dot * p.scale_log2;
            const float next_max = fmaxf(run_max, x);
            const float correction = fast_exp2(run_max - next_max);
            const float weight = fast_exp2(x - next_max);
            run_max = next_max;
            run_sum = run_sum * correction + (quad == 0 ? weight : 0.0f);   // the quad's sums are added up below
            // the weight takes the rounding the tensor-core path gives P
            T packed_weight = from_float<T>(weight);
            const float rounded_weight = to_float<T>(packed_weight);
#pragma unroll
            for (int nt = 0; nt < NTILES; ++nt) {
                const uint32_t value = v32[nt * 4 + quad];   // columns nt*8 + 2*quad, +1
                o[nt][0] = o[nt][0] * correction + rounded_weight * low(value);
                o[nt][1] = o[nt][1] * correction + rounded_weight * high(value);
            }
        }
        run_sum += __shfl_xor_sync(0xffffffffu, run_sum, 1);
        run_sum += __shfl_xor_sync(0xffffffffu, run_sum, 2);
        if (quad == 0) {
            merge_m[warp * 8 + row] = run_max;
            merge_l[warp * 8 + row] = run_sum;
        }
        // Stage `warp` is only ever filled for and read by this warp, and all of its tiles have been consumed.
        float *mine = reinterpret_cast<float *>(aligned + warp * STAGE) + row * HD;
#pragma unroll
        for (int nt = 0; nt < NTILES; ++nt) {
            *reinterpret_cast<float2 *>(mine + nt * 8 + quad * 2) = make_float2(o[nt][0], o[nt][1]);
        }
    }
    // Only now may the next kernel on the stream (the combine) take SM slots: its CTAs then arrive while this
    // launch drains instead of competing with its last wave.  CTAs that left early count as having said so.
    // (A one-wave grid has said so at its top.)
    grid_launch_dependents();
    __syncthreads();

    // ---------------- merge the four warps and write ----------------
    const bool direct = n_splits == 1 && !p.partials_only;
    for (int item = tid; item < p.group * HD; item += kDecodeThreads) {
        const int r = item / HD;
        const int d = item - r * HD;
        float top = -INFINITY;
#pragma unroll
        for (int w = 0; w < kDecodeWarps; ++w) {
            top = fmaxf(top, merge_m[w * 8 + r]);
        }
        float total = 0.0f;
        float value = 0.0f;
#pragma unroll
        for (int w = 0; w < kDecodeWarps; ++w) {
            const float m = merge_m[w * 8 + r];
            const float weight = m == -INFINITY ? 0.0f : fast_exp2(m - top);
            total += merge_l[w * 8 + r] * weight;
            value += reinterpret_cast<const float *>(aligned + w * STAGE)[r * HD + d] * weight;
        }
        const size_t head_row = static_cast<size_t>(b) * p.heads + g * p.group + r;
        const float result = value / total;
        if (direct) {
            static_cast<T *>(p.out)[head_row * HD + d] = from_float<T>(result);
            if (RAGGED && d == 0) ragged.lse_out[head_row] = top + log2f(total);
        } else {
            p.attn_partial[(head_row * p.max_splits + split) * HD + d] = result;
            if (d == 0) {
                // natural-log LSE of the scaled scores: (max2 + log2(sum)) * ln 2
                p.lse_partial[head_row * p.max_splits + split] = (top + log2f(total)) * 0.6931471805599453f;
            }
        }
    }
    // A warp whose wait ran out (status 2 is set, the row's result is void) keeps the CTA alive until copies that were
    // issued into its shared memory have landed.
    if (failed) linger_after_timeout();
    if (!EXTRAS || x.tickets == nullptr || direct || p.partials_only) return;
    // ---------------- the last split of the row to finish folds the row ----------------
    // Every split of a (sequence, KV head) row takes a ticket once its partials are written and visible; the one
    // that draws the last ticket reads all of them back (through L2: they were written by other SMs) and writes the
    // row with the arithmetic of decode_combine_kernel, then puts the counter back to zero for the next launch.
    // It saves a launch, but measured slower than the separate combine kernel on B200 even for one-wave grids (every
    // CTA pays the device-wide fence and the atomic on its way out): the caller decides by passing tickets or not.
    __shared__ int shared_last;
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        uint32_t *ticket = x.tickets + static_cast<size_t>(b) * p.kv_heads + g;
        const uint32_t drawn = atomicAdd(ticket, 1u);
        shared_last = drawn == static_cast<uint32_t>(n_splits - 1) ? 1 : 0;
        if (shared_last) *ticket = 0u;  // every other split of the row has drawn already
    }
    __syncthreads();
    if (shared_last == 0) return;
    __threadfence();
    for (int item = tid; item < p.group * HD; item += kDecodeThreads) {
        const int r = item / HD;
        const int d = item - r * HD;
        const size_t head_row = static_cast<size_t>(b) * p.heads + g * p.group + r;
        const float *lse = p.lse_partial + head_row * p.max_splits;
        float top = -INFINITY;
        for (int s2 = 0; s2 < n_splits; ++s2) top = fmaxf(top, __ldcg(lse + s2));
        float denom = 0.0f;
        for (int s2 = 0; s2 < n_splits; ++s2) denom += expf(__ldcg(lse + s2) - top);
        float sum = 0.0f;
        for (int s2 = 0; s2 < n_splits; ++s2) {
            sum = fmaf(expf(__ldcg(lse + s2) - top), __ldcg(p.attn_partial + (head_row * p.max_splits + s2) * HD + d), sum);
        }
        static_cast<T *>(p.out)[head_row * HD + d] = from_float<T>(sum / denom);
    }
}

template <typename T, int HD>
__global__ void __launch_bounds__(kDecodeThreads, 3)
    paged_decode_kernel(const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map,
                        const DecodeParams p) {
    RaggedDecode none;  // never read by the classic form
    none.pages = nullptr;
    none.first = nullptr;
    none.control = nullptr;
    none.index_width = 4;
    none.lse_out = nullptr;
    none.softcap = 0.0f;
    none.hidden = nullptr;
    StepExtras unused = {};  // never read without EXTRAS
    paged_decode_body<T, HD, false>(k_map, v_map, p, unused, none);
}

// The classic form with the decode step's extras (see paged_decode_body).
template <typename T, int HD>
__global__ void __launch_bounds__(kDecodeThreads, 3)
    paged_decode_step_kernel(const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map,
                             const DecodeParams p, const StepExtras x) {
    RaggedDecode none;  // never read by the classic form
    none.pages = nullptr;
    none.first = nullptr;
    none.control = nullptr;
    none.index_width = 4;
    none.lse_out = nullptr;
    none.softcap = 0.0f;
    none.hidden = nullptr;
    paged_decode_body<T, HD, false, false, true>(k_map, v_map, p, x, none);
}

template <typename T, int HD>
__global__ void __launch_bounds__(kDecodeThreads, 3)
    paged_decode_fused_kernel(const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map,
                              const DecodeParams p, const StepExtras x) {
    RaggedDecode none;  // never read by this form
    none.pages = nullptr;
    none.first = nullptr;
    none.control = nullptr;
    none.index_width = 4;
    none.lse_out = nullptr;
    none.softcap = 0.0f;
    none.hidden = nullptr;
    paged_decode_body<T, HD, false, true, true>(k_map, v_map, p, x, none);
}

template <typename T, int HD, bool OPTIONS>
__global__ void __launch_bounds__(kDecodeThreads, 3)
    paged_decode_ragged_kernel(const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map,
                               const DecodeParams p, const RaggedDecode ragged) {
    StepExtras unused = {};  // never read without EXTRAS
    paged_decode_body<T, HD, true, false, false, OPTIONS>(k_map, v_map, p, unused, ragged);
}

// Folds the split partials of every (sequence, head) row that needed more than one split.
// Follows splitk_reduce_f32 (singe-kernel/src/cpu/attention.rs:2157-2193): out = sum_s exp(lse_s - M) attn_s / sum_s exp(lse_s - M).
// RAGGED: the Tensor-surface form (split size and verdict from the planning kernel, base-2 LSE written too); the
// classic form is a separate instantiation so that it carries none of that code (it measured 2 % slower with it).
template <typename T, bool RAGGED>
__global__ void decode_combine_kernel(T *out, const float *attn_partial, const float *lse_partial, const int32_t *lens,
                                      int heads, int head_dim, int split_tokens, int max_splits, int bound,
                                      const int *ragged_control, float *lse_out) {
    grid_launch_dependents();
    grid_dependency_wait();
    if (RAGGED) {
        if (ragged_control[0] != 0) return;
        split_tokens = ragged_control[1];
        bound = 0x7ffffff0;
    }
    const int b = blockIdx.y;
    const int head = blockIdx.x;
    int len = lens[b];
    len = len < 0 ? 0 : (len > bound ? bound : len);
    const int n = (len + split_tokens - 1) / split_tokens;
    if (n <= 1) {
        return;  // the decode kernel already wrote the row
    }
    const size_t row = static_cast<size_t>(b) * heads + head;
    const float *lse = lse_partial + row * max_splits;
    float top = -INFINITY;
    for (int s = 0; s < n; ++s) top = fmaxf(top, lse[s]);
    float denom = 0.0f;
    for (int s = 0; s < n; ++s) denom += expf(lse[s] - top);
    for (int d = threadIdx.x; d < head_dim; d += blockDim.x) {
        float sum = 0.0f;
        for (int s = 0; s < n; ++s) {
            sum = fmaf(expf(lse[s] - top), attn_partial[(row * max_splits + s) * head_dim + d], sum);
        }
        out[row * head_dim + d] = from_float<T>(sum / denom);
    }
    if (RAGGED && threadIdx.x == 0) {
        lse_out[row] = (top + logf(denom)) * 1.4426950408889634f;  // natural log -> base 2
    }
}

template <typename T, int HD, bool RAGGED>
int launch_decode(cudaStream_t stream, const DecodeParams &params, const StepExtras &extras, const RaggedDecode &shape,
                  const void *key_cache,
                  const void *value_cache, size_t batch) {
    static int configured[kMaxDevices] = {0};  // one table per instantiation, one entry per device
    constexpr int smem = decode_smem_bytes<HD>();
    const bool fused = !RAGGED && extras.qkv != nullptr;
    const bool capped = RAGGED && (shape.softcap > 0.0f || shape.hidden != nullptr);
    // the plain drop-in call takes the kernel without the decode step's extras
    const bool step = !RAGGED && !fused &&
                        (extras.stable_paging != 0 || extras.early_release != 0 || extras.warm.bytes != 0 ||
                         extras.rope_cos != nullptr || extras.tickets != nullptr);
    if (RAGGED) {
        static int configured_capped[kMaxDevices] = {0};
        if (capped) {
            SINGE_CUDA_TRY(ensure_dynamic_shared(paged_decode_ragged_kernel<T, HD, true>, smem, configured_capped));
        } else {
            SINGE_CUDA_TRY(ensure_dynamic_shared(paged_decode_ragged_kernel<T, HD, false>, smem, configured));
        }
    } else if (fused) {
        static int configured_fused[kMaxDevices] = {0};
        SINGE_CUDA_TRY(ensure_dynamic_shared(paged_decode_fused_kernel<T, HD>, smem, configured_fused));
    } else if (step) {
        static int configured_step[kMaxDevices] = {0};
        SINGE_CUDA_TRY(ensure_dynamic_shared(paged_decode_step_kernel<T, HD>, smem, configured_step));
    } else {
        SINGE_CUDA_TRY(ensure_dynamic_shared(paged_decode_kernel<T, HD>, smem, configured));
    }
    CUtensorMap k_map, v_map;
    const uint64_t dims[4] = {static_cast<uint64_t>(HD), static_cast<uint64_t>(params.kv_heads), kPageTokens,
                              static_cast<uint64_t>(params.physical_blocks)};
    const uint64_t strides[3] = {static_cast<uint64_t>(HD) * sizeof(T),
                                 static_cast<uint64_t>(HD) * sizeof(T) * params.kv_heads,
                                 static_cast<uint64_t>(HD) * sizeof(T) * params.kv_heads * kPageTokens};
    const uint32_t box[4] = {64, 1, kPageTokens, 1};
    SINGE_TRY(encode_tensor_map(&k_map, TensorMapType<T>::value, 4, key_cache, dims, strides, box,
                                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B));
    SINGE_TRY(encode_tensor_map(&v_map, TensorMapType<T>::value, 4, value_cache, dims, strides, box,
                                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B));
    // KV heads vary fastest: the CTAs that read the interleaved rows of the same cache pages start together.
    dim3 grid(static_cast<unsigned>(params.kv_heads), static_cast<unsigned>(params.max_splits),
              static_cast<unsigned>(batch));
    if (RAGGED && capped) {
        SINGE_CUDA_TRY(launch_dependent(paged_decode_ragged_kernel<T, HD, true>, grid, dim3(kDecodeThreads), smem,
                                        stream, kLaunchDecode, 1, k_map, v_map, params, shape));
    } else if (RAGGED) {
        SINGE_CUDA_TRY(launch_dependent(paged_decode_ragged_kernel<T, HD, false>, grid, dim3(kDecodeThreads), smem,
                                        stream, kLaunchDecode, 1, k_map, v_map, params, shape));
    } else if (fused) {
        SINGE_CUDA_TRY(launch_dependent(paged_decode_fused_kernel<T, HD>, grid, dim3(kDecodeThreads), smem, stream,
                                        kLaunchDecode, 1, k_map, v_map, params, extras));
    } else if (step) {
        SINGE_CUDA_TRY(launch_dependent(paged_decode_step_kernel<T, HD>, grid, dim3(kDecodeThreads), smem, stream,
                                        kLaunchDecode, 1, k_map, v_map, params, extras));
    } else {
        SINGE_CUDA_TRY(launch_dependent(paged_decode_kernel<T, HD>, grid, dim3(kDecodeThreads), smem, stream,
                                        kLaunchDecode, 1, k_map, v_map, params));
    }
    return launch_status();
}

}  // namespace

// Pages beyond its ring that a CTA pulls into L2 ahead of its dependency wait under SINGE_HINT_STABLE_PAGING.
int g_decode_prefetch_pages = 0;

// True when the tensor-core flash-decode kernel takes this shape.
bool paged_decode_fast_path(size_t heads, size_t kv_heads, size_t head_dim, size_t block_size, const void *key_cache,
                            const void *value_cache, const void *query) {
    const size_t group = heads / kv_heads;
    const bool aligned = ((reinterpret_cast<uintptr_t>(key_cache) | reinterpret_cast<uintptr_t>(value_cache)) & 15u) == 0 &&
                         (reinterpret_cast<uintptr_t>(query) & 3u) == 0;
    return (head_dim == 64 || head_dim == 128) && block_size == kPageTokens && group >= 1 && group <= 8 && aligned;
}

size_t paged_decode_split_tokens(size_t key_len_bound, size_t max_splits, size_t block_size) {
    if (max_splits == 0) max_splits = 1;
    if (block_size == 0) block_size = 1;
    size_t per = (key_len_bound + max_splits - 1) / max_splits;
    per = (per + block_size - 1) / block_size * block_size;
    return per == 0 ? block_size : per;
}

// Launches the flash-decode kernel and, unless `partials_only`, the combine.  The caller has validated the
// configuration and chosen the fast path.  T is selected by `element` (0 = bf16, 1 = f16).
int paged_decode_splitk(cudaStream_t stream, int element, void *out, float *attn_scratch, float *lse_scratch,
                        const void *query, const void *key_cache, const void *value_cache,
                        const int32_t *actual_seq_lens, const uint32_t *block_table, size_t batch, size_t heads,
                        size_t kv_heads, size_t head_dim, size_t physical_blocks, size_t block_table_batch_stride,
                        size_t max_splits, float scale, bool partials_only, uint32_t *status,
                        const RaggedDecode *ragged, unsigned hints, const QueryRotation *rotation, uint32_t *tickets,
                        const FusedStep *fused) {
    DecodeParams params;
    StepExtras extras;
    extras.tickets = ragged == nullptr && !partials_only ? tickets : nullptr;
    extras.qkv = nullptr;
    extras.qkv_stride = 0;
    extras.key_rows = extras.value_rows = nullptr;
    extras.write_pages = extras.write_slots = nullptr;
    if (fused != nullptr && ragged == nullptr && rotation != nullptr && element == 0 && !partials_only) {
        extras.qkv = fused->qkv;
        extras.qkv_stride = fused->qkv_stride;
        extras.key_rows = const_cast<void *>(key_cache);
        extras.value_rows = const_cast<void *>(value_cache);
        extras.write_pages = fused->write_pages;
        extras.write_slots = fused->write_slots;
    }
    extras.rope_cos = extras.rope_sin = extras.rope_positions = extras.query_gain = nullptr;
    extras.rope_index_width = 8;
    extras.rope_capacity = 0;
    extras.query_norm = 0;
    extras.query_norm_eps = 0.0f;
    if (rotation != nullptr && ragged == nullptr) {
        extras.rope_cos = rotation->cos;
        extras.rope_sin = rotation->sin;
        extras.rope_positions = rotation->positions;
        extras.rope_index_width = rotation->index_width;
        extras.rope_capacity = rotation->capacity;
        extras.query_gain = rotation->gain;
        extras.query_norm = rotation->normalise;
        extras.query_norm_eps = rotation->eps;
    }
    RaggedDecode none;
    none.pages = nullptr;
    none.first = nullptr;
    none.control = nullptr;
    none.index_width = 4;
    none.lse_out = nullptr;
    none.softcap = 0.0f;
    none.hidden = nullptr;
    const RaggedDecode &shape = ragged != nullptr ? *ragged : none;
    params.out = out;
    params.attn_partial = attn_scratch;
    params.lse_partial = lse_scratch;
    params.query = query;
    params.lens = actual_seq_lens;
    params.table = block_table;
    params.batch = static_cast<int>(batch);
    params.heads = static_cast<int>(heads);
    params.kv_heads = static_cast<int>(kv_heads);
    params.group = static_cast<int>(heads / kv_heads);
    params.physical_blocks = static_cast<int>(physical_blocks);
    params.table_stride = static_cast<int>(block_table_batch_stride);
    const size_t bound = block_table_batch_stride * kPageTokens;
    params.split_tokens = static_cast<int>(paged_decode_split_tokens(bound, max_splits, kPageTokens));
    params.max_splits = static_cast<int>(max_splits);
    params.partials_only = partials_only ? 1 : 0;
    extras.stable_paging = (ragged == nullptr && (hints & SINGE_HINT_STABLE_PAGING) != 0) ? 1 : 0;
    // One wave: three CTAs are resident per SM.
    extras.early_release = kv_heads * max_splits * batch <= static_cast<size_t>(3 * device_sm_count()) ? 1 : 0;
    extras.prefetch_pages = g_decode_prefetch_pages;
    extras.warm = ragged == nullptr ? take_pending_warm() : WarmRange{nullptr, 0};
    params.scale_log2 = scale * 1.4426950408889634f;
    params.status = status;
    if (batch > 65535 || max_splits > 65535 || kv_heads > 0x7fffffffull) {
        return SINGE_ERR_UNSUPPORTED_CONFIGURATION;
    }
    int result;
    if (element == 0) {
        if (ragged != nullptr) {
            result = head_dim == 128
                         ? launch_decode<__nv_bfloat16, 128, true>(stream, params, extras, shape, key_cache, value_cache, batch)
                         : launch_decode<__nv_bfloat16, 64, true>(stream, params, extras, shape, key_cache, value_cache, batch);
        } else {
            result = head_dim == 128
                         ? launch_decode<__nv_bfloat16, 128, false>(stream, params, extras, shape, key_cache, value_cache, batch)
                         : launch_decode<__nv_bfloat16, 64, false>(stream, params, extras, shape, key_cache, value_cache, batch);
        }
    } else {
        if (ragged != nullptr) {
            result = head_dim == 128 ? launch_decode<__half, 128, true>(stream, params, extras, shape, key_cache, value_cache, batch)
                                     : launch_decode<__half, 64, true>(stream, params, extras, shape, key_cache, value_cache, batch);
        } else {
            result = head_dim == 128 ? launch_decode<__half, 128, false>(stream, params, extras, shape, key_cache, value_cache, batch)
                                     : launch_decode<__half, 64, false>(stream, params, extras, shape, key_cache, value_cache, batch);
        }
    }
    SINGE_TRY(result);
    if (!partials_only && max_splits > 1 && extras.tickets == nullptr) {
        dim3 grid(static_cast<unsigned>(heads), static_cast<unsigned>(batch));
        const int threads = head_dim >= 128 ? 128 : 64;
#define SINGE_COMBINE(T, RAGGED_)                                                                                  \
    SINGE_CUDA_TRY(launch_dependent(decode_combine_kernel<T, RAGGED_>, grid, dim3(threads), 0, stream, kLaunchCombine, \
                                    1, static_cast<T *>(out), attn_scratch, lse_scratch, actual_seq_lens,            \
                                    params.heads, static_cast<int>(head_dim), params.split_tokens,                   \
                                    params.max_splits, static_cast<int>(bound), shape.control, shape.lse_out))
        if (element == 0) {
            if (ragged != nullptr) {
                SINGE_COMBINE(__nv_bfloat16, true);
            } else {
                SINGE_COMBINE(__nv_bfloat16, false);
            }
        } else {
            if (ragged != nullptr) {
                SINGE_COMBINE(__half, true);
            } else {
                SINGE_COMBINE(__half, false);
            }
        }
#undef SINGE_COMBINE
        return launch_status();
    }
    return SINGE_OK;
}

}  // namespace singe

// -------------------------------------------------------------------------------------------------
// Decode with library-resident scratch: an entry point that never allocates.
//
// Some hosts cannot let this library call cudaMalloc.  A runtime that follows the reference's rule that
// operators never allocate hands every byte of device memory to its own pool at start-up, so a library-side
// cudaMalloc has nothing left to take (or fragments the pool); a latency-critical decode loop cannot afford
// the device-wide synchronisation cudaMalloc and cudaFree imply.  The reference's paged-decode signature has
// no scratch parameter either, so such a caller has nowhere to pass split-K scratch.  For them the split
// partials live in the fixed array below, which every GPU that loads the library carries until the process
// exits.
// -------------------------------------------------------------------------------------------------
namespace singe {
namespace {

// 2 Mi floats = 8 MiB: partials [batch, heads, splits, head_dim] followed by their LSEs [batch, heads, splits].
constexpr size_t kStaticScratchFloats = size_t(2) << 20;
static __device__ __align__(256) float g_decode_static_scratch[kStaticScratchFloats];

// In host code the array's name is only a handle for the runtime, not a device address; the address the
// kernels need is looked up once per device, with that device current.
int static_scratch_address(float **address) {
    static float *resolved[kMaxDevices] = {nullptr};
    int device = 0;
    SINGE_CUDA_TRY(cudaGetDevice(&device));
    if (device < 0 || device >= kMaxDevices) {
        return SINGE_ERR_UNSUPPORTED_CONFIGURATION;
    }
    if (resolved[device] == nullptr) {
        void *pointer = nullptr;
        SINGE_CUDA_TRY(cudaGetSymbolAddress(&pointer, g_decode_static_scratch));
        if (pointer == nullptr) {
            return SINGE_ERR_NULL_POINTER;
        }
        resolved[device] = static_cast<float *>(pointer);
    }
    *address = resolved[device];
    return SINGE_OK;
}

}  // namespace
}  // namespace singe

extern "C" {

size_t singe_paged_kv_decode_attention_static_scratch_floats(void) { return singe::kStaticScratchFloats; }

int singe_paged_kv_decode_attention_static_bf16(singe_stream_t stream, void *out, const void *query,
                                                const void *key_cache, const void *value_cache,
                                                const int32_t *actual_seq_lens, const uint32_t *block_table,
                                                size_t batch, size_t heads, size_t kv_heads, size_t head_dim,
                                                size_t block_size, size_t physical_blocks,
                                                size_t block_table_batch_stride, float scale) {
    using namespace singe;
    if (batch == 0 || heads == 0 || kv_heads == 0 || head_dim == 0 || block_size == 0 || physical_blocks == 0 ||
        block_table_batch_stride == 0 || heads % kv_heads != 0 || !(scale - scale == 0.0f)) {
        return SINGE_ERR_INVALID_LENGTH;
    }
    if (!fits_i32(batch) || !fits_i32(heads) || !fits_i32(kv_heads) || !fits_i32(head_dim) || !fits_i32(block_size) ||
        !fits_i32(physical_blocks) || !fits_i32(block_table_batch_stride)) {
        return SINGE_ERR_LENGTH_EXCEEDS_I32;
    }
    if (out == nullptr || query == nullptr || key_cache == nullptr || value_cache == nullptr ||
        actual_seq_lens == nullptr || block_table == nullptr) {
        return SINGE_ERR_NULL_POINTER;
    }
    if (!paged_decode_fast_path(heads, kv_heads, head_dim, block_size, key_cache, value_cache, query)) {
        return SINGE_ERR_UNSUPPORTED_CONFIGURATION;
    }
    // One split needs batch * heads * (head_dim + 1) floats; a problem that does not fit even unsplit is refused.
    size_t per_split = 0;
    if (__builtin_mul_overflow(batch, heads, &per_split) || __builtin_mul_overflow(per_split, head_dim + 1, &per_split)) {
        return SINGE_ERR_SIZE_OVERFLOW;
    }
    if (per_split > kStaticScratchFloats) {
        return SINGE_ERR_STATIC_SCRATCH_EXCEEDED;
    }
    // ~512 keys per split, capped by what the fixed array holds.
    size_t splits = (block_table_batch_stride * block_size + 511) / 512;
    const size_t room = kStaticScratchFloats / per_split;
    if (splits > room) splits = room;
    if (splits < 1) splits = 1;
    float *scratch = nullptr;
    SINGE_TRY(static_scratch_address(&scratch));
    const size_t rows = batch * heads * splits;
    // Every partial the combine reads is written by the decode kernel of the same call, so nothing in the
    // array has to start at zero; what an earlier call left behind is never read.
    return paged_decode_splitk(static_cast<cudaStream_t>(stream), 0, out, scratch, scratch + rows * head_dim, query,
                               key_cache, value_cache, actual_seq_lens, block_table, batch, heads, kv_heads, head_dim,
                               physical_blocks, block_table_batch_stride, splits, scale, false, device_error_word(), nullptr,
                               0u, nullptr, nullptr, nullptr);
}

}  // extern "C"
