// Packed variable-length flash-attention prefill on the tcgen05 tensor core (bf16 or f16, head_dim 128, GQA).
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
//   warps 0-3  softmax of tile A, one thread per query row (= tensor-memory lane); warps 4-7 the same for tile B.
//              The softmax is the bottleneck next to the MMAs (instruction issue and the 16 exp2 per clock of the
//              special-function unit), so its steady state is a single pass with as few instructions per score as
//              possible: scores come out of tensor memory 32 columns at a time (the next load in flight while the
//              current chunk is processed), p = exp2(s * scale - base) as packed f32x2 arithmetic, the row sum,
//              the bf16 pack, and P goes back over S with tcgen05.st.  No row maximum is taken: `base` only has to
//              keep the numbers in range, the result does not depend on it (out = O / sum, LSE = base +
//              log2(sum)).  The first key tile takes the exact row maximum as base (a two-pass tile); afterwards
//              the row is re-based by an exact power of two whenever its running sum passes 2^16 (O in tensor
//              memory and the sum are scaled, at the start of the next tile, when the previous P V has retired).
//              A row whose scores jump by more than ~2^64 from one key tile to the next would overflow this
//              scheme.  Such a row gets a NaN as its LSE and raises a sticky per-device flag; the second launch of
//              the same kernel in SAFE mode, where every tile takes its exact row maximum first, leaves at once
//              while the flag has never been raised, and otherwise finds the marked items among its share and
//              recomputes exactly those.
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
#include <type_traits>

#include "common.cuh"
#include "tcgen05.cuh"

namespace singe {

namespace {

constexpr int kPrefillThreads = 320;
constexpr int kTile = 128;           // rows of one query tile, and keys per key tile
constexpr int kPair = 2 * kTile;     // query rows per CTA
constexpr int kChunk = 32;           // score columns taken out of tensor memory at a time
constexpr int kHalfTileBytes = kTile * 128;       // one TMA box: 128 rows x 128 bytes
constexpr int kTileBytes = 2 * kHalfTileBytes;    // 32 KB
constexpr int kPageTokens = 16;                   // paged form: tokens per cache page
constexpr int kPageBytes = kPageTokens * 128;     // one page box: 16 rows x 128 bytes
constexpr int kMaxRankTiles = 1024;               // heaviest-first dispatch: sequences up to 256 Ki tokens
constexpr float kRescaleThreshold = 8.0f;         // two-pass tiles: re-base when the max grew by 2^8 (log2 units)
constexpr float kRebaseLimit = 65536.0f;          // single-pass tiles: re-base a row when its sum passes 2^16
constexpr float kOverflowLimit = 1.8446744e19f;   // 2^64: beyond this the CTA is redone in SAFE mode
constexpr int kRedoCapacity = 2048;               // marked items one CTA lists; past that it redoes its whole share

// Raised (never lowered) by the first launch when a row leaves the single-pass range.  While it is zero the second
// launch has nothing to look for; once it is set every later call pays the scan of the LSE marks.
__device__ unsigned g_out_of_range_seen = 0;

struct PrefillParams {
    void *out;
    float *lse;
    const int32_t *lens_q;    // nullptr: the dense form, every sequence has uniform_q queries and uniform_kv keys,
    const int32_t *lens_kv;   //          sequence b starts at row b * uniform_q (queries) / b * uniform_kv (keys)
    const int32_t *offsets;
    int uniform_q;
    int uniform_kv;
    int lse_rows;   // 0: LSE is [total_q, heads] (packed forms); > 0: [batch, heads, lse_rows] (fmha_prefill_lse)
    int exact;      // 1: the exact-maximum launch walks every item (16-bit floats whose range the single-pass
                    // softmax would leave); 0: it only redoes what the first launch marked
    int batch;
    int heads;
    int kv_heads;
    int total_q;
    int total_kv;
    // paged form: keys and values live in a cache [pages, 16, kv_heads, 128] behind a block table [batch, table_stride]
    const uint32_t *block_table;
    int table_stride;
    int cache_pages;
    int causal;     // 0: none; 1: key index > query index hidden (sequence-local, the kernel surface's mask);
                    // 2: the queries are the sequence's last tokens (query i sits at position len_kv - len_q + i)
    float scale_log2;
    uint32_t *error;
};

// Lengths and first rows of sequence b.  DENSE is a template argument of the kernel: as run-time branches these four
// cost the packed form 2.5 % (every warp of a CTA decodes every work item).
template <bool DENSE>
__device__ __forceinline__ int seq_len_q(const PrefillParams &p, int b) { return DENSE ? p.uniform_q : p.lens_q[b]; }
template <bool DENSE>
__device__ __forceinline__ int seq_len_kv(const PrefillParams &p, int b) { return DENSE ? p.uniform_kv : p.lens_kv[b]; }
template <bool DENSE>
__device__ __forceinline__ int seq_offset_q(const PrefillParams &p, int b) { return DENSE ? b * p.uniform_q : p.offsets[b]; }
template <bool DENSE>
__device__ __forceinline__ int seq_offset_kv(const PrefillParams &p, int b) { return DENSE ? b * p.uniform_kv : p.offsets[b]; }

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

// Folds the 32 raw scores of one chunk into four running maxima (independent chains).  MASKED handles tiles where
// some keys are hidden (the diagonal tile and a sequence's last tile) and a negative scale; `limit` counts the
// visible columns from the chunk's first.
template <bool MASKED>
__device__ __forceinline__ void chunk_max(const uint32_t (&sc)[kChunk], int limit, float sign, float (&m)[4]) {
    if (MASKED) {
#pragma unroll
        for (int i = 0; i < kChunk; i += 4) {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                if (i + u < limit) m[u] = fmaxf(m[u], __uint_as_float(sc[i + u]) * sign);
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < kChunk; i += 8) {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                m[u] = max3(m[u], __uint_as_float(sc[i + 2 * u]), __uint_as_float(sc[i + 2 * u + 1]));
            }
        }
    }
}

// P = exp2(s * scale + bias) for one chunk of 32 scores: the bf16 pairs go back to tensor memory (16 packed
// columns at `tmem_p`), the unrounded values are added to two running f32x2 sums.  Scores are handled as f32x2
// pairs.  (Evaluating part of the exponentials as a polynomial on the FMA pipe was measured slower at every ratio:
// with one softmax warp per scheduler the extra instructions cost more than the special-function unit saves.)
template <typename T, bool MASKED>
__device__ __forceinline__ void chunk_exp_store(const uint32_t (&sc)[kChunk], uint32_t tmem_p, float2 scale2,
                                                float2 bias2, int limit, float2 (&sum)[2]) {
    uint32_t packed[kChunk / 2];
#pragma unroll
    for (int i = 0; i < kChunk; i += 2) {
        const float2 x = __ffma2_rn(make_float2(__uint_as_float(sc[i]), __uint_as_float(sc[i + 1])), scale2, bias2);
        float2 e;
        e.x = exp2_approx(x.x);
        e.y = exp2_approx(x.y);
        if (MASKED) {
            e.x = (i < limit) ? e.x : 0.0f;
            e.y = (i + 1 < limit) ? e.y : 0.0f;
        }
        sum[(i >> 1) & 1] = __fadd2_rn(sum[(i >> 1) & 1], e);
        packed[i >> 1] = pack2<T>(e.x, e.y);
    }
    tmem_st_x16(tmem_p, packed);
}

// One row of one key tile: S (128 f32 columns at `tmem_s`) -> P (64 packed columns over the same place), chunk by
// chunk with the next chunk's load in flight.
template <typename T, bool MASKED>
__device__ __forceinline__ void tile_exp(uint32_t tmem_s, float2 scale2, float2 bias2, int limit, float2 (&sum)[2]) {
    uint32_t buf[2][kChunk];
    tmem_ld_x32(tmem_s, buf[0]);
#pragma unroll
    for (int c = 0; c < kTile / kChunk; ++c) {
        tmem_wait_ld_into(buf[c & 1]);
        if (c + 1 < kTile / kChunk) tmem_ld_x32(tmem_s + (c + 1) * kChunk, buf[(c + 1) & 1]);
        chunk_exp_store<T, MASKED>(buf[c & 1], tmem_s + c * (kChunk / 2), scale2, bias2, limit - c * kChunk, sum);
    }
}

// Exact maximum of the visible raw scores (times `sign`) of one row of one key tile.
template <bool MASKED>
__device__ __forceinline__ float tile_max(uint32_t tmem_s, int limit, float sign) {
    float m[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
    uint32_t buf[2][kChunk];
    tmem_ld_x32(tmem_s, buf[0]);
#pragma unroll
    for (int c = 0; c < kTile / kChunk; ++c) {
        tmem_wait_ld_into(buf[c & 1]);
        if (c + 1 < kTile / kChunk) tmem_ld_x32(tmem_s + (c + 1) * kChunk, buf[(c + 1) & 1]);
        chunk_max<MASKED>(buf[c & 1], limit - c * kChunk, sign, m);
    }
    return fmaxf(fmaxf(m[0], m[1]), fmaxf(m[2], m[3]));
}

// Multiplies this thread's row of O (HD f32 columns of tensor memory) by `factor`.
template <int HD>
__device__ __forceinline__ void scale_o_row(uint32_t tmem_o, float factor) {
#pragma unroll 1
    for (int c = 0; c < HD; c += 32) {
        uint32_t r[32];
        tmem_ld_x32(tmem_o + c, r);
        tmem_wait_ld_into(r);
#pragma unroll
        for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * factor);
        tmem_st_x32(tmem_o + c, r);
    }
    tmem_wait_st();
}

// One unit of work: 256 query rows (tiles A and B) of one (sequence, head).
struct Item {
    int head;
    int kv_head;
    int seq;        // sequence index (row of the block table in the paged form)
    int offset;     // first packed query row of the sequence
    int offset_kv;  // first packed key row of the sequence (the same row except in the dense form)
    int q0;         // sequence-local index of the first query row
    int len_q;
    int len_kv;
    int shift;      // causal mask: query row i sees keys 0 .. max(i + shift, 0); 0 for the sequence-local mask,
                    // len_kv - len_q when the queries are the sequence's last tokens
    int tiles[2];   // key tiles tile A / tile B need (0: no real row, or no visible key)
    int key_tiles;  // max of the two
    bool valid;     // false: the sequence's offsets leave the packed tensors
};

__device__ __forceinline__ int pairs_of(int len_q) { return (max(len_q, 0) + kPair - 1) / kPair; }

// Items are numbered heaviest first: rank = index / heads walks the query pairs of all sequences from the highest
// pair index down (under a causal mask a pair's work grows with its index), head = index % heads.  `counts[t]` is
// the number of sequences that have a pair t, `tmax` the largest pair count.  Every lane of the calling warp
// takes part and receives the same answer.
template <bool DENSE>
__device__ __forceinline__ Item decode_item(const PrefillParams &p, const int *counts, int tmax, int index, int lane) {
    constexpr unsigned kFull = 0xffffffffu;
    Item item;
    int rank = index / p.heads;
    item.head = index - rank * p.heads;
    item.kv_head = item.head / (p.heads / p.kv_heads);
    int pair = -1;
    for (int first = 0; first < tmax && pair < 0; first += 32) {
        const int t = tmax - 1 - (first + lane);
        const int count = t >= 0 ? counts[t] : 0;
        int prefix = count;  // inclusive prefix sum over the lanes
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int other = __shfl_up_sync(kFull, prefix, d);
            if (lane >= d) prefix += other;
        }
        const unsigned hit = __ballot_sync(kFull, rank < prefix);
        if (hit != 0) {
            const int where = __ffs(hit) - 1;
            pair = tmax - 1 - (first + where);
            rank -= __shfl_sync(kFull, prefix - count, where);
        } else {
            rank -= __shfl_sync(kFull, prefix, 31);
        }
    }
    int seq = -1;
    for (int first = 0; first < p.batch && seq < 0 && pair >= 0; first += 32) {
        const int b = first + lane;
        const bool has = b < p.batch && pairs_of(seq_len_q<DENSE>(p, b)) > pair;
        const unsigned mask = __ballot_sync(kFull, has);
        const int n = __popc(mask);
        if (rank < n) {
            seq = first + static_cast<int>(__fns(mask, 0, rank + 1));
        } else {
            rank -= n;
        }
    }
    item.valid = false;
    item.seq = seq < 0 ? 0 : seq;
    item.offset = 0;
    item.offset_kv = 0;
    item.q0 = max(pair, 0) * kPair;
    item.len_q = 0;
    item.len_kv = 0;
    item.shift = 0;
    item.tiles[0] = item.tiles[1] = 0;
    item.key_tiles = 0;
    if (seq < 0) return item;
    item.len_q = max(seq_len_q<DENSE>(p, seq), 0);
    item.len_kv = max(seq_len_kv<DENSE>(p, seq), 0);
    item.offset = seq_offset_q<DENSE>(p, seq);
    item.offset_kv = seq_offset_kv<DENSE>(p, seq);
    item.valid = item.offset >= 0 && item.offset + item.len_q <= p.total_q &&
                 (p.block_table != nullptr ? item.len_kv <= p.table_stride * kPageTokens
                                           : item.offset_kv + item.len_kv <= p.total_kv);
    if (!item.valid) return item;
    item.shift = p.causal == 2 ? item.len_kv - item.len_q : 0;
#pragma unroll
    for (int x = 0; x < 2; ++x) {
        const int first = item.q0 + x * kTile;
        const int real = min(max(item.len_q - first, 0), kTile);
        int visible = real > 0 ? item.len_kv : 0;
        if (p.causal && real > 0) visible = min(visible, max(first + real - 1 + item.shift, 0) + 1);
        item.tiles[x] = (visible + kTile - 1) / kTile;
    }
    item.key_tiles = max(item.tiles[0], item.tiles[1]);
    return item;
}

// SAFE = false: the first launch.  One persistent CTA per SM walks its share of the items (item round r of CTA c is
// index r * grid + c on even rounds and r * grid + grid - 1 - c on odd ones, which evens out the heaviest-first
// order); all pipelines run on across items, so the next item's loads and first MMAs overlap the current item's
// last tile and epilogue.  Softmax is single-pass after an item's first key tile.
// SAFE = true: the second launch, same grid and same shares: it leaves at once unless the flag above is raised, and
// otherwise recomputes it with the exact row maximum on every tile.
// PAGED: K and V tiles are gathered from 16-token cache pages through the block table (eight page boxes per
// 128-key tile and 64-wide half; the boxes land back to back, which is the layout one 128-row box would have).
// HD = 128 or 64: with 64 a tile is a single 128-byte-wide box (the second half of every 32 KB buffer stays unused).
// DENSE: uniform lengths, sequences back to back, LSE laid out [batch, heads, queries] (fmha_prefill_lse).
template <typename T, int HD, bool SAFE, bool PAGED, bool DENSE>
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
    constexpr int kHalves = HD / 64;                       // 128-byte-wide boxes per tile
    constexpr int kLoadBytes = kHalves * kHalfTileBytes;   // bytes one tile load delivers
    const uint32_t bar_q_full = bars;         // [2 tiles]
    const uint32_t bar_q_empty = bars + 16;   // [2 tiles]
    const uint32_t bar_k_full = bars + 32;    // [2 stages]
    const uint32_t bar_k_empty = bars + 48;   // [2]
    const uint32_t bar_v_full = bars + 64;    // [2]
    const uint32_t bar_v_empty = bars + 80;   // [2]
    const uint32_t bar_s_full = bars + 96;    // [2 tiles]
    const uint32_t bar_p_full = bars + 112;   // [2 tiles], one arrival per softmax warp of the tile
    const uint32_t bar_o_full = bars + 128;   // [2 tiles]
    const uint32_t bar_o_empty = bars + 144;  // [2 tiles], one arrival per softmax warp of the tile
    constexpr int kBarriers = 20;
    const uint32_t words = bars + 8 * kBarriers;
    volatile uint32_t *holder_ptr = reinterpret_cast<volatile uint32_t *>(smem_raw + (words - raw));
    volatile int *shared_tmax = reinterpret_cast<volatile int *>(smem_raw + (words + 4 - raw));
    volatile int *shared_ranks = reinterpret_cast<volatile int *>(smem_raw + (words + 8 - raw));
    int *counts = reinterpret_cast<int *>(smem_raw + (words + 32 - raw));  // [kMaxRankTiles]
    volatile int *redo_list = reinterpret_cast<volatile int *>(counts + kMaxRankTiles);  // [kRedoCapacity], SAFE only

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    if (SAFE && !p.exact && *reinterpret_cast<volatile unsigned *>(&g_out_of_range_seen) == 0u) {
        return;  // no first launch on this device has ever marked a row
    }

    // ---- the table behind the heaviest-first item order ----
    {
        int tmax = 0;
        for (int b = 0; b < p.batch; ++b) tmax = max(tmax, pairs_of(seq_len_q<DENSE>(p, b)));
        tmax = min(tmax, kMaxRankTiles);
        for (int t = tid; t < tmax; t += kPrefillThreads) {
            int count = 0;
            for (int b = 0; b < p.batch; ++b) count += pairs_of(seq_len_q<DENSE>(p, b)) > t ? 1 : 0;
            counts[t] = count;
        }
        __syncthreads();
        if (tid == 0) {
            int ranks = 0;
            for (int t = 0; t < tmax; ++t) ranks += counts[t];
            *shared_tmax = tmax;
            *shared_ranks = ranks;
        }
        __syncthreads();
    }
    const int tmax = *shared_tmax;
    const long long total_items = static_cast<long long>(*shared_ranks) * p.heads;
    // index of this CTA's share number `round`, or -1 past the end
    auto share_index = [&](int round) -> int {
        const long long first = static_cast<long long>(round) * gridDim.x;
        const long long index = first + ((round & 1) ? gridDim.x - 1 - blockIdx.x : blockIdx.x);
        return index < total_items ? static_cast<int>(index) : -1;
    };
    // where the LSE of (item, sequence-local query row) lives
    auto lse_at = [&](const Item &item, int row) -> float * {
        if (DENSE) {
            return p.lse + (static_cast<size_t>(item.seq) * p.heads + item.head) * p.lse_rows + row;
        }
        return p.lse + (static_cast<size_t>(item.offset) + row) * p.heads + item.head;
    };
    int listed = -1;  // SAFE: number of marked items in redo_list, or -1 = walk the whole share
    if (SAFE && !p.exact) {
        // The first launch leaves a NaN as the LSE of every row it could not finish in range: list the marked items.
        int found = 0;
        bool overflow = false;
        for (int round = 0;; ++round) {
            const int index = share_index(round);
            if (index < 0) break;
            const Item item = decode_item<DENSE>(p, counts, tmax, index, lane);
            const int row = item.q0 + tid;
            const bool marked = item.valid && item.key_tiles > 0 && tid < kPair && row < item.len_q &&
                                isnan(*lse_at(item, row));
            if (__syncthreads_or(marked ? 1 : 0) != 0) {
                if (found < kRedoCapacity) {
                    if (tid == 0) redo_list[found] = index;
                    ++found;
                } else {
                    overflow = true;
                }
            }
        }
        __syncthreads();
        if (found == 0) return;
        listed = overflow ? -1 : found;
    }
    // index of the item this CTA works on in `round`, or -1 when it is done
    auto item_index = [&](int round) -> int {
        if (SAFE && listed >= 0) return round < listed ? redo_list[round] : -1;
        return share_index(round);
    };

    if (tid == 0) {
        for (int i = 0; i < kBarriers; ++i) {
            const bool by_warps = i == 14 || i == 15 || i == 18 || i == 19;  // p_full[2], o_empty[2]
            mbar_init(bars + 8 * i, by_warps ? 4 : 1);
        }
        mbar_init_fence();
    }
    if (warp == 8) {
        tmem_alloc(words, 512);
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
        }
        int g = 0;                // key tiles loaded so far, over all items: stage g & 1, use (g >> 1)
        int q_loads[2] = {0, 0};  // Q tiles loaded so far
        auto wait_lane0 = [&](uint32_t bar, uint32_t parity) -> bool {
            int ok = 1;
            if (lane == 0) ok = mbar_wait(bar, parity) ? 1 : 0;
            return __shfl_sync(0xffffffffu, ok, 0) != 0;
        };
        for (int round = 0; !failed; ++round) {
            const int index = item_index(round);
            if (index < 0) break;
            const Item item = decode_item<DENSE>(p, counts, tmax, index, lane);
            if (item.key_tiles == 0) continue;
#pragma unroll
            for (int x = 0; x < 2; ++x) {
                if (item.tiles[x] == 0 || failed) continue;
                // the tile's buffer is free when the previous item's last Q K^T of this tile has retired
                if (q_loads[x] > 0 && !wait_lane0(bar_q_empty + x * 8, (q_loads[x] - 1) & 1)) {
                    failed = true;
                    continue;
                }
                ++q_loads[x];
                if (lane == 0) {
                    mbar_expect_tx(bar_q_full + x * 8, kLoadBytes);
                    const int row0 = item.offset + item.q0 + x * kTile;
                    tma_load_3d(q_smem + x * kTileBytes, &q_map, bar_q_full + x * 8, 0, item.head, row0);
                    if (kHalves == 2) {
                        tma_load_3d(q_smem + x * kTileBytes + kHalfTileBytes, &q_map, bar_q_full + x * 8, 64,
                                    item.head, row0);
                    }
                }
            }
            for (int j = 0; j < item.key_tiles && !failed; ++j, ++g) {
                const int stage = g & 1;
                const int row0 = item.offset_kv + j * kTile;
                if (g >= 2 && !wait_lane0(bar_k_empty + stage * 8, ((g >> 1) - 1) & 1)) {
                    failed = true;
                    break;
                }
                // paged form: lanes 0-15 each own one (page, half) box of the tile; a page past the sequence's last
                // one is replaced by the sequence's first page (finite data that the mask hides), a page id outside
                // the cache likewise, with status 1
                int32_t page = 0;
                if (PAGED) {
                    const int pages_of_sequence = (item.len_kv + kPageTokens - 1) / kPageTokens;
                    const int wanted = j * (kTile / kPageTokens) + (lane & 7);
                    const uint32_t *row = p.block_table + static_cast<size_t>(item.seq) * p.table_stride;
                    uint32_t id = row[wanted < pages_of_sequence ? wanted : 0];
                    if (id >= static_cast<uint32_t>(p.cache_pages)) {
                        report_status(p.error, kStatusIndexOutOfBounds);
                        id = 0u;
                    }
                    page = static_cast<int32_t>(id);
                }
                if (lane == 0) mbar_expect_tx(bar_k_full + stage * 8, kLoadBytes);
                __syncwarp();
                if (PAGED) {
                    if (lane < 8 * kHalves) {
                        const int half = lane >> 3;
                        tma_load_4d(k_smem + stage * kTileBytes + half * kHalfTileBytes + (lane & 7) * kPageBytes, &k_map,
                                    bar_k_full + stage * 8, half * 64, item.kv_head, 0, page);
                    }
                } else if (lane == 0) {
                    tma_load_3d(k_smem + stage * kTileBytes, &k_map, bar_k_full + stage * 8, 0, item.kv_head, row0);
                    if (kHalves == 2) {
                        tma_load_3d(k_smem + stage * kTileBytes + kHalfTileBytes, &k_map, bar_k_full + stage * 8, 64,
                                    item.kv_head, row0);
                    }
                }
                if (g >= 2 && !wait_lane0(bar_v_empty + stage * 8, ((g >> 1) - 1) & 1)) {
                    failed = true;
                    break;
                }
                if (lane == 0) mbar_expect_tx(bar_v_full + stage * 8, kLoadBytes);
                __syncwarp();
                if (PAGED) {
                    if (lane < 8 * kHalves) {
                        const int half = lane >> 3;
                        tma_load_4d(v_smem + stage * kTileBytes + half * kHalfTileBytes + (lane & 7) * kPageBytes, &v_map,
                                    bar_v_full + stage * 8, half * 64, item.kv_head, 0, page);
                    }
                } else if (lane == 0) {
                    tma_load_3d(v_smem + stage * kTileBytes, &v_map, bar_v_full + stage * 8, 0, item.kv_head, row0);
                    if (kHalves == 2) {
                        tma_load_3d(v_smem + stage * kTileBytes + kHalfTileBytes, &v_map, bar_v_full + stage * 8, 64,
                                    item.kv_head, row0);
                    }
                }
            }
        }
    } else if (warp == 8) {
        // ---------------- MMA issuer ----------------
        constexpr bool kIsBf16 = std::is_same<T, __nv_bfloat16>::value;
        constexpr uint32_t kIdescQK = make_instr_desc(kTile, kTile, kIsBf16, 0, 0);      // A, B K-major
        constexpr uint32_t kIdescPV = make_instr_desc(kTile, HD, kIsBf16, 0, 1);   // B (V) MN-major
        auto wait_all = [&](uint32_t bar, uint32_t parity) -> bool {
            return __all_sync(0xffffffffu, mbar_wait(bar, parity) ? 1 : 0) != 0;
        };
        // S_x = Q_x K(stage)^T; `last` releases the Q tile
        auto issue_qk = [&](int x, int stage, bool last) {
            if (lane == 0) {
                const uint32_t q_tile = q_smem + x * kTileBytes;
                const uint32_t k_tile = k_smem + stage * kTileBytes;
#pragma unroll
                for (int ks = 0; ks < HD / 16; ++ks) {
                    const uint32_t within = (ks >> 2) * kHalfTileBytes + (ks & 3) * 32;
                    umma_ss(tmem_base + x * kTile, make_smem_desc(q_tile + within, 16, 1024),
                            make_smem_desc(k_tile + within, 16, 1024), kIdescQK, ks > 0 ? 1u : 0u);
                }
                tcgen05_commit(bar_s_full + x * 8);
                if (last) tcgen05_commit(bar_q_empty + x * 8);
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
                    umma_ts(tmem_base + 2 * kTile + x * HD, tmem_base + x * kTile + ks * 8,
                            make_smem_desc(v_tile + ks * 2048, kHalfTileBytes, 1024), kIdescPV,
                            (accumulate || ks > 0) ? 1u : 0u);
                }
                if (last) tcgen05_commit(bar_o_full + x * 8);
            }
            __syncwarp();
        };
        int g = 0;                 // key tiles consumed so far, over all items
        int q_uses[2] = {0, 0};    // Q tiles consumed so far
        int p_uses[2] = {0, 0};    // P tiles consumed so far
        int o_done[2] = {0, 0};    // outputs handed to the epilogue so far
        int round = 0;
        // the next item with work, or key_tiles == 0 when there is none
        auto next_item = [&]() -> Item {
            Item item;
            item.key_tiles = 0;
            for (;;) {
                const int index = item_index(round);
                if (index < 0) {
                    item.key_tiles = 0;
                    return item;
                }
                ++round;
                item = decode_item<DENSE>(p, counts, tmax, index, lane);
                if (item.key_tiles > 0) return item;
            }
        };
        // first Q K^T of both tiles of `item` on key stage `stage` (already waited for)
        auto first_qk = [&](const Item &item, int x, int stage) -> bool {
            if (item.tiles[x] == 0) return true;
            if (!wait_all(bar_q_full + x * 8, q_uses[x] & 1)) return false;
            ++q_uses[x];
            tcgen05_fence_after();
            issue_qk(x, stage, item.tiles[x] == 1);
            return true;
        };
        Item item = next_item();
        if (item.key_tiles > 0) {
            if (!wait_all(bar_k_full, 0)) failed = true;
            if (!failed && (!first_qk(item, 0, 0) || !first_qk(item, 1, 0))) failed = true;
            if (!failed) {
                if (lane == 0) tcgen05_commit(bar_k_empty);
                __syncwarp();
            }
        }
        while (item.key_tiles > 0 && !failed) {
            const Item following = next_item();
            for (int j = 0; j < item.key_tiles && !failed; ++j, ++g) {
                const int stage = g & 1;
                const int next = (g + 1) & 1;
                const bool more = j + 1 < item.key_tiles;          // this item has another key tile
                const bool onward = more || following.key_tiles > 0;  // some Q K^T follows on key tile g + 1
                if (!wait_all(bar_v_full + stage * 8, (g >> 1) & 1)) {
                    failed = true;
                    break;
                }
#pragma unroll
                for (int x = 0; x < 2; ++x) {
                    if (failed) continue;
                    if (j < item.tiles[x]) {
                        // the previous item's epilogue must have taken O out of tensor memory
                        if (j == 0 && o_done[x] > 0 && !wait_all(bar_o_empty + x * 8, (o_done[x] - 1) & 1)) {
                            failed = true;
                            continue;
                        }
                        if (!wait_all(bar_p_full + x * 8, p_uses[x] & 1)) {
                            failed = true;
                            continue;
                        }
                        ++p_uses[x];
                        tcgen05_fence_after();
                        const bool last = j == item.tiles[x] - 1;
                        issue_pv(x, stage, j > 0, last);
                        if (last) ++o_done[x];
                    }
                    if (x == 1) {
                        if (lane == 0) tcgen05_commit(bar_v_empty + stage * 8);
                        __syncwarp();
                    }
                    if (onward) {
                        if (x == 0) {
                            if (!wait_all(bar_k_full + next * 8, ((g + 1) >> 1) & 1)) {
                                failed = true;
                                continue;
                            }
                            tcgen05_fence_after();
                        }
                        if (more) {
                            if (j + 1 < item.tiles[x]) issue_qk(x, next, j + 2 == item.tiles[x]);
                        } else if (!first_qk(following, x, next)) {
                            failed = true;
                            continue;
                        }
                        if (x == 1) {
                            if (lane == 0) tcgen05_commit(bar_k_empty + next * 8);
                            __syncwarp();
                        }
                    }
                }
            }
            item = following;
        }
    } else {
        // ---------------- softmax / correction / epilogue: warps 0-3 tile A, warps 4-7 tile B ----------------
        const int x = warp >> 2;
        const int quarter = warp & 3;                  // tensor-memory lanes 32*quarter .. +31
        const int local_row = quarter * 32 + lane;
        const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
        const uint32_t tmem_s = tmem_base + x * kTile + lane_base;
        const uint32_t tmem_o = tmem_base + 2 * kTile + x * HD + lane_base;
        const float2 scale2 = make_float2(p.scale_log2, p.scale_log2);
        const float sign = p.scale_log2 < 0.0f ? -1.0f : 1.0f;
        int s_uses = 0;   // score tiles consumed so far, over all items
        int o_uses = 0;   // outputs taken so far
        for (int round = 0; !failed; ++round) {
            const int index = item_index(round);
            if (index < 0) break;
            const Item item = decode_item<DENSE>(p, counts, tmax, index, lane);
            if (!item.valid) {
                if (warp == 0 && lane == 0) report_status(p.error, kStatusIndexOutOfBounds);
                continue;
            }
            const int row = item.q0 + x * kTile + local_row;    // sequence-local query index
            const bool real = row < item.len_q;
            const size_t token = static_cast<size_t>(item.offset) + (real ? row : 0);
            T *dst = static_cast<T *>(p.out) + (token * p.heads + item.head) * HD;
            float *lse_row = lse_at(item, real ? row : 0);
            const int my_tiles = x == 0 ? item.tiles[0] : item.tiles[1];
            if (my_tiles == 0) {
                // No key is visible to this tile's rows: zeros and LSE -1e20.
                if (real) {
#pragma unroll
                    for (int i = 0; i < HD / 8; ++i) reinterpret_cast<uint4 *>(dst)[i] = make_uint4(0u, 0u, 0u, 0u);
                    *lse_row = -1.0e20f;
                }
                continue;
            }
            float base_log2 = -INFINITY;  // what P, O and the row sum are relative to (log2 units); finite after tile 0
            float row_sum = 0.0f;
            bool in_range = true;
            for (int j = 0; j < my_tiles && !failed; ++j, ++s_uses) {
                if (!__all_sync(0xffffffffu, mbar_wait(bar_s_full + x * 8, s_uses & 1) ? 1 : 0)) {
                    failed = true;
                    break;
                }
                tcgen05_fence_after();  // S(j) is ready, and with it every earlier MMA of this tile: O holds P V up to j-1
                // number of keys of this key tile the row may see
                int limit = item.len_kv - j * kTile;
                if (p.causal) limit = min(limit, max(row + item.shift, 0) + 1 - j * kTile);
                limit = real ? limit : 0;
                const bool partial = __any_sync(0xffffffffu, limit < kTile);

                if (SAFE || j == 0) {
                    float wanted = (partial || sign < 0.0f) ? tile_max<true>(tmem_s, limit, sign)
                                                            : tile_max<false>(tmem_s, limit, sign);
                    wanted = fmaxf(base_log2, wanted * fabsf(p.scale_log2));
                    wanted = wanted == -INFINITY ? 0.0f : wanted;  // nothing visible yet: any base will do
                    // Re-base O only when some row's max grew past the threshold; then every row of the warp does.
                    const bool grow = wanted > base_log2 + kRescaleThreshold;
                    if (__any_sync(0xffffffffu, grow)) {
                        if (j > 0) {
                            const float factor = exp2_approx(base_log2 - wanted);
                            row_sum *= factor;
                            scale_o_row<HD>(tmem_o, factor);
                        }
                        base_log2 = wanted;
                    }
                } else if (__any_sync(0xffffffffu, row_sum > kRebaseLimit)) {
                    // Single-pass tiles: pull the row back by the exponent of its sum, an exact power of two.
                    const int exponent = row_sum > kRebaseLimit ? ((__float_as_int(row_sum) >> 23) & 0xff) - 127 : 0;
                    const float factor = __int_as_float((127 - exponent) << 23);
                    row_sum *= factor;
                    base_log2 += static_cast<float>(exponent);
                    scale_o_row<HD>(tmem_o, factor);
                }
                const float2 bias2 = make_float2(-base_log2, -base_log2);
                float2 sum[2] = {make_float2(row_sum, 0.0f), make_float2(0.0f, 0.0f)};
                if (partial) {
                    tile_exp<T, true>(tmem_s, scale2, bias2, limit, sum);
                } else {
                    tile_exp<T, false>(tmem_s, scale2, bias2, limit, sum);
                }
                row_sum = (sum[0].x + sum[0].y) + (sum[1].x + sum[1].y);
                tmem_wait_st();
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(bar_p_full + x * 8);
                }
                in_range = in_range && row_sum < kOverflowLimit;  // false for inf and NaN too
            }
            if (failed) break;
            // ---- epilogue: O / sum -> bf16, LSE ----
            if (!__all_sync(0xffffffffu, mbar_wait(bar_o_full + x * 8, o_uses & 1) ? 1 : 0)) {
                failed = true;
                break;
            }
            ++o_uses;
            tcgen05_fence_after();
            const bool empty = row_sum == 0.0f;
            const float inverse = empty ? 0.0f : 1.0f / row_sum;
#pragma unroll 1
            for (int c = 0; c < HD; c += 32) {
                uint32_t r[32];
                tmem_ld_x32(tmem_o + c, r);
                tmem_wait_ld_into(r);
                if (c + 32 == HD) {
                    // O is out of tensor memory: the next item's first P V may overwrite it
                    tcgen05_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_o_empty + x * 8);
                }
                if (real) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint4 word;
                        word.x = pack2<T>(__uint_as_float(r[i]) * inverse, __uint_as_float(r[i + 1]) * inverse);
                        word.y = pack2<T>(__uint_as_float(r[i + 2]) * inverse, __uint_as_float(r[i + 3]) * inverse);
                        word.z = pack2<T>(__uint_as_float(r[i + 4]) * inverse, __uint_as_float(r[i + 5]) * inverse);
                        word.w = pack2<T>(__uint_as_float(r[i + 6]) * inverse, __uint_as_float(r[i + 7]) * inverse);
                        if (empty) word = make_uint4(0u, 0u, 0u, 0u);
                        *reinterpret_cast<uint4 *>(dst + c + i) = word;
                    }
                }
            }
            if (real) {
                float value = empty ? -1.0e20f : (base_log2 + log2f(row_sum)) * 0.6931471805599453f;
                if (!SAFE && !in_range) {
                    value = __int_as_float(0x7fc00000);  // has the second launch redo the item
                    atomicExch(&g_out_of_range_seen, 1u);
                }
                *lse_row = value;
            }
        }
    }
    if (failed && lane == 0) {
        report_status(p.error, kStatusWaitTimeout);
    }
    if (failed) linger_after_timeout();
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 8) {
        tcgen05_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

constexpr int kPrefillSmem = 6 * kTileBytes + 8 * 20 + 32 + kMaxRankTiles * 4 + kRedoCapacity * 4 + 1024;

}  // namespace

bool prefill_fast_path(size_t heads, size_t kv_heads, size_t head_dim, size_t total_query_tokens, const void *query,
                       const void *key, const void *value, const void *out) {
    // The heaviest-first item table holds kMaxRankTiles query pairs per sequence.
    if (total_query_tokens / kPair + 1 > kMaxRankTiles) return false;
    const uintptr_t all = reinterpret_cast<uintptr_t>(query) | reinterpret_cast<uintptr_t>(key) |
                          reinterpret_cast<uintptr_t>(value) | reinterpret_cast<uintptr_t>(out);
    return (head_dim == 128 || head_dim == 64) && heads % kv_heads == 0 && heads <= 65535 && (all & 15u) == 0;
}

namespace {

template <typename T, int HD, bool PAGED, bool DENSE = false>
int launch_prefill(cudaStream_t stream, const CUtensorMap &q_map, const CUtensorMap &k_map, const CUtensorMap &v_map,
                   const PrefillParams &params, unsigned persistent) {
    SINGE_CUDA_TRY(cudaFuncSetAttribute(prefill_tcgen05_kernel<T, HD, true, PAGED, DENSE>,
                                        cudaFuncAttributeMaxDynamicSharedMemorySize, kPrefillSmem));
    if (std::is_same<T, __nv_bfloat16>::value) {
        SINGE_CUDA_TRY(cudaFuncSetAttribute(prefill_tcgen05_kernel<__nv_bfloat16, HD, false, PAGED, DENSE>,
                                            cudaFuncAttributeMaxDynamicSharedMemorySize, kPrefillSmem));
        prefill_tcgen05_kernel<__nv_bfloat16, HD, false, PAGED, DENSE>
            <<<persistent, kPrefillThreads, kPrefillSmem, stream>>>(q_map, k_map, v_map, params);
        SINGE_TRY(launch_status());
    }
    // bf16: the redo pass over the same shares, a no-op while the device's out-of-range flag has never been raised.
    // f16 (params.exact): the only pass.  P must stay below 65504 there, so every tile takes its exact row maximum.
    prefill_tcgen05_kernel<T, HD, true, PAGED, DENSE><<<persistent, kPrefillThreads, kPrefillSmem, stream>>>(q_map, k_map, v_map,
                                                                                                  params);
    return launch_status();
}

}  // namespace

// Packed queries over packed keys/values (block_table == nullptr: key/value are [total_kv_tokens, kv_heads, 128]) or
// over a paged cache (key/value are [cache_pages, 16, kv_heads, 128], rows of block_table [batch, table_stride] list
// each sequence's pages).  lens_q == nullptr selects the dense form: `uniform_q` queries and `uniform_kv` keys per
// sequence, back to back, and an LSE laid out [batch, heads, uniform_q].  is_f16: IEEE half instead of bf16.
int prefill_tcgen05(cudaStream_t stream, bool is_f16, void *out, float *lse, const void *query, const void *key,
                    const void *value, const int32_t *lens_q, const int32_t *lens_kv, const int32_t *offsets,
                    size_t batch, size_t total_query_tokens, size_t total_kv_tokens, size_t heads, size_t kv_heads,
                    size_t head_dim, int causal, float scale, const uint32_t *block_table, size_t table_stride,
                    size_t cache_pages, size_t uniform_q, size_t uniform_kv) {
    if (head_dim != 128 && head_dim != 64) return SINGE_ERR_UNSUPPORTED_WIDTH;
    const uint64_t kHeadDim = head_dim;
    int device = 0, sms = 0;
    SINGE_CUDA_TRY(cudaGetDevice(&device));
    SINGE_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
    const bool paged = block_table != nullptr;
    const CUtensorMapDataType type = is_f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    CUtensorMap q_map, k_map, v_map;
    const uint32_t box[3] = {64, 1, kTile};
    {
        const uint64_t dims[3] = {kHeadDim, heads, total_query_tokens};
        const uint64_t strides[2] = {kHeadDim * 2, kHeadDim * 2 * heads};
        SINGE_TRY(encode_tensor_map(&q_map, type, 3, query, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B,
                                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B));
    }
    if (paged) {
        const uint64_t dims[4] = {kHeadDim, kv_heads, kPageTokens, cache_pages};
        const uint64_t strides[3] = {kHeadDim * 2, kHeadDim * 2 * kv_heads, kHeadDim * 2 * kv_heads * kPageTokens};
        const uint32_t page_box[4] = {64, 1, kPageTokens, 1};
        SINGE_TRY(encode_tensor_map(&k_map, type, 4, key, dims, strides, page_box, CU_TENSOR_MAP_SWIZZLE_128B,
                                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B));
        SINGE_TRY(encode_tensor_map(&v_map, type, 4, value, dims, strides, page_box, CU_TENSOR_MAP_SWIZZLE_128B,
                                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B));
    } else {
        const uint64_t dims[3] = {kHeadDim, kv_heads, total_kv_tokens};
        const uint64_t strides[2] = {kHeadDim * 2, kHeadDim * 2 * kv_heads};
        SINGE_TRY(encode_tensor_map(&k_map, type, 3, key, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B,
                                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B));
        SINGE_TRY(encode_tensor_map(&v_map, type, 3, value, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B,
                                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B));
    }
    PrefillParams params;
    params.out = out;
    params.lse = lse;
    params.lens_q = lens_q;
    params.lens_kv = lens_kv;
    params.offsets = offsets;
    params.uniform_q = static_cast<int>(uniform_q);
    params.uniform_kv = static_cast<int>(uniform_kv);
    params.lse_rows = lens_q == nullptr ? static_cast<int>(uniform_q) : 0;
    params.exact = is_f16 ? 1 : 0;
    params.batch = static_cast<int>(batch);
    params.heads = static_cast<int>(heads);
    params.kv_heads = static_cast<int>(kv_heads);
    params.total_q = static_cast<int>(total_query_tokens);
    params.total_kv = static_cast<int>(total_kv_tokens);
    params.block_table = block_table;
    params.table_stride = static_cast<int>(table_stride);
    params.cache_pages = static_cast<int>(cache_pages);
    params.causal = causal == 2 ? 2 : (causal ? 1 : 0);
    params.scale_log2 = scale * 1.4426950408889634f;
    params.error = device_error_word();
    // Upper bound on the items: every sequence can add one partial 256-row pair.
    const size_t items = (total_query_tokens / kPair + batch) * heads;
    if (items > 0x7fffffffull) return SINGE_ERR_LENGTH_EXCEEDS_I32;
    if (items == 0) return SINGE_OK;
    const unsigned persistent = static_cast<unsigned>(items < static_cast<size_t>(sms) ? items : sms);
    if (lens_q == nullptr) {
        // the dense form: ragged keys only
        if (paged) return SINGE_ERR_UNSUPPORTED_CONFIGURATION;
        if (head_dim == 64) {
            return is_f16 ? launch_prefill<__half, 64, false, true>(stream, q_map, k_map, v_map, params, persistent)
                          : launch_prefill<__nv_bfloat16, 64, false, true>(stream, q_map, k_map, v_map, params, persistent);
        }
        return is_f16 ? launch_prefill<__half, 128, false, true>(stream, q_map, k_map, v_map, params, persistent)
                      : launch_prefill<__nv_bfloat16, 128, false, true>(stream, q_map, k_map, v_map, params, persistent);
    }
    if (head_dim == 64) {
        if (is_f16) {
            return paged ? launch_prefill<__half, 64, true>(stream, q_map, k_map, v_map, params, persistent)
                         : launch_prefill<__half, 64, false>(stream, q_map, k_map, v_map, params, persistent);
        }
        return paged ? launch_prefill<__nv_bfloat16, 64, true>(stream, q_map, k_map, v_map, params, persistent)
                     : launch_prefill<__nv_bfloat16, 64, false>(stream, q_map, k_map, v_map, params, persistent);
    }
    if (is_f16) {
        return paged ? launch_prefill<__half, 128, true>(stream, q_map, k_map, v_map, params, persistent)
                     : launch_prefill<__half, 128, false>(stream, q_map, k_map, v_map, params, persistent);
    }
    return paged ? launch_prefill<__nv_bfloat16, 128, true>(stream, q_map, k_map, v_map, params, persistent)
                 : launch_prefill<__nv_bfloat16, 128, false>(stream, q_map, k_map, v_map, params, persistent);
}

int prefill_tcgen05_bf16(cudaStream_t stream, void *out, float *lse, const void *query, const void *key,
                         const void *value, const int32_t *lens_q, const int32_t *lens_kv, const int32_t *offsets,
                         size_t batch, size_t total_query_tokens, size_t total_kv_tokens, size_t heads,
                         size_t kv_heads, size_t head_dim, int causal, float scale, const uint32_t *block_table,
                         size_t table_stride, size_t cache_pages) {
    return prefill_tcgen05(stream, false, out, lse, query, key, value, lens_q, lens_kv, offsets, batch,
                           total_query_tokens, total_kv_tokens, heads, kv_heads, head_dim, causal, scale, block_table,
                           table_stride, cache_pages, 0, 0);
}

}  // namespace singe
