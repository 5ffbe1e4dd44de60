// C-ABI entry points of the attention surfaces: host-side validation that mirrors the reference's
// config validators, dispatch between the specialised kernels and the general one, and the policies
// that describe each surface to the general kernel.
#include <cmath>
#include <mutex>

#include "attention_general.cuh"
#include <type_traits>

#include "common.cuh"

namespace singe {

// paged_decode.cu
bool paged_decode_fast_path(size_t heads, size_t kv_heads, size_t head_dim, size_t block_size, const void *key_cache,
                            const void *value_cache, const void *query);
size_t paged_decode_split_tokens(size_t key_len_bound, size_t max_splits, size_t block_size);
int paged_decode_splitk(cudaStream_t stream, int element, void *out, float *attn_scratch, float *lse_scratch,
                        const void *query, const void *key_cache, const void *value_cache,
                        const int32_t *actual_seq_lens, const uint32_t *block_table, size_t batch, size_t heads,
                        size_t kv_heads, size_t head_dim, size_t physical_blocks, size_t block_table_batch_stride,
                        size_t max_splits, float scale, bool partials_only, uint32_t *status,
                        const RaggedDecode *ragged, unsigned hints, const QueryRotation *rotation, uint32_t *tickets,
                        const FusedStep *fused);
extern int g_decode_prefetch_pages;
// prefill_tcgen05.cu
bool prefill_fast_path(size_t heads, size_t kv_heads, size_t head_dim, size_t total_query_tokens, const void *query,
                       const void *key, const void *value, const void *out);
int prefill_tcgen05_bf16(cudaStream_t stream, void *out, float *lse, const void *query, const void *key,
                         const void *value, const int32_t *lens_q, const int32_t *lens_kv, const int32_t *offsets,
                         size_t batch, size_t total_query_tokens, size_t total_kv_tokens, size_t heads,
                         size_t kv_heads, size_t head_dim, int causal, float scale, const uint32_t *block_table,
                         size_t table_stride, size_t cache_pages);
int prefill_tcgen05(cudaStream_t stream, bool is_f16, void *out, float *lse, const void *query, const void *key,
                    const void *value, const int32_t *lens_q, const int32_t *lens_kv, const int32_t *offsets,
                    size_t batch, size_t total_query_tokens, size_t total_kv_tokens, size_t heads, size_t kv_heads,
                    size_t head_dim, int causal, float scale, const uint32_t *block_table, size_t table_stride,
                    size_t cache_pages, size_t uniform_q, size_t uniform_kv);
// kv_cache_write.cu
int kv_cache_write(cudaStream_t stream, void *key_cache, void *value_cache, const void *keys, const void *values,
                   const void *write_pages, const void *write_slots, int index_width, size_t tokens, size_t kv_heads,
                   size_t head_dim, size_t pages, size_t page_size, uint32_t *status, size_t element_bytes);

namespace {

bool finite(float value) { return value == value && value - value == 0.0f; }

// validate_paged_kv_decode_attention_config (singe-kernel/src/cuda/attention/mod.rs:2963-2985)
int validate_paged_decode(size_t batch, size_t heads, size_t kv_heads, size_t head_dim, size_t block_size,
                          size_t physical_blocks, size_t stride, float scale) {
    if (batch == 0 || heads == 0 || kv_heads == 0 || head_dim == 0 || block_size == 0 || physical_blocks == 0 ||
        stride == 0 || heads % kv_heads != 0 || !finite(scale)) {
        return SINGE_ERR_INVALID_LENGTH;
    }
    if (!fits_i32(batch) || !fits_i32(heads) || !fits_i32(kv_heads) || !fits_i32(head_dim) || !fits_i32(block_size) ||
        !fits_i32(physical_blocks) || !fits_i32(stride)) {
        return SINGE_ERR_LENGTH_EXCEEDS_I32;
    }
    return SINGE_OK;
}

// validate_paged_kv_prefill_attention_config (singe-kernel/src/cuda/attention/mod.rs:2987-3011)
int validate_paged_prefill(size_t batch, size_t total, size_t heads, size_t kv_heads, size_t head_dim,
                           size_t block_size, size_t physical_blocks, size_t stride, float scale) {
    if (total == 0) return SINGE_ERR_INVALID_LENGTH;
    if (!fits_i32(total)) return SINGE_ERR_LENGTH_EXCEEDS_I32;
    return validate_paged_decode(batch, heads, kv_heads, head_dim, block_size, physical_blocks, stride, scale);
}

// validate_ragged_kv_prefill_attention_config (singe-kernel/src/cuda/attention/mod.rs:3013-3040)
int validate_ragged_prefill(size_t batch, size_t total_q, size_t total_kv, size_t heads, size_t kv_heads,
                            size_t head_dim, float scale) {
    if (batch == 0 || total_q == 0 || total_kv == 0 || heads == 0 || kv_heads == 0 || head_dim == 0 ||
        heads % kv_heads != 0 || !finite(scale)) {
        return SINGE_ERR_INVALID_LENGTH;
    }
    if (!fits_i32(batch) || !fits_i32(total_q) || !fits_i32(total_kv) || !fits_i32(heads) || !fits_i32(kv_heads) ||
        !fits_i32(head_dim)) {
        return SINGE_ERR_LENGTH_EXCEEDS_I32;
    }
    return SINGE_OK;
}

// ---------------------------------------------------------------------------------------------
// Policies of the general kernel
// ---------------------------------------------------------------------------------------------

// paged_kv_decode_attention (singe-kernel/src/cpu/attention.rs:1172-1246): one query per sequence.
template <typename T>
struct DecodePagedPolicy {
    const T *query;
    T *out;
    const T *key_cache;
    const T *value_cache;
    const int32_t *lens;
    const uint32_t *table;
    int heads, kv_heads, head_dim, block_size;
    long long physical_blocks, stride;

    __device__ int locate(size_t row, RowPlan<T> &plan) const {
        const size_t b = row / heads;
        const int head = static_cast<int>(row - b * heads);
        long long len = lens[b];
        if (len < 0) len = 0;
        if (len > stride * block_size) return -1;
        plan.query = query + row * head_dim;
        plan.out = out + row * head_dim;
        plan.lse = nullptr;
        plan.start = 0;
        plan.end = static_cast<int>(len);
        plan.kv_head = head / (heads / kv_heads);
        plan.handle = static_cast<long long>(b) * stride;
        return 1;
    }
    __device__ long long key_offset(const RowPlan<T> &plan, int pos) const {
        const long long block = table[plan.handle + pos / block_size];
        if (block >= physical_blocks) return -1;
        return ((block * block_size + pos % block_size) * kv_heads + plan.kv_head) * head_dim;
    }
    __device__ const T *key_base() const { return key_cache; }
    __device__ const T *value_base() const { return value_cache; }
};

// paged / ragged packed prefill (singe-kernel/src/cpu/attention.rs:1248-1420).  table == nullptr selects ragged.
template <typename T>
struct PackedPrefillPolicy {
    const T *query;
    T *out;
    float *lse;
    const T *key;
    const T *value;
    const int32_t *lens_q;
    const int32_t *lens_kv;
    const int32_t *offsets;
    const uint32_t *table;
    int batch, heads, kv_heads, head_dim, block_size, causal;
    long long physical_blocks, stride, total_query_tokens, total_kv_tokens;

    __device__ int locate(size_t row, RowPlan<T> &plan) const {
        const long long token = static_cast<long long>(row / heads);
        const int head = static_cast<int>(row - static_cast<size_t>(token) * heads);
        int owner = -1;
        long long local = 0;
        for (int b = 0; b < batch; ++b) {
            const long long first = offsets[b];
            const long long count = lens_q[b];
            if (token >= first && token < first + count) {
                owner = b;
                local = token - first;
                break;
            }
        }
        if (owner < 0) return 0;
        long long keys = lens_kv[owner];
        if (keys < 0) keys = 0;
        if (table != nullptr) {
            if (keys > stride * block_size) return -1;
        } else {
            if (static_cast<long long>(offsets[owner]) + keys > total_kv_tokens) return -1;
        }
        long long end = keys;
        if (causal == 1 && local + 1 < end) end = local + 1;
        if (causal == 2) {
            // the queries are the sequence's last tokens (attend_paged, backend/cpu/normalization/attention.rs:481-483)
            long long position = keys + local - static_cast<long long>(lens_q[owner]);
            if (position < 0) position = 0;
            if (position + 1 < end) end = position + 1;
        }
        plan.query = query + row * head_dim;
        plan.out = out + row * head_dim;
        plan.lse = lse + row;
        plan.start = 0;
        plan.end = static_cast<int>(end);
        plan.kv_head = head / (heads / kv_heads);
        plan.handle = table != nullptr ? static_cast<long long>(owner) * stride : static_cast<long long>(offsets[owner]);
        return 1;
    }
    __device__ long long key_offset(const RowPlan<T> &plan, int pos) const {
        if (table != nullptr) {
            const long long block = table[plan.handle + pos / block_size];
            if (block >= physical_blocks) return -1;
            return ((block * block_size + pos % block_size) * kv_heads + plan.kv_head) * head_dim;
        }
        return ((plan.handle + pos) * kv_heads + plan.kv_head) * head_dim;
    }
    __device__ const T *key_base() const { return key; }
    __device__ const T *value_base() const { return value; }
};

// Tensor::paged_attention (singe/src/backend/cpu/normalization/attention.rs:424-540) with the refusals of
// check_paged_values (singe/src/backend/spec/neural/attention.rs:363-416) applied to the row's own sequence.
template <typename T, typename Index>
struct TensorPagedPolicy {
    const T *query;
    T *out;
    float *lse;
    const T *key_cache;
    const T *value_cache;
    const Index *query_offsets;
    const Index *page_offsets;
    const Index *pages;
    const Index *last_page_lengths;
    int sequences, heads, kv_heads, head_dim, page_size, causal;
    long long tokens, cache_pages, table_len, window;
    const int *skip_when_zero;  // the planning kernel's verdict: 0 = the tiled decode kernel serves this call

    __device__ int locate(size_t row, RowPlan<T> &plan) const {
        if (skip_when_zero != nullptr && *skip_when_zero == 0) return 0;
        const long long token = static_cast<long long>(row / heads);
        const int head = static_cast<int>(row - static_cast<size_t>(token) * heads);
        int owner = -1;
        long long first_query = 0, end_query = 0;
        for (int s = 0; s < sequences; ++s) {
            const long long first = static_cast<long long>(query_offsets[s]);
            const long long last = static_cast<long long>(query_offsets[s + 1]);
            if (token >= first && token < last) {
                owner = s;
                first_query = first;
                end_query = last;
                break;
            }
        }
        if (owner < 0) return 0;
        if (first_query < 0 || end_query > tokens) return -1;
        const long long first_page = static_cast<long long>(page_offsets[owner]);
        const long long last_page = static_cast<long long>(page_offsets[owner + 1]);
        if (first_page < 0 || first_page > last_page || last_page > table_len) return -1;
        const long long page_count = last_page - first_page;
        long long keys = 0;
        if (page_count > 0) {
            const long long last_length = static_cast<long long>(last_page_lengths[owner]);
            if (last_length < 0 || last_length > page_size) return -1;
            keys = (page_count - 1) * page_size + last_length;
        }
        const long long queries = end_query - first_query;
        long long position = keys + (token - first_query) - queries;  // queries are the sequence's last tokens
        if (position < 0) position = 0;
        long long end = keys;
        if (causal && position + 1 < end) end = position + 1;
        long long start = 0;
        if (window > 0 && position + 1 > window) start = position + 1 - window;
        if (end < start) end = start;
        plan.query = query + row * head_dim;
        plan.out = out + row * head_dim;
        plan.lse = lse + row;
        plan.start = static_cast<int>(start);
        plan.end = static_cast<int>(end);
        plan.kv_head = head / (heads / kv_heads);
        plan.handle = first_page;
        return 1;
    }
    __device__ long long key_offset(const RowPlan<T> &plan, int pos) const {
        const long long page = static_cast<long long>(pages[plan.handle + pos / page_size]);
        if (page < 0 || page >= cache_pages) return -1;
        return ((page * page_size + pos % page_size) * kv_heads + plan.kv_head) * head_dim;
    }
    __device__ const T *key_base() const { return key_cache; }
    __device__ const T *value_base() const { return value_cache; }
};

// The whole-table refusal of check_paged_values: any sequence with bad offsets, pages or last length sets the status.
// One warp per sequence; its lanes share the sequence's page list.
template <typename Index>
__device__ __forceinline__ void check_paged_values_body(const Index *query_offsets, const Index *page_offsets,
                                                        const Index *pages, const Index *last_page_lengths,
                                                        int sequences, long long tokens, long long cache_pages,
                                                        long long table_len, long long page_size, uint32_t *status,
                                                        int block, int blocks) {
    const int lane = threadIdx.x & 31;
    const int warps = (blocks * blockDim.x) >> 5;
    for (int s = (block * blockDim.x + threadIdx.x) >> 5; s < sequences; s += warps) {
        const long long qf = static_cast<long long>(query_offsets[s]), ql = static_cast<long long>(query_offsets[s + 1]);
        const long long pf = static_cast<long long>(page_offsets[s]), pl = static_cast<long long>(page_offsets[s + 1]);
        bool bad = !(0 <= qf && qf <= ql && ql <= tokens) || !(0 <= pf && pf <= pl && pl <= table_len);
        if (!bad && pf != pl) {
            const long long last = static_cast<long long>(last_page_lengths[s]);
            bad = last < 0 || last > page_size;
            for (long long i = pf + lane; i < pl && !bad; i += 32) {
                const long long page = static_cast<long long>(pages[i]);
                bad = page < 0 || page >= cache_pages;
            }
        }
        if (bad) report_status(status, kStatusIndexOutOfBounds);
    }
}

template <typename Index>
__global__ void check_paged_values_kernel(const Index *query_offsets, const Index *page_offsets, const Index *pages,
                                          const Index *last_page_lengths, int sequences, long long tokens,
                                          long long cache_pages, long long table_len, long long page_size,
                                          uint32_t *status) {
    check_paged_values_body<Index>(query_offsets, page_offsets, pages, last_page_lengths, sequences, tokens, cache_pages,
                                   table_len, page_size, status, blockIdx.x, gridDim.x);
}

// Decides, on the device, whether a Tensor-surface call is a plain decode batch (sequence b owns exactly query
// token b, every paging value is valid) and, if so, turns the paging tensors into what the tiled decode kernel
// reads: lens[b], first[b] (index of the sequence's first page) and the tokens per split for `split_budget` splits
// of the longest sequence.  control[0] = 0 hands the call to the tiled kernel, 1 to the general kernel.
// A sliding window (window > 0: the query at position keys - 1 sees keys >= keys - window) skips whole pages here:
// first[b] moves to the page that holds the first visible key, lens[b] counts from that page's start and hidden[b]
// (0 .. page_size - 1) is the number of keys at the front of that page the window still hides.
template <typename Index>
__device__ __forceinline__ void plan_paged_decode_body(const Index *query_offsets, const Index *page_offsets,
                                                       const Index *pages, const Index *last_page_lengths,
                                                       int sequences, long long cache_pages, long long table_len,
                                                       long long page_size, int split_budget, int min_piece,
                                                       int *lens, long long *first, int *control, long long window,
                                                       int *hidden) {
    __shared__ int shared_bad;
    __shared__ int shared_longest;
    if (threadIdx.x == 0) {
        shared_bad = 0;
        shared_longest = 0;
    }
    __syncthreads();
    int bad = 0;
    int longest = 0;
    for (int s = threadIdx.x; s < sequences; s += blockDim.x) {
        const long long qf = static_cast<long long>(query_offsets[s]), ql = static_cast<long long>(query_offsets[s + 1]);
        const long long pf = static_cast<long long>(page_offsets[s]), pl = static_cast<long long>(page_offsets[s + 1]);
        long long keys = 0;
        if (qf != s || ql != s + 1 || !(0 <= pf && pf <= pl && pl <= table_len)) {
            bad = 1;
        } else if (pf != pl) {
            const long long last = static_cast<long long>(last_page_lengths[s]);
            if (last < 0 || last > page_size) bad = 1;
            keys = (pl - pf - 1) * page_size + last;
            if (keys > 0x7ffffff0ll) bad = 1;
        }
        long long skipped = 0;   // whole pages in front of the window
        if (window > 0 && !bad) {
            const long long lowest = keys > window ? keys - window : 0;
            skipped = lowest / page_size;
            hidden[s] = static_cast<int>(lowest - skipped * page_size);
            keys -= skipped * page_size;
        } else if (window > 0) {
            hidden[s] = 0;
        }
        lens[s] = bad ? 0 : static_cast<int>(keys);
        first[s] = bad ? 0 : pf + skipped;
        longest = max(longest, bad ? 0 : static_cast<int>(keys));
    }
    // every page id the table holds must address the cache (the general kernel skips the rows of a bad one)
    for (long long i = threadIdx.x; i < table_len; i += blockDim.x) {
        const long long page = static_cast<long long>(pages[i]);
        if (page < 0 || page >= cache_pages) bad = 1;
    }
    if (bad) atomicExch(&shared_bad, 1);
    atomicMax(&shared_longest, longest);
    __syncthreads();
    if (threadIdx.x == 0) {
        control[0] = shared_bad;
        // The budget bounds the grid; pieces are not made shorter than 512 keys for its sake (the split size the
        // kernel-surface decode uses), so a batch whose longest sequence needs fewer splits leaves the rest unused.
        long long per = (static_cast<long long>(shared_longest) + split_budget - 1) / split_budget;
        if (per < min_piece) per = min_piece;
        const long long rounded = (per + page_size - 1) / page_size * page_size;
        control[1] = static_cast<int>(rounded < page_size ? page_size : rounded);
    }
}

template <typename Index>
__global__ void plan_paged_decode_kernel(const Index *query_offsets, const Index *page_offsets, const Index *pages,
                                         const Index *last_page_lengths, int sequences, long long cache_pages,
                                         long long table_len, long long page_size, int split_budget, int min_piece,
                                         int *lens, long long *first, int *control, long long window, int *hidden) {
    plan_paged_decode_body<Index>(query_offsets, page_offsets, pages, last_page_lengths, sequences, cache_pages,
                                  table_len, page_size, split_budget, min_piece, lens, first, control, window, hidden);
}

// Both of the above in one launch: the last block plans, the others check (one launch gap fewer per call).
template <typename Index>
__global__ void check_and_plan_kernel(const Index *query_offsets, const Index *page_offsets, const Index *pages,
                                      const Index *last_page_lengths, int sequences, long long tokens,
                                      long long cache_pages, long long table_len, long long page_size,
                                      uint32_t *status, int split_budget, int min_piece, int *lens, long long *first,
                                      int *control, long long window, int *hidden) {
    if (blockIdx.x == gridDim.x - 1) {
        plan_paged_decode_body<Index>(query_offsets, page_offsets, pages, last_page_lengths, sequences, cache_pages,
                                      table_len, page_size, split_budget, min_piece, lens, first, control, window,
                                      hidden);
    } else {
        check_paged_values_body<Index>(query_offsets, page_offsets, pages, last_page_lengths, sequences, tokens,
                                       cache_pages, table_len, page_size, status, blockIdx.x, gridDim.x - 1);
    }
}

// Dense layouts with explicit strides: Tensor::attend [B,H,L,D] over [B,G,S,D]
// (singe/src/backend/cpu/normalization/attention.rs:191-276) and fmha_prefill_lse [B,L,H,D] over [B,S,G,D]
// (singe-kernel/src/cpu/attention.rs:1758-1833).
template <typename T>
struct DensePolicy {
    const T *query;
    T *out;
    float *lse;
    const T *key;
    const T *value;
    int heads, kv_heads, query_len, key_len, head_dim, causal;
    long long window;
    long long q_batch, q_head, q_row;     // element strides of query/out
    long long k_batch, k_head, k_row;     // element strides of key/value
    long long lse_batch, lse_head, lse_row;
    const T *sinks;  // [heads] one sink logit per head, or nullptr

    __device__ int locate(size_t row, RowPlan<T> &plan) const {
        const long long i = static_cast<long long>(row % query_len);
        const long long bh = static_cast<long long>(row / query_len);
        const long long head = bh % heads;
        const long long b = bh / heads;
        long long end = key_len;
        if (causal && i + 1 < end) end = i + 1;
        long long start = 0;
        if (window > 0 && i + 1 > window) start = i + 1 - window;
        if (end < start) end = start;
        const long long at = b * q_batch + head * q_head + i * q_row;
        plan.query = query + at;
        plan.out = out + at;
        plan.lse = lse == nullptr ? nullptr : lse + b * lse_batch + head * lse_head + i * lse_row;
        plan.start = static_cast<int>(start);
        plan.end = static_cast<int>(end);
        plan.kv_head = static_cast<int>(head / (heads / kv_heads));
        plan.handle = b * k_batch + plan.kv_head * k_head;
        if (sinks != nullptr) plan.sink = to_float<T>(sinks[head]);
        return 1;
    }
    __device__ long long key_offset(const RowPlan<T> &plan, int pos) const { return plan.handle + pos * k_row; }
    __device__ const T *key_base() const { return key; }
    __device__ const T *value_base() const { return value; }
};

// One decode query per (batch, head) over contiguous keys/values [B, S, G, D], cut into `splits` key ranges: row
// (b, head, s) attends keys [s * per_split, min(S, (s + 1) * per_split)) and leaves its normalised partial in
// out [B, H, splits, D] and its natural-log LSE in lse [B, H, splits] (fmha_decode_splitk_f32,
// singe-kernel/src/cuda/attention/fmha.rs:1073-1117); splitk_reduce_kernel folds them.
template <typename T>
struct DenseSplitPolicy {
    const T *query;
    T *out;
    float *lse;
    const T *key;
    const T *value;
    int heads, kv_heads, key_len, head_dim, splits, per_split;

    __device__ int locate(size_t row, RowPlan<T> &plan) const {
        const long long split = static_cast<long long>(row % splits);
        const long long bh = static_cast<long long>(row / splits);
        const long long head = bh % heads;
        const long long b = bh / heads;
        long long start = split * per_split;
        long long end = start + per_split;
        if (end > key_len) end = key_len;
        if (start > end) start = end;
        plan.query = query + bh * head_dim;
        plan.out = out + static_cast<long long>(row) * head_dim;
        plan.lse = lse + row;
        plan.start = static_cast<int>(start);
        plan.end = static_cast<int>(end);
        plan.kv_head = static_cast<int>(head / (heads / kv_heads));
        plan.handle = (b * key_len * kv_heads + plan.kv_head) * head_dim;
        return 1;
    }
    __device__ long long key_offset(const RowPlan<T> &plan, int pos) const {
        return plan.handle + static_cast<long long>(pos) * kv_heads * head_dim;
    }
    __device__ const T *key_base() const { return key; }
    __device__ const T *value_base() const { return value; }
};

// ---------------------------------------------------------------------------------------------
// Per-device split-K workspace of the drop-in decode entry points
// ---------------------------------------------------------------------------------------------
// The reference's scratch-less signatures leave the library to find split-K scratch.  One buffer per device, shared by
// every stream: calls that use it must not overlap on the GPU (callers that run decode on several streams of one
// device at once pass their own scratch through the *_splitk_reduce_* entry points).  Growth happens outside stream
// capture only and never frees: a CUDA graph captured earlier has the old address baked in, so a buffer that was ever
// handed out stays allocated until singe_release_workspaces() or process exit.
struct Workspace {
    float *data = nullptr;
    size_t floats = 0;
    float *retired[32] = {nullptr};
    int retired_count = 0;
};
Workspace g_workspace[kMaxDevices];
std::mutex g_workspace_mutex;

int workspace_for(cudaStream_t stream, size_t floats, float **data) {
    const int device = device_slot();
    if (device < 0) return SINGE_ERR_UNSUPPORTED_CONFIGURATION;
    std::lock_guard<std::mutex> guard(g_workspace_mutex);
    Workspace &space = g_workspace[device];
    if (space.floats < floats) {
        cudaStreamCaptureStatus capture = cudaStreamCaptureStatusNone;
        SINGE_CUDA_TRY(cudaStreamIsCapturing(stream, &capture));
        if (capture != cudaStreamCaptureStatusNone) {
            return SINGE_ERR_AUTOTUNE_DURING_CAPTURE;
        }
        if (space.data != nullptr && space.retired_count >= 32) return SINGE_ERR_UNSUPPORTED_CONFIGURATION;
        // Doubling keeps the number of retired buffers logarithmic in the largest problem seen.
        size_t grown = floats + floats / 2;
        if (grown < 2 * space.floats) grown = 2 * space.floats;
        float *fresh = nullptr;
        SINGE_CUDA_TRY(cudaMalloc(&fresh, grown * sizeof(float)));
        if (space.data != nullptr) space.retired[space.retired_count++] = space.data;
        space.data = fresh;
        space.floats = grown;
    }
    *data = space.data;
    return SINGE_OK;
}

int release_workspaces() {
    const int device = device_slot();
    if (device < 0) return SINGE_ERR_UNSUPPORTED_CONFIGURATION;
    std::lock_guard<std::mutex> guard(g_workspace_mutex);
    Workspace &space = g_workspace[device];
    SINGE_CUDA_TRY(cudaDeviceSynchronize());
    for (int i = 0; i < space.retired_count; ++i) cudaFree(space.retired[i]);
    space.retired_count = 0;
    if (space.data != nullptr) cudaFree(space.data);
    space.data = nullptr;
    space.floats = 0;
    return SINGE_OK;
}

// Splits the drop-in decode uses when the caller gives no budget: ~512-token splits, more when few CTAs would run.
size_t default_splits(size_t batch, size_t kv_heads, size_t bound_tokens) {
    size_t splits = (bound_tokens + 511) / 512;
    const size_t wanted = static_cast<size_t>(device_sm_count()) * 4;
    const size_t rows = batch * kv_heads;
    if (rows * splits < wanted) {
        const size_t more = (wanted + rows - 1) / rows;
        const size_t finest = (bound_tokens + 127) / 128;
        splits = more < finest ? more : finest;
    }
    if (splits < 1) splits = 1;
    if (splits > 256) splits = 256;
    return splits;
}

// Split count of the drop-in decode, whose caller gives no budget and whose lengths are device data.  Pieces of 512 keys
// by default (default_splits); a larger piece out of the sizes measured on B200 when a wave model prefers it: a grid
// of C = batch * kv_heads * ceil(bound / piece) CTAs runs in ceil(C / slots) waves (three CTAs per SM) of piece + 200
// key-times each -- a CTA's start-up is worth about 200 keys of streaming -- with every sequence taken at the bound.
// Only choices that still make 2.5 waves compete, so that batches whose real lengths are well below the bound keep
// enough CTAs in flight.  Measured on 20 mixes (8 - 128 sequences, bounds 1024 - 8192, equal and uniformly drawn
// lengths): 3.5 % less time in total, no mix more than 1 % slower, and the 32-sequence / 4096-key shape 4 - 5 %
// faster on each of six draws of its lengths.
size_t wave_aware_splits(size_t batch, size_t kv_heads, size_t bound_tokens, size_t page) {
    const size_t base = default_splits(batch, kv_heads, bound_tokens);
    const double slots = 3.0 * static_cast<double>(device_sm_count());
    auto cost_of = [&](size_t splits, double *waves_out) {
        size_t piece = (bound_tokens + splits - 1) / splits;
        piece = (piece + page - 1) / page * page;
        const size_t live = (bound_tokens + piece - 1) / piece;
        const double waves = static_cast<double>(batch * kv_heads * live) / slots;
        if (waves_out != nullptr) *waves_out = waves;
        return std::ceil(waves) * static_cast<double>(piece + 200);
    };
    size_t best = base;
    double best_cost = cost_of(base, nullptr);
    const size_t sizes[] = {640, 832, 1024, 1360, 2048};
    for (size_t size : sizes) {
        const size_t splits = (bound_tokens + size - 1) / size;
        if (splits < 1 || splits >= base) continue;  // never finer than the default
        double waves = 0.0;
        const double cost = cost_of(splits, &waves);
        if (waves >= 2.5 && cost < best_cost) {
            best = splits;
            best_cost = cost;
        }
    }
    return best;
}

template <typename T>
int decode_general(cudaStream_t stream, void *out, const void *query, const void *key_cache, const void *value_cache,
                   const int32_t *lens, const uint32_t *table, size_t batch, size_t heads, size_t kv_heads,
                   size_t head_dim, size_t block_size, size_t physical_blocks, size_t stride, float scale) {
    DecodePagedPolicy<T> policy;
    policy.query = static_cast<const T *>(query);
    policy.out = static_cast<T *>(out);
    policy.key_cache = static_cast<const T *>(key_cache);
    policy.value_cache = static_cast<const T *>(value_cache);
    policy.lens = lens;
    policy.table = table;
    policy.heads = static_cast<int>(heads);
    policy.kv_heads = static_cast<int>(kv_heads);
    policy.head_dim = static_cast<int>(head_dim);
    policy.block_size = static_cast<int>(block_size);
    policy.physical_blocks = static_cast<long long>(physical_blocks);
    policy.stride = static_cast<long long>(stride);
    return launch_attention_general<T>(stream, policy, batch * heads, head_dim, scale, LseKind::None, 0.0f, nullptr);
}

// element: 0 bf16, 1 f16
int decode_half(cudaStream_t stream, int element, void *out, const void *query, const void *key_cache,
                const void *value_cache, const int32_t *lens, const uint32_t *table, size_t batch, size_t heads,
                size_t kv_heads, size_t head_dim, size_t block_size, size_t physical_blocks, size_t stride,
                float scale) {
    SINGE_TRY(validate_paged_decode(batch, heads, kv_heads, head_dim, block_size, physical_blocks, stride, scale));
    if (out == nullptr || query == nullptr || key_cache == nullptr || value_cache == nullptr || lens == nullptr ||
        table == nullptr) {
        return SINGE_ERR_NULL_POINTER;
    }
    // The tiled kernel puts the batch in a grid dimension of at most 65535; larger batches keep the general kernel.
    if (batch <= 65535 && paged_decode_fast_path(heads, kv_heads, head_dim, block_size, key_cache, value_cache, query)) {
        const size_t splits = wave_aware_splits(batch, kv_heads, stride * block_size, block_size);
        float *scratch = nullptr;
        const size_t rows = batch * heads * splits;
        SINGE_TRY(workspace_for(stream, rows * (head_dim + 1), &scratch));
        return paged_decode_splitk(stream, element, out, scratch, scratch + rows * head_dim, query, key_cache,
                                   value_cache, lens, table, batch, heads, kv_heads, head_dim, physical_blocks, stride,
                                   splits, scale, false, device_error_word(), nullptr, 0u, nullptr, nullptr, nullptr);
    }
    if (element == 0) {
        return decode_general<__nv_bfloat16>(stream, out, query, key_cache, value_cache, lens, table, batch, heads,
                                             kv_heads, head_dim, block_size, physical_blocks, stride, scale);
    }
    return decode_general<__half>(stream, out, query, key_cache, value_cache, lens, table, batch, heads, kv_heads,
                                  head_dim, block_size, physical_blocks, stride, scale);
}

int decode_splitk_half(cudaStream_t stream, int element, void *out, float *attn_scratch, float *lse_scratch,
                       const void *query, const void *key_cache, const void *value_cache, const int32_t *lens,
                       const uint32_t *table, size_t batch, size_t heads, size_t kv_heads, size_t head_dim,
                       size_t block_size, size_t physical_blocks, size_t stride, size_t max_splits, float scale,
                       bool partials_only, unsigned hints = 0u, const QueryRotation *rotation = nullptr,
                       uint32_t *tickets = nullptr, const FusedStep *fused = nullptr, uint32_t *status = nullptr) {
    SINGE_TRY(validate_paged_decode(batch, heads, kv_heads, head_dim, block_size, physical_blocks, stride, scale));
    if (max_splits == 0) return SINGE_ERR_INVALID_LENGTH;  // validate_fmha_decode_splitk_reduce_config, mod.rs:2553-2559
    if (!fits_i32(max_splits)) return SINGE_ERR_LENGTH_EXCEEDS_I32;
    if ((out == nullptr && !partials_only) || attn_scratch == nullptr || lse_scratch == nullptr || query == nullptr ||
        key_cache == nullptr || value_cache == nullptr || lens == nullptr || table == nullptr) {
        return SINGE_ERR_NULL_POINTER;
    }
    if (!paged_decode_fast_path(heads, kv_heads, head_dim, block_size, key_cache, value_cache, query)) {
        return SINGE_ERR_UNSUPPORTED_CONFIGURATION;
    }
    return paged_decode_splitk(stream, element, out, attn_scratch, lse_scratch, query, key_cache, value_cache, lens,
                               table, batch, heads, kv_heads, head_dim, physical_blocks, stride, max_splits, scale,
                               partials_only, status != nullptr ? status : device_error_word(), nullptr, hints, rotation,
                               tickets, fused);
}

template <typename T>
int packed_prefill_general(cudaStream_t stream, void *out, float *lse, const void *query, const void *key,
                           const void *value, const int32_t *lens_q, const int32_t *lens_kv, const int32_t *offsets,
                           const uint32_t *table, size_t batch, size_t total_q, size_t total_kv, size_t heads,
                           size_t kv_heads, size_t head_dim, size_t block_size, size_t physical_blocks, size_t stride,
                           int causal, float scale) {
    PackedPrefillPolicy<T> policy;
    policy.query = static_cast<const T *>(query);
    policy.out = static_cast<T *>(out);
    policy.lse = lse;
    policy.key = static_cast<const T *>(key);
    policy.value = static_cast<const T *>(value);
    policy.lens_q = lens_q;
    policy.lens_kv = lens_kv;
    policy.offsets = offsets;
    policy.table = table;
    policy.batch = static_cast<int>(batch);
    policy.heads = static_cast<int>(heads);
    policy.kv_heads = static_cast<int>(kv_heads);
    policy.head_dim = static_cast<int>(head_dim);
    policy.block_size = static_cast<int>(block_size);
    policy.causal = causal == 2 ? 2 : (causal ? 1 : 0);
    policy.physical_blocks = static_cast<long long>(physical_blocks);
    policy.stride = static_cast<long long>(stride);
    policy.total_query_tokens = static_cast<long long>(total_q);
    policy.total_kv_tokens = static_cast<long long>(total_kv);
    return launch_attention_general<T>(stream, policy, total_q * heads, head_dim, scale, LseKind::Natural, -1.0e20f,
                                       nullptr);
}

template <typename T, typename Index>
int tensor_paged(cudaStream_t stream, void *out, float *lse, const void *query, const void *key_cache,
                 const void *value_cache, const void *query_offsets, const void *page_offsets, const void *pages,
                 const void *last_page_lengths, size_t tokens, size_t heads, size_t kv_heads, size_t head_dim,
                 size_t page_size, size_t cache_pages, size_t sequences, size_t table_len, float scale, int causal,
                 size_t window, uint32_t *status, float softcap) {
    TensorPagedPolicy<T, Index> policy;
    policy.query = static_cast<const T *>(query);
    policy.out = static_cast<T *>(out);
    policy.lse = lse;
    policy.key_cache = static_cast<const T *>(key_cache);
    policy.value_cache = static_cast<const T *>(value_cache);
    policy.query_offsets = static_cast<const Index *>(query_offsets);
    policy.page_offsets = static_cast<const Index *>(page_offsets);
    policy.pages = static_cast<const Index *>(pages);
    policy.last_page_lengths = static_cast<const Index *>(last_page_lengths);
    policy.sequences = static_cast<int>(sequences);
    policy.heads = static_cast<int>(heads);
    policy.kv_heads = static_cast<int>(kv_heads);
    policy.head_dim = static_cast<int>(head_dim);
    policy.page_size = static_cast<int>(page_size);
    policy.causal = causal ? 1 : 0;
    policy.tokens = static_cast<long long>(tokens);
    policy.cache_pages = static_cast<long long>(cache_pages);
    policy.table_len = static_cast<long long>(table_len);
    policy.window = static_cast<long long>(window);
    policy.skip_when_zero = nullptr;
    bool checked = status == nullptr;  // no status word, no whole-table check
    auto check_alone = [&]() -> int {
        const unsigned blocks = static_cast<unsigned>((sequences + 3) / 4);  // four warps, one sequence each
        check_paged_values_kernel<Index><<<blocks > 256 ? 256 : blocks, 128, 0, stream>>>(
            policy.query_offsets, policy.page_offsets, policy.pages, policy.last_page_lengths, policy.sequences,
            policy.tokens, policy.cache_pages, policy.table_len, static_cast<long long>(page_size), status);
        return launch_status();
    };
    // One query token per sequence: possibly a plain decode batch (with or without a sliding window).  Whether it is one depends on the
    // paging tensors, which live on the device, so a planning kernel decides there: it either hands the call to
    // the tiled flash-decode kernel (and the general kernel below finds nothing to do) or leaves it to the general
    // kernel (and the tiled kernel's CTAs leave at once).
    constexpr bool kHalfType = sizeof(T) == 2;
    if (kHalfType && tokens == sequences && sequences <= 65535 &&
        paged_decode_fast_path(heads, kv_heads, head_dim, page_size, key_cache, value_cache, query)) {
        // split budget: ~512-key splits of a sequence twice the average length (the real lengths are device data)
        const size_t average = table_len * page_size / sequences;
        size_t guess = 2 * average;
        if (window > 0 && guess > window + page_size) guess = window + page_size;  // what a window leaves of a sequence
        if (guess < page_size) guess = page_size;
        const size_t splits = wave_aware_splits(sequences, kv_heads, guess, page_size);
        // pieces of at least 512 keys when that still gives the machine enough CTAs (what default_splits assumes)
        const int min_piece = sequences * kv_heads * ((guess + 511) / 512) >= static_cast<size_t>(device_sm_count()) * 4
                                  ? 512
                                  : 128;
        const size_t rows = tokens * heads * splits;
        const size_t partial_floats = rows * (head_dim + 1);
        const size_t plan_floats = 4 * sequences + 16;  // lens (int32), first (int64), control, hidden (int32)
        float *scratch = nullptr;
        const int grown = workspace_for(stream, partial_floats + plan_floats + 4, &scratch);
        if (grown == SINGE_OK) {
            // 8-byte aligned plan area behind the partials
            uintptr_t plan_at = reinterpret_cast<uintptr_t>(scratch + partial_floats);
            plan_at = (plan_at + 7u) & ~static_cast<uintptr_t>(7u);
            long long *first = reinterpret_cast<long long *>(plan_at);
            int *lens = reinterpret_cast<int *>(first + sequences);
            int *control = lens + sequences;
            int *hidden = control + 8;
            const long long window_keys = window > 0x7fffffffull ? 0x7fffffffll : static_cast<long long>(window);
            if (!checked) {
                const unsigned blocks = static_cast<unsigned>((sequences + 7) / 8);  // eight warps, one sequence each
                check_and_plan_kernel<Index><<<(blocks > 256 ? 256 : blocks) + 1, 256, 0, stream>>>(
                    policy.query_offsets, policy.page_offsets, policy.pages, policy.last_page_lengths,
                    policy.sequences, policy.tokens, policy.cache_pages, policy.table_len,
                    static_cast<long long>(page_size), status, static_cast<int>(splits), min_piece, lens, first, control,
                    window_keys, hidden);
                checked = true;
            } else {
                plan_paged_decode_kernel<Index><<<1, 256, 0, stream>>>(
                    policy.query_offsets, policy.page_offsets, policy.pages, policy.last_page_lengths,
                    policy.sequences, policy.cache_pages, policy.table_len, static_cast<long long>(page_size),
                    static_cast<int>(splits), min_piece, lens, first, control, window_keys, hidden);
            }
            SINGE_TRY(launch_status());
            RaggedDecode ragged;
            ragged.pages = pages;
            ragged.first = first;
            ragged.control = control;
            ragged.index_width = static_cast<int>(sizeof(Index));
            ragged.lse_out = lse;
            ragged.softcap = softcap;
            ragged.hidden = window > 0 ? hidden : nullptr;
            const int element = std::is_same<T, __nv_bfloat16>::value ? 0 : 1;
            SINGE_TRY(paged_decode_splitk(stream, element, out, scratch, scratch + rows * head_dim, query, key_cache,
                                          value_cache, lens, nullptr, sequences, heads, kv_heads, head_dim,
                                          cache_pages, 1, splits, scale, false,
                                          status != nullptr ? status : device_error_word(), &ragged, 0u, nullptr,
                                          nullptr, nullptr));
            policy.skip_when_zero = control;
        } else if (grown != SINGE_ERR_AUTOTUNE_DURING_CAPTURE) {
            return grown;
        }
        // (workspace growth refused under stream capture: the general kernel serves the call)
    }
    if (!checked) SINGE_TRY(check_alone());
    return launch_attention_general<T>(stream, policy, tokens * heads, head_dim, scale, LseKind::Base2, -INFINITY,
                                       status, softcap);
}

template <typename T>
int tensor_paged_entry(singe_stream_t stream, void *out, float *lse, const void *query, const void *key_cache,
                       const void *value_cache, const void *query_offsets, const void *page_offsets,
                       const void *pages, const void *last_page_lengths, int index_width, size_t tokens, size_t heads,
                       size_t kv_heads, size_t head_dim, size_t page_size, size_t cache_pages, size_t sequences,
                       size_t table_len, float scale, int causal, size_t window, uint32_t *status,
                       float softcap = 0.0f) {
    if (!(softcap >= 0.0f) || !finite(softcap)) return SINGE_ERR_INVALID_ARGUMENT;
    // paged_attention_problem (singe/src/backend/spec/neural/attention.rs:337-361)
    if (heads == 0 || kv_heads == 0 || head_dim == 0 || page_size == 0 || heads % kv_heads != 0 || !finite(scale)) {
        return SINGE_ERR_INVALID_ARGUMENT;
    }
    if (index_width != 4 && index_width != 8) return SINGE_ERR_INVALID_ARGUMENT;
    if (!fits_i32(tokens) || !fits_i32(heads) || !fits_i32(head_dim) || !fits_i32(page_size) ||
        !fits_i32(cache_pages) || !fits_i32(sequences) || !fits_i32(table_len)) {
        return SINGE_ERR_LENGTH_EXCEEDS_I32;
    }
    if (tokens == 0 || sequences == 0) return SINGE_OK;
    if (out == nullptr || lse == nullptr || query == nullptr || key_cache == nullptr || value_cache == nullptr ||
        query_offsets == nullptr || page_offsets == nullptr || last_page_lengths == nullptr ||
        (pages == nullptr && table_len != 0)) {
        return SINGE_ERR_NULL_POINTER;
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (index_width == 8) {
        return tensor_paged<T, long long>(s, out, lse, query, key_cache, value_cache, query_offsets, page_offsets,
                                          pages, last_page_lengths, tokens, heads, kv_heads, head_dim, page_size,
                                          cache_pages, sequences, table_len, scale, causal, window, status, softcap);
    }
    return tensor_paged<T, int>(s, out, lse, query, key_cache, value_cache, query_offsets, page_offsets, pages,
                                last_page_lengths, tokens, heads, kv_heads, head_dim, page_size, cache_pages, sequences,
                                table_len, scale, causal, window, status, softcap);
}

template <typename T>
int dense_entry(cudaStream_t stream, T *out, float *lse, const T *query, const T *key, const T *value, size_t batch,
                size_t heads, size_t kv_heads, size_t query_len, size_t key_len, size_t head_dim, float scale,
                int causal, size_t window, bool bshd, float softcap = 0.0f, const T *sinks = nullptr) {
    if (batch == 0 || heads == 0 || kv_heads == 0 || query_len == 0 || key_len == 0 || head_dim == 0 ||
        heads % kv_heads != 0 || !finite(scale)) {
        return SINGE_ERR_INVALID_LENGTH;
    }
    if (!fits_i32(batch) || !fits_i32(heads) || !fits_i32(query_len) || !fits_i32(key_len) || !fits_i32(head_dim)) {
        return SINGE_ERR_LENGTH_EXCEEDS_I32;
    }
    if (out == nullptr || query == nullptr || key == nullptr || value == nullptr) return SINGE_ERR_NULL_POINTER;
    if (!(softcap >= 0.0f) || !finite(softcap)) return SINGE_ERR_INVALID_ARGUMENT;
    DensePolicy<T> policy;
    policy.sinks = sinks;
    policy.query = query;
    policy.out = out;
    policy.lse = lse;
    policy.key = key;
    policy.value = value;
    policy.heads = static_cast<int>(heads);
    policy.kv_heads = static_cast<int>(kv_heads);
    policy.query_len = static_cast<int>(query_len);
    policy.key_len = static_cast<int>(key_len);
    policy.head_dim = static_cast<int>(head_dim);
    policy.causal = causal ? 1 : 0;
    policy.window = static_cast<long long>(window);
    const long long d = static_cast<long long>(head_dim);
    if (bshd) {
        policy.q_batch = static_cast<long long>(query_len) * heads * d;
        policy.q_head = d;
        policy.q_row = static_cast<long long>(heads) * d;
        policy.k_batch = static_cast<long long>(key_len) * kv_heads * d;
        policy.k_head = d;
        policy.k_row = static_cast<long long>(kv_heads) * d;
    } else {
        policy.q_batch = static_cast<long long>(heads) * query_len * d;
        policy.q_head = static_cast<long long>(query_len) * d;
        policy.q_row = d;
        policy.k_batch = static_cast<long long>(kv_heads) * key_len * d;
        policy.k_head = static_cast<long long>(key_len) * d;
        policy.k_row = d;
    }
    policy.lse_batch = static_cast<long long>(heads) * query_len;
    policy.lse_head = static_cast<long long>(query_len);
    policy.lse_row = 1;
    return launch_attention_general<T>(stream, policy, batch * heads * query_len, head_dim, scale,
                                       lse == nullptr ? LseKind::None : LseKind::Natural, -INFINITY, nullptr, softcap);
}

// splitk_reduce_f32 (singe-kernel/src/cpu/attention.rs:2157-2193) with SplitKReduceConfig strides.
__global__ void splitk_reduce_kernel(float *out, const float *attn, const float *lse, int heads, int splits,
                                     int head_dim, long long attn_batch, long long attn_head, long long attn_split,
                                     long long lse_batch, long long lse_head, long long out_batch, long long out_head) {
    const int b = blockIdx.y;
    const int head = blockIdx.x;
    const float *row_lse = lse + b * lse_batch + head * lse_head;
    float top = -INFINITY;
    for (int s = 0; s < splits; ++s) top = fmaxf(top, row_lse[s]);
    float denom = 0.0f;
    for (int s = 0; s < splits; ++s) denom += expf(row_lse[s] - top);
    const float *row_attn = attn + b * attn_batch + head * attn_head;
    for (int d = threadIdx.x; d < head_dim; d += blockDim.x) {
        float sum = 0.0f;
        for (int s = 0; s < splits; ++s) {
            sum = fmaf(expf(row_lse[s] - top), row_attn[s * attn_split + d], sum);
        }
        out[b * out_batch + head * out_head + d] = sum / denom;
    }
}

}  // namespace
}  // namespace singe

using namespace singe;

extern "C" {

int singe_kernel_sys_version(void) { return 1001; }

int singe_release_workspaces(void) { return release_workspaces(); }

const char *singe_status_string(int status) {
    switch (status) {
        case SINGE_OK: return "ok";
        case SINGE_ERR_INVALID_LENGTH: return "invalid length";
        case SINGE_ERR_LENGTH_TOO_SHORT: return "length too short";
        case SINGE_ERR_LENGTH_EXCEEDS_I32: return "length exceeds i32";
        case SINGE_ERR_NULL_POINTER: return "null pointer";
        case SINGE_ERR_SIZE_OVERFLOW: return "size overflow";
        case SINGE_ERR_UNSUPPORTED_WIDTH: return "unsupported width";
        case SINGE_ERR_UNSUPPORTED_CONFIGURATION: return "unsupported configuration";
        case SINGE_ERR_LENGTH_MISMATCH: return "length mismatch";
        case SINGE_ERR_INDEX_OUT_OF_BOUNDS: return "index out of bounds";
        case SINGE_ERR_INVALID_ARGUMENT: return "invalid argument";
        case SINGE_ERR_OUT_OF_RANGE: return "out of range";
        case SINGE_ERR_AUTOTUNE_DURING_CAPTURE: return "workspace growth during cuda graph capture";
        case SINGE_ERR_STATIC_SCRATCH_EXCEEDED: return "problem exceeds the library's fixed scratch array";
        default: return status >= SINGE_ERR_CUDA_BASE ? "cuda runtime error" : "unknown status";
    }
}

int singe_kv_cache_write_bf16(singe_stream_t stream, void *key_cache, void *value_cache, const void *keys,
                              const void *values, const void *write_pages, const void *write_slots, int index_width,
                              size_t tokens, size_t kv_heads, size_t head_dim, size_t pages, size_t page_size,
                              uint32_t *status) {
    return kv_cache_write(static_cast<cudaStream_t>(stream), key_cache, value_cache, keys, values, write_pages,
                          write_slots, index_width, tokens, kv_heads, head_dim, pages, page_size, status, 2);
}

int singe_kv_cache_write_f16(singe_stream_t stream, void *key_cache, void *value_cache, const void *keys,
                             const void *values, const void *write_pages, const void *write_slots, int index_width,
                             size_t tokens, size_t kv_heads, size_t head_dim, size_t pages, size_t page_size,
                             uint32_t *status) {
    return kv_cache_write(static_cast<cudaStream_t>(stream), key_cache, value_cache, keys, values, write_pages,
                          write_slots, index_width, tokens, kv_heads, head_dim, pages, page_size, status, 2);
}

int singe_kv_cache_write_f32(singe_stream_t stream, void *key_cache, void *value_cache, const void *keys,
                             const void *values, const void *write_pages, const void *write_slots, int index_width,
                             size_t tokens, size_t kv_heads, size_t head_dim, size_t pages, size_t page_size,
                             uint32_t *status) {
    return kv_cache_write(static_cast<cudaStream_t>(stream), key_cache, value_cache, keys, values, write_pages,
                          write_slots, index_width, tokens, kv_heads, head_dim, pages, page_size, status, 4);
}

int singe_paged_kv_decode_attention_bf16(singe_stream_t stream, void *out, const void *query, const void *key_cache,
                                         const void *value_cache, const int32_t *actual_seq_lens,
                                         const uint32_t *block_table, size_t batch, size_t heads, size_t kv_heads,
                                         size_t head_dim, size_t block_size, size_t physical_blocks,
                                         size_t block_table_batch_stride, float scale) {
    return decode_half(static_cast<cudaStream_t>(stream), 0, out, query, key_cache, value_cache, actual_seq_lens,
                       block_table, batch, heads, kv_heads, head_dim, block_size, physical_blocks,
                       block_table_batch_stride, scale);
}

int singe_paged_kv_decode_attention_f16(singe_stream_t stream, void *out, const void *query, const void *key_cache,
                                        const void *value_cache, const int32_t *actual_seq_lens,
                                        const uint32_t *block_table, size_t batch, size_t heads, size_t kv_heads,
                                        size_t head_dim, size_t block_size, size_t physical_blocks,
                                        size_t block_table_batch_stride, float scale) {
    return decode_half(static_cast<cudaStream_t>(stream), 1, out, query, key_cache, value_cache, actual_seq_lens,
                       block_table, batch, heads, kv_heads, head_dim, block_size, physical_blocks,
                       block_table_batch_stride, scale);
}

int singe_paged_kv_decode_attention_f32(singe_stream_t stream, float *out, const float *query, const float *key_cache,
                                        const float *value_cache, const int32_t *actual_seq_lens,
                                        const uint32_t *block_table, size_t batch, size_t heads, size_t kv_heads,
                                        size_t head_dim, size_t block_size, size_t physical_blocks,
                                        size_t block_table_batch_stride, float scale) {
    SINGE_TRY(validate_paged_decode(batch, heads, kv_heads, head_dim, block_size, physical_blocks,
                                    block_table_batch_stride, scale));
    if (out == nullptr || query == nullptr || key_cache == nullptr || value_cache == nullptr ||
        actual_seq_lens == nullptr || block_table == nullptr) {
        return SINGE_ERR_NULL_POINTER;
    }
    return decode_general<float>(static_cast<cudaStream_t>(stream), out, query, key_cache, value_cache,
                                 actual_seq_lens, block_table, batch, heads, kv_heads, head_dim, block_size,
                                 physical_blocks, block_table_batch_stride, scale);
}

size_t singe_paged_kv_decode_default_splits(size_t batch, size_t kv_heads, size_t key_len_bound, size_t block_size) {
    if (batch == 0 || kv_heads == 0 || key_len_bound == 0 || block_size == 0) return 1;
    return wave_aware_splits(batch, kv_heads, key_len_bound, block_size);
}

size_t singe_paged_kv_decode_split_tokens(size_t key_len_bound, size_t max_splits, size_t block_size) {
    return paged_decode_split_tokens(key_len_bound, max_splits, block_size);
}

int singe_paged_kv_decode_splitk_bf16(singe_stream_t stream, float *attn_scratch, float *lse_scratch,
                                      const void *query, const void *key_cache, const void *value_cache,
                                      const int32_t *actual_seq_lens, const uint32_t *block_table, size_t batch,
                                      size_t heads, size_t kv_heads, size_t head_dim, size_t block_size,
                                      size_t physical_blocks, size_t block_table_batch_stride, size_t max_splits,
                                      float scale) {
    return decode_splitk_half(static_cast<cudaStream_t>(stream), 0, nullptr, attn_scratch, lse_scratch, query,
                              key_cache, value_cache, actual_seq_lens, block_table, batch, heads, kv_heads, head_dim,
                              block_size, physical_blocks, block_table_batch_stride, max_splits, scale, true);
}

int singe_paged_kv_decode_splitk_reduce_bf16(singe_stream_t stream, void *out, float *attn_scratch,
                                             float *lse_scratch, const void *query, const void *key_cache,
                                             const void *value_cache, const int32_t *actual_seq_lens,
                                             const uint32_t *block_table, size_t batch, size_t heads, size_t kv_heads,
                                             size_t head_dim, size_t block_size, size_t physical_blocks,
                                             size_t block_table_batch_stride, size_t max_splits, float scale) {
    return decode_splitk_half(static_cast<cudaStream_t>(stream), 0, out, attn_scratch, lse_scratch, query, key_cache,
                              value_cache, actual_seq_lens, block_table, batch, heads, kv_heads, head_dim, block_size,
                              physical_blocks, block_table_batch_stride, max_splits, scale, false);
}

int singe_paged_kv_decode_step_bf16(singe_stream_t stream, void *out, float *attn_scratch, float *lse_scratch,
                                    const void *query, const void *key_cache, const void *value_cache,
                                    const int32_t *actual_seq_lens, const uint32_t *block_table, size_t batch,
                                    size_t heads, size_t kv_heads, size_t head_dim, size_t block_size,
                                    size_t physical_blocks, size_t block_table_batch_stride, size_t max_splits,
                                    float scale, unsigned hints, uint32_t *tickets) {
    return decode_splitk_half(static_cast<cudaStream_t>(stream), 0, out, attn_scratch, lse_scratch, query, key_cache,
                              value_cache, actual_seq_lens, block_table, batch, heads, kv_heads, head_dim, block_size,
                              physical_blocks, block_table_batch_stride, max_splits, scale, false, hints, nullptr,
                              tickets);
}

int singe_rotary_paged_kv_decode_attention_bf16(singe_stream_t stream, void *out, float *attn_scratch,
                                                float *lse_scratch, const void *query, const void *key_cache,
                                                const void *value_cache, const int32_t *actual_seq_lens,
                                                const uint32_t *block_table, const void *cos_table,
                                                const void *sin_table, const void *positions, int index_width,
                                                size_t batch, size_t heads, size_t kv_heads, size_t head_dim,
                                                size_t block_size, size_t physical_blocks,
                                                size_t block_table_batch_stride, size_t max_splits, size_t capacity,
                                                float scale, int normalise_query, const void *query_norm_weight,
                                                float eps, unsigned hints) {
    if (cos_table == nullptr || sin_table == nullptr || positions == nullptr) return SINGE_ERR_NULL_POINTER;
    if (index_width != 4 && index_width != 8) return SINGE_ERR_INVALID_ARGUMENT;
    if (capacity == 0) return SINGE_ERR_INVALID_LENGTH;
    if (!fits_i32(capacity)) return SINGE_ERR_LENGTH_EXCEEDS_I32;
    if (((reinterpret_cast<uintptr_t>(cos_table) | reinterpret_cast<uintptr_t>(sin_table) |
          reinterpret_cast<uintptr_t>(query_norm_weight)) & 3u) != 0) {
        return SINGE_ERR_INVALID_ARGUMENT;
    }
    QueryRotation rotation;
    rotation.cos = cos_table;
    rotation.sin = sin_table;
    rotation.positions = positions;
    rotation.index_width = index_width;
    rotation.capacity = static_cast<int>(capacity);
    rotation.gain = query_norm_weight;
    rotation.normalise = normalise_query != 0 ? 1 : 0;
    rotation.eps = eps;
    return decode_splitk_half(static_cast<cudaStream_t>(stream), 0, out, attn_scratch, lse_scratch, query, key_cache,
                              value_cache, actual_seq_lens, block_table, batch, heads, kv_heads, head_dim, block_size,
                              physical_blocks, block_table_batch_stride, max_splits, scale, false, hints, &rotation);
}

int singe_decode_step_attention_bf16(singe_stream_t stream, void *out, float *attn_scratch, float *lse_scratch,
                                     const void *qkv, size_t qkv_row_stride, void *key_cache, void *value_cache,
                                     const int32_t *actual_seq_lens, const uint32_t *block_table,
                                     const void *cos_table, const void *sin_table, const void *positions,
                                     const void *write_pages, const void *write_slots, int index_width, size_t batch,
                                     size_t heads, size_t kv_heads, size_t head_dim, size_t block_size,
                                     size_t physical_blocks, size_t block_table_batch_stride, size_t max_splits,
                                     size_t capacity, float scale, unsigned hints, uint32_t *tickets,
                                     uint32_t *status) {
    if (qkv == nullptr || cos_table == nullptr || sin_table == nullptr || positions == nullptr ||
        write_pages == nullptr || write_slots == nullptr) {
        return SINGE_ERR_NULL_POINTER;
    }
    if (index_width != 4 && index_width != 8) return SINGE_ERR_INVALID_ARGUMENT;
    if (capacity == 0 || qkv_row_stride < (heads + 2 * kv_heads) * head_dim) return SINGE_ERR_INVALID_LENGTH;
    if (!fits_i32(capacity) || !fits_i32(qkv_row_stride)) return SINGE_ERR_LENGTH_EXCEEDS_I32;
    if (((reinterpret_cast<uintptr_t>(cos_table) | reinterpret_cast<uintptr_t>(sin_table) |
          reinterpret_cast<uintptr_t>(qkv)) & 3u) != 0 || qkv_row_stride % 2 != 0) {
        return SINGE_ERR_INVALID_ARGUMENT;
    }
    QueryRotation rotation;
    rotation.cos = cos_table;
    rotation.sin = sin_table;
    rotation.positions = positions;
    rotation.index_width = index_width;
    rotation.capacity = static_cast<int>(capacity);
    rotation.gain = nullptr;
    rotation.normalise = 0;
    rotation.eps = 0.0f;
    FusedStep fused;
    fused.qkv = qkv;
    fused.qkv_stride = static_cast<long long>(qkv_row_stride);
    fused.write_pages = write_pages;
    fused.write_slots = write_slots;
    return decode_splitk_half(static_cast<cudaStream_t>(stream), 0, out, attn_scratch, lse_scratch, qkv, key_cache,
                              value_cache, actual_seq_lens, block_table, batch, heads, kv_heads, head_dim, block_size,
                              physical_blocks, block_table_batch_stride, max_splits, scale, false, hints, &rotation,
                              tickets, &fused, status);
}

int singe_paged_kv_decode_set_prefetch(int pages) {
    if (pages < 0 || pages > 4096) return SINGE_ERR_INVALID_ARGUMENT;
    g_decode_prefetch_pages = pages;
    return SINGE_OK;
}

int singe_paged_kv_decode_splitk_reduce_f16(singe_stream_t stream, void *out, float *attn_scratch, float *lse_scratch,
                                            const void *query, const void *key_cache, const void *value_cache,
                                            const int32_t *actual_seq_lens, const uint32_t *block_table, size_t batch,
                                            size_t heads, size_t kv_heads, size_t head_dim, size_t block_size,
                                            size_t physical_blocks, size_t block_table_batch_stride,
                                            size_t max_splits, float scale) {
    return decode_splitk_half(static_cast<cudaStream_t>(stream), 1, out, attn_scratch, lse_scratch, query, key_cache,
                              value_cache, actual_seq_lens, block_table, batch, heads, kv_heads, head_dim, block_size,
                              physical_blocks, block_table_batch_stride, max_splits, scale, false);
}

int singe_splitk_reduce_f32(singe_stream_t stream, float *out, const float *attn_splitk, const float *lse_splitk,
                            size_t batch, size_t heads, size_t splits, size_t head_dim, size_t attn_batch_stride,
                            size_t attn_head_stride, size_t attn_split_stride, size_t lse_batch_stride,
                            size_t lse_head_stride, size_t output_batch_stride, size_t output_head_stride) {
    // validate_splitk_reduce_config (singe-kernel/src/cuda/attention/mod.rs): every extent non-zero and within i32.
    if (batch == 0 || heads == 0 || splits == 0 || head_dim == 0) return SINGE_ERR_INVALID_LENGTH;
    if (attn_split_stride < head_dim || attn_head_stride < splits * attn_split_stride - (attn_split_stride - head_dim) ||
        lse_head_stride < splits || output_head_stride < head_dim) {
        return SINGE_ERR_INVALID_LENGTH;
    }
    if (!fits_i32(batch) || !fits_i32(heads) || !fits_i32(splits) || !fits_i32(head_dim)) {
        return SINGE_ERR_LENGTH_EXCEEDS_I32;
    }
    if (out == nullptr || attn_splitk == nullptr || lse_splitk == nullptr) return SINGE_ERR_NULL_POINTER;
    if (batch > 65535) return SINGE_ERR_UNSUPPORTED_CONFIGURATION;
    dim3 grid(static_cast<unsigned>(heads), static_cast<unsigned>(batch));
    splitk_reduce_kernel<<<grid, 128, 0, static_cast<cudaStream_t>(stream)>>>(
        out, attn_splitk, lse_splitk, static_cast<int>(heads), static_cast<int>(splits), static_cast<int>(head_dim),
        static_cast<long long>(attn_batch_stride), static_cast<long long>(attn_head_stride),
        static_cast<long long>(attn_split_stride), static_cast<long long>(lse_batch_stride),
        static_cast<long long>(lse_head_stride), static_cast<long long>(output_batch_stride),
        static_cast<long long>(output_head_stride));
    return launch_status();
}

// fmha_decode_splitk_reduce_f32 with FmhaDecodeSplitKReduceConfig::contiguous
// (singe-kernel/src/cuda/attention/fmha.rs:1155-1241, mod.rs:454-477,2511-2560): the decode over contiguous keys and
// values cut into min(max_splits, key_len) key ranges, then the log-sum-exp fold.
int singe_fmha_decode_splitk_reduce_f32(singe_stream_t stream, float *out, float *attn_scratch, float *lse_scratch,
                                        const float *query, const float *key, const float *value, size_t batch,
                                        size_t key_len, size_t heads, size_t kv_heads, size_t head_dim,
                                        size_t max_splits, float scale) {
    if (batch == 0 || key_len == 0 || heads == 0 || kv_heads == 0 || head_dim == 0 || max_splits == 0 ||
        heads % kv_heads != 0 || !finite(scale)) {
        return SINGE_ERR_INVALID_LENGTH;
    }
    if (!fits_i32(batch) || !fits_i32(key_len) || !fits_i32(heads) || !fits_i32(head_dim) ||
        !fits_i32(batch * heads) || !fits_i32(key_len * kv_heads) || !fits_i32(key_len * kv_heads * head_dim)) {
        return SINGE_ERR_LENGTH_EXCEEDS_I32;  // (each product is checked before it becomes a factor of the next)
    }
    if (out == nullptr || attn_scratch == nullptr || lse_scratch == nullptr || query == nullptr || key == nullptr ||
        value == nullptr) {
        return SINGE_ERR_NULL_POINTER;
    }
    const size_t splits = max_splits < key_len ? max_splits : key_len;
    if (!fits_i32(splits) || !fits_i32(batch * heads * splits)) return SINGE_ERR_LENGTH_EXCEEDS_I32;
    DenseSplitPolicy<float> policy;
    policy.query = query;
    policy.out = attn_scratch;
    policy.lse = lse_scratch;
    policy.key = key;
    policy.value = value;
    policy.heads = static_cast<int>(heads);
    policy.kv_heads = static_cast<int>(kv_heads);
    policy.key_len = static_cast<int>(key_len);
    policy.head_dim = static_cast<int>(head_dim);
    policy.splits = static_cast<int>(splits);
    policy.per_split = static_cast<int>((key_len + splits - 1) / splits);
    SINGE_TRY(launch_attention_general<float>(static_cast<cudaStream_t>(stream), policy, batch * heads * splits, head_dim,
                                              scale, LseKind::Natural, -1.0e20f, nullptr));
    return singe_splitk_reduce_f32(stream, out, attn_scratch, lse_scratch, batch, heads, splits, head_dim,
                                   heads * splits * head_dim, splits * head_dim, head_dim, heads * splits, splits,
                                   heads * head_dim, head_dim);
}

int singe_paged_attention_bf16(singe_stream_t stream, void *out, float *lse, const void *query, const void *key_cache,
                               const void *value_cache, const void *query_offsets, const void *page_offsets,
                               const void *pages, const void *last_page_lengths, int index_width, size_t tokens,
                               size_t heads, size_t kv_heads, size_t head_dim, size_t page_size, size_t cache_pages,
                               size_t sequences, size_t table_len, float scale, int causal, size_t window,
                               uint32_t *status) {
    return tensor_paged_entry<__nv_bfloat16>(stream, out, lse, query, key_cache, value_cache, query_offsets,
                                             page_offsets, pages, last_page_lengths, index_width, tokens, heads,
                                             kv_heads, head_dim, page_size, cache_pages, sequences, table_len, scale,
                                             causal, window, status);
}

int singe_paged_attention_f32(singe_stream_t stream, float *out, float *lse, const float *query,
                              const float *key_cache, const float *value_cache, const void *query_offsets,
                              const void *page_offsets, const void *pages, const void *last_page_lengths,
                              int index_width, size_t tokens, size_t heads, size_t kv_heads, size_t head_dim,
                              size_t page_size, size_t cache_pages, size_t sequences, size_t table_len, float scale,
                              int causal, size_t window, uint32_t *status) {
    return tensor_paged_entry<float>(stream, out, lse, query, key_cache, value_cache, query_offsets, page_offsets,
                                     pages, last_page_lengths, index_width, tokens, heads, kv_heads, head_dim,
                                     page_size, cache_pages, sequences, table_len, scale, causal, window, status);
}

// Tensor::paged_attention with every AttentionOptions field the path has: window and softcap.
int singe_paged_attention_options_bf16(singe_stream_t stream, void *out, float *lse, const void *query,
                                       const void *key_cache, const void *value_cache, const void *query_offsets,
                                       const void *page_offsets, const void *pages, const void *last_page_lengths,
                                       int index_width, size_t tokens, size_t heads, size_t kv_heads, size_t head_dim,
                                       size_t page_size, size_t cache_pages, size_t sequences, size_t table_len,
                                       float scale, int causal, size_t window, float softcap, uint32_t *status) {
    return tensor_paged_entry<__nv_bfloat16>(stream, out, lse, query, key_cache, value_cache, query_offsets,
                                             page_offsets, pages, last_page_lengths, index_width, tokens, heads,
                                             kv_heads, head_dim, page_size, cache_pages, sequences, table_len, scale,
                                             causal, window, status, softcap);
}

int singe_paged_attention_options_f32(singe_stream_t stream, float *out, float *lse, const float *query,
                                      const float *key_cache, const float *value_cache, const void *query_offsets,
                                      const void *page_offsets, const void *pages, const void *last_page_lengths,
                                      int index_width, size_t tokens, size_t heads, size_t kv_heads, size_t head_dim,
                                      size_t page_size, size_t cache_pages, size_t sequences, size_t table_len,
                                      float scale, int causal, size_t window, float softcap, uint32_t *status) {
    return tensor_paged_entry<float>(stream, out, lse, query, key_cache, value_cache, query_offsets, page_offsets,
                                     pages, last_page_lengths, index_width, tokens, heads, kv_heads, head_dim,
                                     page_size, cache_pages, sequences, table_len, scale, causal, window, status,
                                     softcap);
}

// Tensor::attend with window, softcap and sinks.
int singe_attend_f32(singe_stream_t stream, float *out, const float *query, const float *key, const float *value,
                     size_t batch, size_t heads, size_t kv_heads, size_t query_len, size_t key_len, size_t head_dim,
                     float scale, int causal, size_t window, float softcap, const float *sinks) {
    return dense_entry<float>(static_cast<cudaStream_t>(stream), out, nullptr, query, key, value, batch, heads,
                              kv_heads, query_len, key_len, head_dim, scale, causal, window, false, softcap, sinks);
}

// bf16 / f16, head_dim 128, 16-token pages: the tcgen05 prefill kernel gathers its K/V tiles through the block table.
// Returns true when it took the call (its status is then in *status).  kind: 0 f32, 1 bf16, 2 f16.
static bool paged_prefill_tensor_core(int kind, singe_stream_t stream, void *out, float *lse, const void *query, const void *key_cache,
                               const void *value_cache, const int32_t *lens_q, const int32_t *lens_kv,
                               const int32_t *offsets, const uint32_t *block_table, size_t batch,
                               size_t total_query_tokens, size_t heads, size_t kv_heads, size_t head_dim,
                               size_t block_size, size_t physical_blocks, size_t stride, int causal, float scale,
                               int *status) {
    if (kind == 0 || block_size != 16 ||
        !prefill_fast_path(heads, kv_heads, head_dim, total_query_tokens, query, key_cache, value_cache, out)) {
        return false;
    }
    *status = singe::prefill_tcgen05(static_cast<cudaStream_t>(stream), kind == 2, out, lse, query, key_cache,
                                     value_cache, lens_q, lens_kv, offsets, batch, total_query_tokens, 0, heads,
                                     kv_heads, head_dim, causal, scale, block_table, stride, physical_blocks, 0, 0);
    return true;
}

#define SINGE_PAGED_PREFILL(NAME, T, POINTER)                                                                         \
    int NAME(singe_stream_t stream, POINTER *out, float *lse, const POINTER *query, const POINTER *key_cache,         \
             const POINTER *value_cache, const int32_t *actual_seq_lens_q, const int32_t *actual_seq_lens_kv,         \
             const int32_t *actual_seq_offsets, const uint32_t *block_table, size_t batch,                            \
             size_t total_query_tokens, size_t heads, size_t kv_heads, size_t head_dim, size_t block_size,            \
             size_t physical_blocks, size_t block_table_batch_stride, int causal, float scale) {                      \
        SINGE_TRY(validate_paged_prefill(batch, total_query_tokens, heads, kv_heads, head_dim, block_size,            \
                                         physical_blocks, block_table_batch_stride, scale));                          \
        if (out == nullptr || lse == nullptr || query == nullptr || key_cache == nullptr || value_cache == nullptr || \
            actual_seq_lens_q == nullptr || actual_seq_lens_kv == nullptr || actual_seq_offsets == nullptr ||         \
            block_table == nullptr) {                                                                                 \
            return SINGE_ERR_NULL_POINTER;                                                                            \
        }                                                                                                             \
        int tensor_core_status = SINGE_OK;                                                                            \
        if (paged_prefill_tensor_core(std::is_same<T, __nv_bfloat16>::value ? 1 : (std::is_same<T, __half>::value ? 2 : 0), stream, out, lse, query, key_cache, value_cache, actual_seq_lens_q,          \
                                         actual_seq_lens_kv, actual_seq_offsets, block_table, batch,                  \
                                         total_query_tokens, heads, kv_heads, head_dim, block_size, physical_blocks,  \
                                         block_table_batch_stride, causal, scale, &tensor_core_status)) {             \
            return tensor_core_status;                                                                                \
        }                                                                                                             \
        return packed_prefill_general<T>(static_cast<cudaStream_t>(stream), out, lse, query, key_cache, value_cache,  \
                                         actual_seq_lens_q, actual_seq_lens_kv, actual_seq_offsets, block_table,      \
                                         batch, total_query_tokens, 0, heads, kv_heads, head_dim, block_size,         \
                                         physical_blocks, block_table_batch_stride, causal, scale);                   \
    }

SINGE_PAGED_PREFILL(singe_paged_kv_prefill_attention_bf16, __nv_bfloat16, void)
SINGE_PAGED_PREFILL(singe_paged_kv_prefill_attention_f16, __half, void)
SINGE_PAGED_PREFILL(singe_paged_kv_prefill_attention_f32, float, float)
#undef SINGE_PAGED_PREFILL

int singe_ragged_kv_prefill_attention_f32(singe_stream_t stream, float *out, float *lse, const float *query,
                                          const float *key, const float *value, const int32_t *actual_seq_lens_q,
                                          const int32_t *actual_seq_lens_kv, const int32_t *actual_seq_offsets,
                                          size_t batch, size_t total_query_tokens, size_t total_kv_tokens,
                                          size_t heads, size_t kv_heads, size_t head_dim, int causal, float scale) {
    SINGE_TRY(validate_ragged_prefill(batch, total_query_tokens, total_kv_tokens, heads, kv_heads, head_dim, scale));
    if (out == nullptr || lse == nullptr || query == nullptr || key == nullptr || value == nullptr ||
        actual_seq_lens_q == nullptr || actual_seq_lens_kv == nullptr || actual_seq_offsets == nullptr) {
        return SINGE_ERR_NULL_POINTER;
    }
    return packed_prefill_general<float>(static_cast<cudaStream_t>(stream), out, lse, query, key, value,
                                         actual_seq_lens_q, actual_seq_lens_kv, actual_seq_offsets, nullptr, batch,
                                         total_query_tokens, total_kv_tokens, heads, kv_heads, head_dim, 1, 1, 1,
                                         causal, scale);
}

}  // extern "C"

template <typename T>
static int ragged_prefill_16bit(singe_stream_t stream, void *out, float *lse, const void *query, const void *key,
                                const void *value, const int32_t *actual_seq_lens_q,
                                const int32_t *actual_seq_lens_kv, const int32_t *actual_seq_offsets, size_t batch,
                                size_t total_query_tokens, size_t total_kv_tokens, size_t heads, size_t kv_heads,
                                size_t head_dim, int causal, float scale) {
    SINGE_TRY(validate_ragged_prefill(batch, total_query_tokens, total_kv_tokens, heads, kv_heads, head_dim, scale));
    if (out == nullptr || lse == nullptr || query == nullptr || key == nullptr || value == nullptr ||
        actual_seq_lens_q == nullptr || actual_seq_lens_kv == nullptr || actual_seq_offsets == nullptr) {
        return SINGE_ERR_NULL_POINTER;
    }
    if (prefill_fast_path(heads, kv_heads, head_dim, total_query_tokens, query, key, value, out)) {
        return prefill_tcgen05(static_cast<cudaStream_t>(stream), std::is_same<T, __half>::value, out, lse, query, key,
                               value, actual_seq_lens_q, actual_seq_lens_kv, actual_seq_offsets, batch,
                               total_query_tokens, total_kv_tokens, heads, kv_heads, head_dim, causal, scale, nullptr,
                               0, 0, 0, 0);
    }
    return packed_prefill_general<T>(static_cast<cudaStream_t>(stream), out, lse, query, key, value,
                                     actual_seq_lens_q, actual_seq_lens_kv, actual_seq_offsets, nullptr, batch,
                                     total_query_tokens, total_kv_tokens, heads, kv_heads, head_dim, 1, 1, 1, causal,
                                     scale);
}

extern "C" {

int singe_ragged_kv_prefill_attention_bf16(singe_stream_t stream, void *out, float *lse, const void *query,
                                           const void *key, const void *value, const int32_t *actual_seq_lens_q,
                                           const int32_t *actual_seq_lens_kv, const int32_t *actual_seq_offsets,
                                           size_t batch, size_t total_query_tokens, size_t total_kv_tokens,
                                           size_t heads, size_t kv_heads, size_t head_dim, int causal, float scale) {
    return ragged_prefill_16bit<__nv_bfloat16>(stream, out, lse, query, key, value, actual_seq_lens_q,
                                               actual_seq_lens_kv, actual_seq_offsets, batch, total_query_tokens,
                                               total_kv_tokens, heads, kv_heads, head_dim, causal, scale);
}

int singe_ragged_kv_prefill_attention_f16(singe_stream_t stream, void *out, float *lse, const void *query,
                                          const void *key, const void *value, const int32_t *actual_seq_lens_q,
                                          const int32_t *actual_seq_lens_kv, const int32_t *actual_seq_offsets,
                                          size_t batch, size_t total_query_tokens, size_t total_kv_tokens,
                                          size_t heads, size_t kv_heads, size_t head_dim, int causal, float scale) {
    return ragged_prefill_16bit<__half>(stream, out, lse, query, key, value, actual_seq_lens_q, actual_seq_lens_kv,
                                        actual_seq_offsets, batch, total_query_tokens, total_kv_tokens, heads,
                                        kv_heads, head_dim, causal, scale);
}

int singe_ragged_kv_prefill_attention_cache_write_bf16(
    singe_stream_t stream, void *out, float *lse, const void *query, const void *key, const void *value,
    const int32_t *actual_seq_lens_q, const int32_t *actual_seq_lens_kv, const int32_t *actual_seq_offsets,
    size_t batch, size_t total_query_tokens, size_t total_kv_tokens, size_t heads, size_t kv_heads, size_t head_dim,
    int causal, float scale, void *key_cache, void *value_cache, const void *write_pages, const void *write_slots,
    int index_width, size_t pages, size_t page_size, uint32_t *status) {
    // The cache write is pure HBM copy and the attention is tensor-bound: they are enqueued back to back on the
    // caller's stream so one call performs the prompt step's KvCache::write + attention.
    SINGE_TRY(kv_cache_write(static_cast<cudaStream_t>(stream), key_cache, value_cache, key, value, write_pages,
                             write_slots, index_width, total_kv_tokens, kv_heads, head_dim, pages, page_size, status,
                             2));
    return singe_ragged_kv_prefill_attention_bf16(stream, out, lse, query, key, value, actual_seq_lens_q,
                                                  actual_seq_lens_kv, actual_seq_offsets, batch, total_query_tokens,
                                                  total_kv_tokens, heads, kv_heads, head_dim, causal, scale);
}

int singe_fmha_prefill_lse_f32(singe_stream_t stream, float *out, float *lse, const float *query, const float *key,
                               const float *value, size_t batch, size_t query_len, size_t key_len, size_t heads,
                               size_t kv_heads, size_t head_dim, float scale, int causal) {
    if (lse == nullptr) return SINGE_ERR_NULL_POINTER;
    return dense_entry<float>(static_cast<cudaStream_t>(stream), out, lse, query, key, value, batch, heads, kv_heads,
                              query_len, key_len, head_dim, scale, causal, 0, true);
}

}  // extern "C"

// fmha_prefill_lse over 16-bit floats: [B, L, H, 128] queries over [B, S, G, 128] keys and values are the packed
// prefill's dense form (uniform lengths, sequences back to back) on the tensor core; other widths, an empty key axis
// and unaligned tensors take the general kernel.
template <typename T>
static int dense_prefill_16bit(singe_stream_t stream, void *out, float *lse, const void *query, const void *key,
                               const void *value, size_t batch, size_t query_len, size_t key_len, size_t heads,
                               size_t kv_heads, size_t head_dim, float scale, int causal) {
    if (lse == nullptr) return SINGE_ERR_NULL_POINTER;
    const size_t total_q = batch * query_len, total_kv = batch * key_len;
    if (out != nullptr && query != nullptr && key != nullptr && value != nullptr && batch > 0 && query_len > 0 &&
        key_len > 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && finite(scale) &&
        total_q <= 0x7fffffffull && total_kv <= 0x7fffffffull &&
        prefill_fast_path(heads, kv_heads, head_dim, total_q, query, key, value, out)) {
        return prefill_tcgen05(static_cast<cudaStream_t>(stream), std::is_same<T, __half>::value, out, lse, query, key,
                               value, nullptr, nullptr, nullptr, batch, total_q, total_kv, heads, kv_heads, head_dim,
                               causal ? 1 : 0, scale, nullptr, 0, 0, query_len, key_len);
    }
    return dense_entry<T>(static_cast<cudaStream_t>(stream), static_cast<T *>(out), lse, static_cast<const T *>(query),
                          static_cast<const T *>(key), static_cast<const T *>(value), batch, heads, kv_heads,
                          query_len, key_len, head_dim, scale, causal, 0, true);
}

extern "C" {

int singe_fmha_prefill_lse_bf16(singe_stream_t stream, void *out, float *lse, const void *query, const void *key,
                                const void *value, size_t batch, size_t query_len, size_t key_len, size_t heads,
                                size_t kv_heads, size_t head_dim, float scale, int causal) {
    return dense_prefill_16bit<__nv_bfloat16>(stream, out, lse, query, key, value, batch, query_len, key_len, heads,
                                              kv_heads, head_dim, scale, causal);
}

int singe_fmha_prefill_lse_f16(singe_stream_t stream, void *out, float *lse, const void *query, const void *key,
                               const void *value, size_t batch, size_t query_len, size_t key_len, size_t heads,
                               size_t kv_heads, size_t head_dim, float scale, int causal) {
    return dense_prefill_16bit<__half>(stream, out, lse, query, key, value, batch, query_len, key_len, heads,
                                       kv_heads, head_dim, scale, causal);
}

int singe_scaled_dot_product_attention_f32(singe_stream_t stream, float *out, const float *query, const float *key,
                                           const float *value, size_t batch, size_t heads, size_t kv_heads,
                                           size_t query_len, size_t key_len, size_t head_dim, float scale, int causal,
                                           size_t window) {
    return dense_entry<float>(static_cast<cudaStream_t>(stream), out, nullptr, query, key, value, batch, heads,
                              kv_heads, query_len, key_len, head_dim, scale, causal, window, false);
}

}  // extern "C"
