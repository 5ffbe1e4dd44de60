/*
 * singe_kernel_sys.h -- the C ABI of libsinge_kernel_sys.so.
 *
 * These are the symbols the (today empty) `singe-kernel-sys` crate of tinrab/singe would bind
 * (singe-kernel-sys/src/lib.rs:1-6) so that the public operators of `singe_kernel::cuda` and the CUDA
 * kernels behind `singe::Tensor` run on hand-written sm_100a kernels.  Each declaration cites the
 * reference interface it replaces (path:line inside tinrab/singe).
 *
 * Conventions, which are the reference's raw-kernel execution contract
 * (singe-kernel/src/cuda/mod.rs:3-13, singe-kernel/docs/kernels.md:55-80):
 *   - every call only ENQUEUES work on `stream` (a CUstream / cudaStream_t passed as void*); nothing
 *     synchronises, and the caller keeps every buffer alive until the queued work completes;
 *   - all pointers are device pointers unless a parameter says "host";
 *   - the caller owns every buffer, scratch included; outputs may be uninitialised and only logical
 *     elements are written;
 *   - sizes are element counts (not bytes) and must fit a signed 32-bit integer, as the reference
 *     checks with `checked_i32_value` (singe-kernel/src/cuda/attention/mod.rs:2963-3011);
 *   - the return value is SINGE_OK or one SINGE_ERR_* code mirroring a variant of
 *     `singe_kernel::error::Error` (singe-kernel/src/error.rs:13-189); CUDA runtime failures come back
 *     as SINGE_ERR_CUDA_BASE + cudaError_t;
 *   - data-dependent index errors (a page or slot outside the cache) never fault: the access is
 *     dropped and code 1 is written to the optional `status` word, the reference's status-word
 *     protocol (singe/src/backend/cuda/kernel_plan/source/paged_attention.rs:52-54,
 *     kernel_plan/mod.rs:192-204).  Code 2 in that word means a bounded device-side wait ran out.
 *
 * There is no CPU fallback: on a machine without a CUDA device the compute entry points return
 * SINGE_ERR_CUDA_BASE + cudaErrorNoDevice (or the driver's own error).
 */
#ifndef SINGE_KERNEL_SYS_H
#define SINGE_KERNEL_SYS_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes: singe-kernel/src/error.rs:13-189 ---- */
#define SINGE_OK 0
#define SINGE_ERR_INVALID_LENGTH 1            /* Error::InvalidLength */
#define SINGE_ERR_LENGTH_TOO_SHORT 2          /* Error::LengthTooShort { .. } */
#define SINGE_ERR_LENGTH_EXCEEDS_I32 3        /* Error::LengthExceedsI32 */
#define SINGE_ERR_NULL_POINTER 4              /* Error::NullPointer */
#define SINGE_ERR_SIZE_OVERFLOW 5             /* Error::SizeOverflow */
#define SINGE_ERR_UNSUPPORTED_WIDTH 6         /* Error::UnsupportedWidth { op, width } */
#define SINGE_ERR_UNSUPPORTED_CONFIGURATION 7 /* Error::UnsupportedConfiguration { op, reason } */
#define SINGE_ERR_LENGTH_MISMATCH 8           /* Error::LengthMismatch */
#define SINGE_ERR_INDEX_OUT_OF_BOUNDS 9       /* singe::Error::IndexOutOfBounds (host-side checks) */
#define SINGE_ERR_INVALID_ARGUMENT 10         /* singe::Error::invalid_argument */
#define SINGE_ERR_OUT_OF_RANGE 11             /* singe::Error::out_of_range */
#define SINGE_ERR_AUTOTUNE_DURING_CAPTURE 12  /* Error::AutotuneDuringCapture (workspace growth under capture) */
#define SINGE_ERR_STATIC_SCRATCH_EXCEEDED 13  /* the problem needs more than the library's fixed scratch array */
#define SINGE_ERR_CUDA_BASE 1000              /* + cudaError_t */

/* Device-side status word values. */
#define SINGE_STATUS_INDEX_OUT_OF_BOUNDS 1u
#define SINGE_STATUS_WAIT_TIMEOUT 2u

typedef void *singe_stream_t; /* CUstream / cudaStream_t */

/* Hints a caller may give the entry points that take a `hints` argument.  They widen what a kernel may read BEFORE
 * the kernels queued ahead of it on the stream have finished (all of this library's decode-path kernels are launched
 * so that their set-up overlaps the kernel before); without a hint a kernel reads nothing early.
 *   SINGE_HINT_STABLE_WEIGHTS : the weight operand is not written by any work still in flight when the call is
 *                               enqueued (a layer parameter): its first tiles are fetched ahead of the wait.
 *   SINGE_HINT_STABLE_PAGING  : lengths and block table are not written by work still in flight, and of the cache
 *                               only each sequence's LAST key position may be (the row the step's cache write
 *                               fills): everything else of the cache is fetched ahead of the wait.
 * The reference has no counterpart: its launches serialise on the stream. */
#define SINGE_HINT_STABLE_WEIGHTS 1u
#define SINGE_HINT_STABLE_PAGING 2u

/* Library version (major * 1000 + minor). */
int singe_kernel_sys_version(void);

/* Static description of a status code. */
const char *singe_status_string(int status);

/* =================================================================================================
 * Slot-mapped KV-cache write
 * Replaces: KvCache::write = two index_put_ scatters at DecodeStep::slots()
 *   (singe/src/nn/decode/cache.rs:97-101, singe/src/nn/decode/step.rs:104-111), whose CPU meaning is
 *   index_write/plan (singe/src/backend/cpu/shape/multi_index.rs:95-125,204-236), and the slot-mapped
 *   store of singe_rotary_cache_write (singe/src/backend/cuda/kernel_plan/source/rotary_cache.rs:238-427).
 * cache[pages[t], slots[t], :, :] = rows[t, :, :] as a byte copy, for keys and values in one launch.
 * A negative page or slot wraps by its extent; a value still outside is dropped and reported through
 * `status` (code 1).  Duplicate positions: unspecified winner, as the reference's CUDA path
 * (singe/src/index/advanced.rs:79).
 *   key_cache, value_cache : [pages, page_size, kv_heads, head_dim]
 *   keys, values           : [tokens, kv_heads, head_dim]; `values`/`value_cache` may both be NULL
 *   write_pages, write_slots : [tokens], int64 when index_width == 8, int32 when index_width == 4
 * ================================================================================================= */
int singe_kv_cache_write_bf16(singe_stream_t stream, void *key_cache, void *value_cache, const void *keys,
                              const void *values, const void *write_pages, const void *write_slots,
                              int index_width, size_t tokens, size_t kv_heads, size_t head_dim, size_t pages,
                              size_t page_size, uint32_t *status);
int singe_kv_cache_write_f16(singe_stream_t stream, void *key_cache, void *value_cache, const void *keys,
                             const void *values, const void *write_pages, const void *write_slots, int index_width,
                             size_t tokens, size_t kv_heads, size_t head_dim, size_t pages, size_t page_size,
                             uint32_t *status);
int singe_kv_cache_write_f32(singe_stream_t stream, void *key_cache, void *value_cache, const void *keys,
                             const void *values, const void *write_pages, const void *write_slots, int index_width,
                             size_t tokens, size_t kv_heads, size_t head_dim, size_t pages, size_t page_size,
                             uint32_t *status);

/* =================================================================================================
 * Paged-KV decode attention (one query token per sequence)
 * Replaces: singe_kernel::cuda::attention::paged_kv_decode_attention_{f32,f16,bf16}
 *   (singe-kernel/src/cuda/attention/paged.rs:118-249; argument order of the launcher call :230-248),
 *   config PagedKvDecodeAttentionConfig (singe-kernel/src/cuda/attention/mod.rs:81-90,686-744,2963-2985),
 *   CPU meaning paged_kv_decode_attention_f32 (singe-kernel/src/cpu/attention.rs:1172-1246).
 *   out, query            : [batch, heads, head_dim]
 *   key_cache, value_cache: [physical_blocks, block_size, kv_heads, head_dim]
 *   actual_seq_lens       : int32 [batch]; a sequence of length 0 writes zeros
 *   block_table           : uint32 [batch, block_table_batch_stride]
 * The bf16/f16 entry points run the split-K flash-decode kernel (TMA-staged pages, tensor-core
 * tiles, log-sum-exp combine) when head_dim is 64 or 128, block_size is 16 and heads/kv_heads <= 8,
 * and a general one-warp-per-row kernel otherwise (also for batch > 65535).  Their split-K partials live in
 * a per-device workspace the library grows on demand (never while the stream is capturing: that returns
 * SINGE_ERR_AUTOTUNE_DURING_CAPTURE; call once outside capture first, or use the *_splitk_reduce_*
 * entry points below with caller-owned scratch).  Every stream of a device shares that one workspace: calls
 * whose kernels can overlap on the GPU (different streams, no event between them) race on it -- run them on
 * one stream at a time or pass caller-owned scratch.  Growth never frees: a buffer that was handed out
 * (and may be baked into a captured CUDA graph) stays allocated until singe_release_workspaces().
 * ================================================================================================= */
int singe_paged_kv_decode_attention_bf16(singe_stream_t stream, void *out, const void *query,
                                         const void *key_cache, const void *value_cache,
                                         const int32_t *actual_seq_lens, const uint32_t *block_table, size_t batch,
                                         size_t heads, size_t kv_heads, size_t head_dim, size_t block_size,
                                         size_t physical_blocks, size_t block_table_batch_stride, float scale);
int singe_paged_kv_decode_attention_f16(singe_stream_t stream, void *out, const void *query, const void *key_cache,
                                        const void *value_cache, const int32_t *actual_seq_lens,
                                        const uint32_t *block_table, size_t batch, size_t heads, size_t kv_heads,
                                        size_t head_dim, size_t block_size, size_t physical_blocks,
                                        size_t block_table_batch_stride, float scale);
int singe_paged_kv_decode_attention_f32(singe_stream_t stream, float *out, const float *query,
                                        const float *key_cache, const float *value_cache,
                                        const int32_t *actual_seq_lens, const uint32_t *block_table, size_t batch,
                                        size_t heads, size_t kv_heads, size_t head_dim, size_t block_size,
                                        size_t physical_blocks, size_t block_table_batch_stride, float scale);

/* -------------------------------------------------------------------------------------------------
 * Paged-KV decode that never allocates (no counterpart in the reference: this entry point exists only here).
 * Same arguments and result as singe_paged_kv_decode_attention_bf16, for hosts that cannot let the library
 * call cudaMalloc: a runtime that gives all device memory to its own pool (the reference's operators never
 * allocate, singe-kernel/src/cuda/attention/mod.rs:3-7), or a decode loop that cannot take the device-wide
 * synchronisation an allocation implies.  The split-K partials live in a fixed array inside the library,
 * singe_paged_kv_decode_attention_static_scratch_floats() floats (8 MiB) per GPU that loads it, held until
 * the process exits.  The call needs batch * heads * (head_dim + 1) floats per split; it lowers the split count
 * to fit and returns SINGE_ERR_STATIC_SCRATCH_EXCEEDED when even one split does not fit.  It takes only the
 * shapes of the tiled kernel (head_dim 64/128, block_size 16, heads/kv_heads <= 8) and calls no cudaMalloc,
 * cudaFree or other allocating routine.  The first call on each device looks up the array's device address
 * (a runtime query, not stream work): make that first call before starting any stream capture.  All calls on
 * a device share the one array, so two calls whose kernels can overlap on the GPU (different streams) race;
 * calls on one stream are ordered and safe.  Nothing in the array has to be cleared between calls.
 * ------------------------------------------------------------------------------------------------- */
size_t singe_paged_kv_decode_attention_static_scratch_floats(void);
int singe_paged_kv_decode_attention_static_bf16(singe_stream_t stream, void *out, const void *query,
                                                const void *key_cache, const void *value_cache,
                                                const int32_t *actual_seq_lens, const uint32_t *block_table,
                                                size_t batch, size_t heads, size_t kv_heads, size_t head_dim,
                                                size_t block_size, size_t physical_blocks,
                                                size_t block_table_batch_stride, float scale);

/* =================================================================================================
 * Split-K decode with caller-owned scratch, and the log-sum-exp combine
 * Replaces: fmha_decode_splitk_{f32,f16,bf16}, splitk_reduce_f32, fmha_decode_splitk_reduce_f32 and their
 *   configs FmhaDecodeSplitKConfig / SplitKReduceConfig / FmhaDecodeSplitKReduceConfig
 *   (singe-kernel/src/cuda/attention/fmha.rs:1038-1313, splitk.rs:187-284, mod.rs:366-499,2232-2560),
 *   CPU meaning splitk_reduce_f32 (singe-kernel/src/cpu/attention.rs:2157-2193).  The reference applies
 *   split-K to contiguous K/V only; here the same partial layout is applied to the paged decode above.
 *
 * Partial layout (singe-kernel/src/cuda/attention/mod.rs:2456-2509):
 *   attn_scratch f32 [batch, heads, max_splits, head_dim]  -- softmax-within-split . V, normalised
 *   lse_scratch  f32 [batch, heads, max_splits]            -- max + ln(sum exp), natural log
 * Split s of a sequence covers keys [s * split_tokens, (s+1) * split_tokens) where
 *   split_tokens = singe_paged_kv_decode_split_tokens(block_table_batch_stride * block_size, max_splits),
 * a multiple of block_size; splits past a sequence's length hold lse = -inf and zeros.
 * The tiled kernel takes batch <= 65535 and max_splits <= 65535 (grid dimensions); beyond that the call
 * returns SINGE_ERR_UNSUPPORTED_CONFIGURATION.
 * ================================================================================================= */

/* Tokens per split for a key-length bound and a split budget (host arithmetic, no device work). */
size_t singe_paged_kv_decode_split_tokens(size_t key_len_bound, size_t max_splits, size_t block_size);

/* The split count singe_paged_kv_decode_attention_{bf16,f16} choose for themselves (host arithmetic; uses the SM
 * count of the current device, 148 when there is none): 512-key pieces, or larger ones out of 640 / 832 / 1024 /
 * 1360 / 2048 when a wave model of the grid prefers them.  A caller that brings its own scratch sizes it with this
 * count to run the same launch. */
size_t singe_paged_kv_decode_default_splits(size_t batch, size_t kv_heads, size_t key_len_bound, size_t block_size);

/* Writes the partials only (all `max_splits` slots of every row are defined afterwards). */
int singe_paged_kv_decode_splitk_bf16(singe_stream_t stream, float *attn_scratch, float *lse_scratch,
                                      const void *query, const void *key_cache, const void *value_cache,
                                      const int32_t *actual_seq_lens, const uint32_t *block_table, size_t batch,
                                      size_t heads, size_t kv_heads, size_t head_dim, size_t block_size,
                                      size_t physical_blocks, size_t block_table_batch_stride, size_t max_splits,
                                      float scale);

/* splitk_reduce_f32 with the strides of SplitKReduceConfig (singe-kernel/src/cuda/attention/mod.rs:2320-2370). */
int singe_splitk_reduce_f32(singe_stream_t stream, float *out, const float *attn_splitk, const float *lse_splitk,
                            size_t batch, size_t heads, size_t splits, size_t head_dim, size_t attn_batch_stride,
                            size_t attn_head_stride, size_t attn_split_stride, size_t lse_batch_stride,
                            size_t lse_head_stride, size_t output_batch_stride, size_t output_head_stride);

/* Decode over CONTIGUOUS keys and values with split-K and the fold in one call.
 * Replaces: fmha_decode_splitk_reduce_f32 + FmhaDecodeSplitKReduceConfig::contiguous
 *   (singe-kernel/src/cuda/attention/fmha.rs:1155-1241, mod.rs:454-477; lengths :2511-2539).
 *   query, out [batch, heads, head_dim]; key, value [batch, key_len, kv_heads, head_dim];
 *   attn_scratch [batch, heads, splits, head_dim], lse_scratch [batch, heads, splits] with
 *   splits = min(max_splits, key_len).  The reference's tuner (tune_fmha_decode_splitk_reduce_f32) picks the split
 *   count by timing; here the caller's max_splits is the split count (TuningChoice::Default's meaning). */
int singe_fmha_decode_splitk_reduce_f32(singe_stream_t stream, float *out, float *attn_scratch, float *lse_scratch,
                                        const float *query, const float *key, const float *value, size_t batch,
                                        size_t key_len, size_t heads, size_t kv_heads, size_t head_dim,
                                        size_t max_splits, float scale);

/* Decode + combine in one call with caller scratch sized for `max_splits` (>= 1). */
int singe_paged_kv_decode_splitk_reduce_bf16(singe_stream_t stream, void *out, float *attn_scratch,
                                             float *lse_scratch, const void *query, const void *key_cache,
                                             const void *value_cache, const int32_t *actual_seq_lens,
                                             const uint32_t *block_table, size_t batch, size_t heads,
                                             size_t kv_heads, size_t head_dim, size_t block_size,
                                             size_t physical_blocks, size_t block_table_batch_stride,
                                             size_t max_splits, float scale);
int singe_paged_kv_decode_splitk_reduce_f16(singe_stream_t stream, void *out, float *attn_scratch,
                                            float *lse_scratch, const void *query, const void *key_cache,
                                            const void *value_cache, const int32_t *actual_seq_lens,
                                            const uint32_t *block_table, size_t batch, size_t heads,
                                            size_t kv_heads, size_t head_dim, size_t block_size,
                                            size_t physical_blocks, size_t block_table_batch_stride,
                                            size_t max_splits, float scale);

/* singe_paged_kv_decode_splitk_reduce_bf16 inside a decode step: same arguments and result plus a `hints` word.
 * With SINGE_HINT_STABLE_PAGING the kernel reads lengths, block table and cache pages ahead of the kernels still
 * running before it on the stream, except the page holding each sequence's last key position (the one row the
 * step's cache write, queued just before, fills); the queries are read after those kernels finish.
 * tickets: uint32 [batch * kv_heads], zero at first use and left zero by every call, or NULL.  With tickets the
 * split that finishes a (sequence, KV head) row last folds the row's partials inside the decode kernel and no
 * combine kernel is launched.  Measured on B200 this is SLOWER than the separate combine kernel even when the grid is
 * one wave (+6 us on a 17 us decode: every CTA pays a device-wide fence and an atomic on its way out), so callers
 * normally pass NULL; the path exists for hosts where a launch costs more than that.
 * No reference counterpart (the reference's launches serialise). */
int singe_paged_kv_decode_step_bf16(singe_stream_t stream, void *out, float *attn_scratch, float *lse_scratch,
                                    const void *query, const void *key_cache, const void *value_cache,
                                    const int32_t *actual_seq_lens, const uint32_t *block_table, size_t batch,
                                    size_t heads, size_t kv_heads, size_t head_dim, size_t block_size,
                                    size_t physical_blocks, size_t block_table_batch_stride, size_t max_splits,
                                    float scale, unsigned hints, uint32_t *tickets);

/* Paged decode that rotates its queries itself: `query` holds the projections BEFORE the rotary embedding, the kernel
 * applies the half-split rotation at positions[b] (cos / sin tables [capacity, head_dim / 2] in bf16; a negative
 * position wraps by capacity, one still outside is reported through the device error word and treated as 0) --
 * optionally after a per-head RMSNorm with gain query_norm_weight [head_dim] (NULL: no gain) -- and then attends as
 * singe_paged_kv_decode_step_bf16 does.  Same rounding as singe_rotary_cache_write_bf16 followed by the decode call.
 * Only the shapes of the tiled kernel (head_dim 64 / 128, block_size 16, heads / kv_heads <= 8).
 * Replaces: singe_rotary_paged_attention and its QueryRotation
 * (singe/src/backend/cuda/kernel_plan/source/paged_attention.rs:535-542,881-977). */
int singe_rotary_paged_kv_decode_attention_bf16(singe_stream_t stream, void *out, float *attn_scratch,
                                                float *lse_scratch, const void *query, const void *key_cache,
                                                const void *value_cache, const int32_t *actual_seq_lens,
                                                const uint32_t *block_table, const void *cos_table,
                                                const void *sin_table, const void *positions, int index_width,
                                                size_t batch, size_t heads, size_t kv_heads, size_t head_dim,
                                                size_t block_size, size_t physical_blocks,
                                                size_t block_table_batch_stride, size_t max_splits, size_t capacity,
                                                float scale, int normalise_query, const void *query_norm_weight,
                                                float eps, unsigned hints);

/* The attention part of a decode step in ONE launch (plus the combine, unless tickets are given): rotary embedding of
 * the queries and of the step's new key, the slot-mapped write of the new key and value rows into the cache, and paged
 * attention over the cached keys and the new one.
 *   qkv       : [batch, qkv_row_stride] bf16, one new token per sequence: heads * head_dim query projections, then
 *               kv_heads * head_dim key and kv_heads * head_dim value projections, all BEFORE the rotary embedding
 *   actual_seq_lens[b] counts the keys INCLUDING the new token (its position + 1); write_pages / write_slots [batch]
 *               say where its K and V rows go (negative values wrap, anything still outside is dropped and reported
 *               through `status`); positions [batch] index the cos / sin tables [capacity, head_dim / 2]
 * The new rows are written by this kernel and not read back from the cache by it, so under SINGE_HINT_STABLE_PAGING
 * every cache page it streams may be requested ahead of the kernels before it.  Same rounding as
 * singe_rotary_cache_write_bf16 followed by the decode call, except that the new key's score is a plain f32 dot
 * product instead of a tensor-core tile (same products, another summation order).
 * Replaces: the fused rotary_cache_write module followed by singe_rotary_paged_attention
 * (singe/src/backend/cuda/kernel_plan/source/rotary_cache.rs:238-427, paged_attention.rs:881-977; recognised in
 * singe/src/compiled/plan/fusion/module.rs:28-74), i.e. GroupedQueryAttention::decode between its projections
 * (singe/src/nn/layers/attention/grouped.rs:92-115). */
int singe_decode_step_attention_bf16(singe_stream_t stream, void *out, float *attn_scratch, float *lse_scratch,
                                     const void *qkv, size_t qkv_row_stride, void *key_cache, void *value_cache,
                                     const int32_t *actual_seq_lens, const uint32_t *block_table,
                                     const void *cos_table, const void *sin_table, const void *positions,
                                     const void *write_pages, const void *write_slots, int index_width, size_t batch,
                                     size_t heads, size_t kv_heads, size_t head_dim, size_t block_size,
                                     size_t physical_blocks, size_t block_table_batch_stride, size_t max_splits,
                                     size_t capacity, float scale, unsigned hints, uint32_t *tickets,
                                     uint32_t *status);

/* Pages beyond its shared-memory ring that each CTA of the hinted decode pulls into L2 ahead of its wait
 * (0 = none, the default).  A tuning knob like singe_matmul_set_staging. */
int singe_paged_kv_decode_set_prefetch(int pages);

/* =================================================================================================
 * Tensor-surface paged attention (FlashInfer-style paging, decode and prefill rows mixed)
 * Replaces: the CUDA kernels registered for Operation::PagedAttention behind Tensor::paged_attention
 *   (singe/src/tensor/neural.rs:405-457; singe_paged_attention / singe_tcgen05_paged_attention /
 *   singe_paged_attention_general in singe/src/backend/cuda/kernel_plan/source/paged_attention.rs:68-208,
 *   544-868 and paged_general.rs:73-247), CPU meaning attend_paged
 *   (singe/src/backend/cpu/normalization/attention.rs:424-540), refusals check_paged_values
 *   (singe/src/backend/spec/neural/attention.rs:363-416).
 *   query, out : [tokens, heads, head_dim];  lse : f32 [tokens, heads], BASE 2, -inf for a row with no key
 *   key_cache, value_cache : [cache_pages, page_size, kv_heads, head_dim]
 *   query_offsets, page_offsets : [sequences + 1]; pages : [table_len]; last_page_lengths : [sequences]
 *   (int64 when index_width == 8, int32 when 4).  Queries are the LAST tokens of their sequence.
 *   window == 0 means no sliding window.  Paging values that would address outside the queries, the
 *   table or the cache set *status = 1 and the affected rows are skipped.
 * ================================================================================================= */
int singe_paged_attention_bf16(singe_stream_t stream, void *out, float *lse, const void *query,
                               const void *key_cache, const void *value_cache, const void *query_offsets,
                               const void *page_offsets, const void *pages, const void *last_page_lengths,
                               int index_width, size_t tokens, size_t heads, size_t kv_heads, size_t head_dim,
                               size_t page_size, size_t cache_pages, size_t sequences, size_t table_len, float scale,
                               int causal, size_t window, uint32_t *status);
int singe_paged_attention_f32(singe_stream_t stream, float *out, float *lse, const float *query,
                              const float *key_cache, const float *value_cache, const void *query_offsets,
                              const void *page_offsets, const void *pages, const void *last_page_lengths,
                              int index_width, size_t tokens, size_t heads, size_t kv_heads, size_t head_dim,
                              size_t page_size, size_t cache_pages, size_t sequences, size_t table_len, float scale,
                              int causal, size_t window, uint32_t *status);

/* The same with the remaining AttentionOptions field of the path, the cap on the scaled scores
 * (singe/src/tensor/neural.rs:26-32; CPU: score = cap * tanh(score / cap) before the softmax,
 * singe/src/backend/cpu/normalization/attention.rs:445,500; CUDA: paged_attention.rs:112,662-672).  softcap == 0: none.
 * Plain decode batches keep the tiled flash-decode kernel (tanh.approx on the score path). */
int singe_paged_attention_options_bf16(singe_stream_t stream, void *out, float *lse, const void *query,
                                       const void *key_cache, const void *value_cache, const void *query_offsets,
                                       const void *page_offsets, const void *pages, const void *last_page_lengths,
                                       int index_width, size_t tokens, size_t heads, size_t kv_heads, size_t head_dim,
                                       size_t page_size, size_t cache_pages, size_t sequences, size_t table_len,
                                       float scale, int causal, size_t window, float softcap, uint32_t *status);
int singe_paged_attention_options_f32(singe_stream_t stream, float *out, float *lse, const float *query,
                                      const float *key_cache, const float *value_cache, const void *query_offsets,
                                      const void *page_offsets, const void *pages, const void *last_page_lengths,
                                      int index_width, size_t tokens, size_t heads, size_t kv_heads, size_t head_dim,
                                      size_t page_size, size_t cache_pages, size_t sequences, size_t table_len,
                                      float scale, int causal, size_t window, float softcap, uint32_t *status);

/* =================================================================================================
 * Packed variable-length prefill attention
 * Replaces: paged_kv_prefill_attention_{f32,bf16} + PagedKvPrefillAttentionConfig and
 *   ragged_kv_prefill_attention_{f32,bf16} + RaggedKvPrefillAttentionConfig
 *   (singe-kernel/src/cuda/attention/paged.rs:256-576, launcher argument order :396-418;
 *   mod.rs:97-123,746-882), CPU meaning singe-kernel/src/cpu/attention.rs:1248-1420.
 *   query, out : [total_query_tokens, heads, head_dim]; lse : f32 [total_query_tokens, heads], natural
 *   log, -1.0e20 for a row that sees no key.  Sequence b owns query tokens
 *   [offsets[b], offsets[b] + lens_q[b]) and keys 0..lens_kv[b]; causal == 1 hides key_index > query_index
 *   with sequence-local indices (singe-kernel/src/cpu/attention.rs:1282,1377).  causal == 2 (an addition, for
 *   prompt chunks behind an earlier context): the queries are the sequence's LAST tokens, query i sits at position
 *   lens_kv[b] - lens_q[b] + i (clamped at 0) and sees the keys up to it -- the mask of Tensor::paged_attention
 *   (singe/src/backend/cpu/normalization/attention.rs:481-483).
 *   ragged: key, value [total_kv_tokens, kv_heads, head_dim], key k of sequence b at row offsets[b] + k.
 * The bf16 and f16 entry points (paged.rs:313-421,479-582) run the tcgen05/TMEM flash-attention kernel when
 * head_dim == 128 (the paged form with 16-token pages: its key tiles are gathered through the block table); f16
 * takes the exact row maximum on every key tile so that the probabilities stay inside the half range.  Other
 * shapes and f32 run the general kernel.
 * ================================================================================================= */
int singe_paged_kv_prefill_attention_bf16(singe_stream_t stream, void *out, float *lse, const void *query,
                                          const void *key_cache, const void *value_cache,
                                          const int32_t *actual_seq_lens_q, const int32_t *actual_seq_lens_kv,
                                          const int32_t *actual_seq_offsets, const uint32_t *block_table,
                                          size_t batch, size_t total_query_tokens, size_t heads, size_t kv_heads,
                                          size_t head_dim, size_t block_size, size_t physical_blocks,
                                          size_t block_table_batch_stride, int causal, float scale);
int singe_paged_kv_prefill_attention_f16(singe_stream_t stream, void *out, float *lse, const void *query,
                                         const void *key_cache, const void *value_cache,
                                         const int32_t *actual_seq_lens_q, const int32_t *actual_seq_lens_kv,
                                         const int32_t *actual_seq_offsets, const uint32_t *block_table,
                                         size_t batch, size_t total_query_tokens, size_t heads, size_t kv_heads,
                                         size_t head_dim, size_t block_size, size_t physical_blocks,
                                         size_t block_table_batch_stride, int causal, float scale);
int singe_paged_kv_prefill_attention_f32(singe_stream_t stream, float *out, float *lse, const float *query,
                                         const float *key_cache, const float *value_cache,
                                         const int32_t *actual_seq_lens_q, const int32_t *actual_seq_lens_kv,
                                         const int32_t *actual_seq_offsets, const uint32_t *block_table,
                                         size_t batch, size_t total_query_tokens, size_t heads, size_t kv_heads,
                                         size_t head_dim, size_t block_size, size_t physical_blocks,
                                         size_t block_table_batch_stride, int causal, float scale);
int singe_ragged_kv_prefill_attention_bf16(singe_stream_t stream, void *out, float *lse, const void *query,
                                           const void *key, const void *value, const int32_t *actual_seq_lens_q,
                                           const int32_t *actual_seq_lens_kv, const int32_t *actual_seq_offsets,
                                           size_t batch, size_t total_query_tokens, size_t total_kv_tokens,
                                           size_t heads, size_t kv_heads, size_t head_dim, int causal, float scale);
int singe_ragged_kv_prefill_attention_f16(singe_stream_t stream, void *out, float *lse, const void *query,
                                          const void *key, const void *value, const int32_t *actual_seq_lens_q,
                                          const int32_t *actual_seq_lens_kv, const int32_t *actual_seq_offsets,
                                          size_t batch, size_t total_query_tokens, size_t total_kv_tokens,
                                          size_t heads, size_t kv_heads, size_t head_dim, int causal, float scale);
int singe_ragged_kv_prefill_attention_f32(singe_stream_t stream, float *out, float *lse, const float *query,
                                          const float *key, const float *value, const int32_t *actual_seq_lens_q,
                                          const int32_t *actual_seq_lens_kv, const int32_t *actual_seq_offsets,
                                          size_t batch, size_t total_query_tokens, size_t total_kv_tokens,
                                          size_t heads, size_t kv_heads, size_t head_dim, int causal, float scale);

/* Prefill with the slot-mapped KV-cache write in the same pass: ragged prefill as above, and every
 * key/value row t is also stored at (write_pages[t], write_slots[t]) of the paged caches, with the
 * semantics of singe_kv_cache_write_bf16.  This is the reference's prompt step: KvCache::write followed
 * by attention inside GroupedQueryAttention::decode (singe/src/nn/layers/attention/grouped.rs:92-115). */
int singe_ragged_kv_prefill_attention_cache_write_bf16(
    singe_stream_t stream, void *out, float *lse, const void *query, const void *key, const void *value,
    const int32_t *actual_seq_lens_q, const int32_t *actual_seq_lens_kv, const int32_t *actual_seq_offsets,
    size_t batch, size_t total_query_tokens, size_t total_kv_tokens, size_t heads, size_t kv_heads, size_t head_dim,
    int causal, float scale, void *key_cache, void *value_cache, const void *write_pages, const void *write_slots,
    int index_width, size_t pages, size_t page_size, uint32_t *status);

/* Dense prefill with log-sum-exp.
 * Replaces: fmha_prefill_lse_{f32,f16,bf16} + FmhaPrefillConfig (singe-kernel/src/cuda/attention/fmha.rs:48-790,
 *   mod.rs:253-274,1602-1756), CPU meaning fmha_prefill_lse_f32 (singe-kernel/src/cpu/attention.rs:1758-1833).
 *   query, out [batch, query_len, heads, head_dim]; key, value [batch, key_len, kv_heads, head_dim];
 *   lse f32 [batch, heads, query_len], natural log.  The 16-bit entry points with head_dim == 128 run the
 *   tcgen05 prefill kernel in its dense form (uniform lengths, sequences back to back). */
int singe_fmha_prefill_lse_f32(singe_stream_t stream, float *out, float *lse, const float *query, const float *key,
                               const float *value, size_t batch, size_t query_len, size_t key_len, size_t heads,
                               size_t kv_heads, size_t head_dim, float scale, int causal);
int singe_fmha_prefill_lse_bf16(singe_stream_t stream, void *out, float *lse, const void *query, const void *key,
                                const void *value, size_t batch, size_t query_len, size_t key_len, size_t heads,
                                size_t kv_heads, size_t head_dim, float scale, int causal);
int singe_fmha_prefill_lse_f16(singe_stream_t stream, void *out, float *lse, const void *query, const void *key,
                               const void *value, size_t batch, size_t query_len, size_t key_len, size_t heads,
                               size_t kv_heads, size_t head_dim, float scale, int causal);

/* =================================================================================================
 * Dense scaled-dot-product attention (Tensor::attend)
 * Replaces: the CUDA kernels of Operation::ScaledDotProductAttention (singe_fused_attention /
 *   singe_tcgen05_attention, singe/src/backend/cuda/kernel_plan/source/attention.rs:179-545), CPU meaning
 *   execute_scaled_dot_product_attention (singe/src/backend/cpu/normalization/attention.rs:191-276).
 *   query, out [batch, heads, query_len, head_dim]; key, value [batch, kv_heads, key_len, head_dim];
 *   causal: query i sees keys 0..min(key_len, i+1); window == 0 means none.
 * ================================================================================================= */
int singe_scaled_dot_product_attention_f32(singe_stream_t stream, float *out, const float *query, const float *key,
                                           const float *value, size_t batch, size_t heads, size_t kv_heads,
                                           size_t query_len, size_t key_len, size_t head_dim, float scale,
                                           int causal, size_t window);

/* Tensor::attend with all of its options: singe_scaled_dot_product_attention_f32 plus the score cap (softcap == 0:
 * none) and per-head sink logits, sinks [heads] or NULL -- a sink takes part in its rows' softmax and weighs no value
 * (singe/src/backend/cpu/normalization/attention.rs:250-263). */
int singe_attend_f32(singe_stream_t stream, float *out, const float *query, const float *key, const float *value,
                     size_t batch, size_t heads, size_t kv_heads, size_t query_len, size_t key_len, size_t head_dim,
                     float scale, int causal, size_t window, float softcap, const float *sinks);

/* =================================================================================================
 * Linear-layer GEMM
 * Replaces: singe_kernel::cuda::matmul::{matmul_bf16_f32, matmul_mma_bf16_f32} + MatmulConfig
 *   (singe-kernel/src/cuda/matmul.rs:45-55,218-230,1302-1378; launcher argument order :1317-1337;
 *   validation :2977-3020) and the eager GEMM behind Linear::forward / Tensor::matmul
 *   (singe/src/nn/layers/linear/mod.rs:49-70, singe/src/backend/cuda/eager/linear_algebra.rs:20-67,
 *   singe_tcgen05_matmul in kernel_plan/source/tcgen05.rs:137-266, singe_dot_product in dot_product.rs:133-243).
 *   CPU meaning: singe-kernel/src/cpu/matmul/mod.rs:12-45, blocked.rs:27-95,
 *   singe/src/backend/cpu/binary/matmul.rs:18-43 (bf16 widened to f32, one rounding of the result).
 * out[rows, columns] = lhs . rhs with f32 accumulation.  lhs is [rows, reduction] or, with
 * transpose_lhs != 0, [reduction, rows] (MatmulConfig::row_major_transposed_lhs :204-216); rhs is either a
 * linear layer's weight [columns, reduction] (transpose_rhs == 1, MatmulConfig::row_major_transposed_rhs)
 * or a row-major [reduction, columns] operand (transpose_rhs == 0, MatmulConfig::row_major :190-202).
 * Operands whose contraction axis is not the contiguous one are read by the tensor core MN-major.  Row
 * strides and start addresses must be multiples of 16 bytes (TMA), else
 * SINGE_ERR_UNSUPPORTED_CONFIGURATION.  `_bf16` rounds the result once to bf16 (Tensor surface);
 * `_f32` keeps f32 (singe-kernel surface).
 * ================================================================================================= */
int singe_matmul_bf16_bf16(singe_stream_t stream, void *out, const void *lhs, const void *rhs, size_t rows,
                           size_t columns, size_t reduction, size_t lhs_row_stride, size_t rhs_row_stride,
                           size_t output_row_stride, int transpose_lhs, int transpose_rhs);
int singe_matmul_bf16_f32(singe_stream_t stream, float *out, const void *lhs, const void *rhs, size_t rows,
                          size_t columns, size_t reduction, size_t lhs_row_stride, size_t rhs_row_stride,
                          size_t output_row_stride, int transpose_lhs, int transpose_rhs);

/* =================================================================================================
 * Decode-step glue (bf16 tensors, f32 arithmetic inside)
 * Replaces the eager tensor ops the reference's Llama block runs between its GEMMs and attention
 * (singe/src/nn/layers/blocks/mod.rs:56-83, singe/src/nn/layers/networks/causal_lm.rs:121-148); the fused forms
 * correspond to the modules its compiled plans recognise (RotaryCacheWrite, singe/src/backend/cuda/compiled/plan/
 * fusion/module.rs:28-74, kernel singe_rotary_cache_write in kernel_plan/source/rotary_cache.rs:238-427).
 * ================================================================================================= */

/* Embedding lookup (singe::nn Embedding = index_select): out[t, :] = table[ids[t], :]; negative ids wrap, ids
 * outside the table write zeros and set *status = 1. */
int singe_embedding_bf16(singe_stream_t stream, void *out, const void *table, const void *ids, int index_width,
                         size_t tokens, size_t width, size_t vocab, uint32_t *status);

/* Residual add fused with RMSNorm (RmsNorm: singe/src/backend/cpu/normalization/standard.rs:43-60):
 *   hidden[r, :] = bf16(hidden[r, :] + delta[r, :])      when delta != NULL
 *   normed[r, :] = hidden[r, :] * 1/sqrt(mean(hidden[r, :]^2) + eps) * weight[:]   when normed != NULL */
int singe_add_rms_norm_bf16(singe_stream_t stream, void *hidden, const void *delta, void *normed, const void *weight,
                            size_t rows, size_t width, float eps);

/* Half-split rotary embedding of Q and K (RotaryAngles::rotate_pairs, singe/src/nn/layers/positional/rotary.rs:
 * 274-304; cos/sin tables [capacity, head_dim/2] in the model dtype, :166-219) fused with KvCache::write
 * (singe/src/nn/decode/cache.rs:97-101).  qkv rows are [heads*D | kv_heads*D | kv_heads*D] (the fused q/k/v
 * projection); q_out [tokens, heads, D] receives the rotated queries, the rotated keys and the values go to
 * (write_pages[t], write_slots[t]) of caches [pages, page_size, kv_heads, D].  Bad positions or slots are dropped
 * and reported through *status = 1. */
int singe_rotary_cache_write_bf16(singe_stream_t stream, void *q_out, const void *qkv, size_t qkv_row_stride,
                                  const void *cos_table, const void *sin_table, const void *positions,
                                  void *key_cache, void *value_cache, const void *write_pages,
                                  const void *write_slots, int index_width, size_t tokens, size_t heads,
                                  size_t kv_heads, size_t head_dim, size_t pages, size_t page_size, size_t capacity,
                                  uint32_t *status);

/* The same with the per-head RMSNorm a model applies to its query and / or key heads before rotating them
 * (RotationNorm, query_norm / key_norm of RotaryCacheInputs,
 * singe/src/backend/cuda/kernel_plan/source/rotary_cache.rs:25-52): every head's head_dim values are scaled by
 * 1 / sqrt(mean(x^2) + eps) and by the gain [head_dim] (NULL: no gain), rounded to bf16 as the separate RmsNorm op
 * returns them, and then rotated.  head_dim / 2 (head_dim / 16 on the 16-byte path) must be a power of two <= 32. */
int singe_rotary_norm_cache_write_bf16(singe_stream_t stream, void *q_out, const void *qkv, size_t qkv_row_stride,
                                       const void *cos_table, const void *sin_table, const void *positions,
                                       void *key_cache, void *value_cache, const void *write_pages,
                                       const void *write_slots, int index_width, size_t tokens, size_t heads,
                                       size_t kv_heads, size_t head_dim, size_t pages, size_t page_size,
                                       size_t capacity, int normalise_query, const void *query_norm_weight,
                                       int normalise_key, const void *key_norm_weight, float eps, uint32_t *status);

/* GatedMlp activation (singe/src/nn/layers/feed_forward/mod.rs:58-66): out = bf16(bf16(silu(gate)) * up);
 * gate and up are [rows, width] views with row stride input_row_stride (halves of a fused gate/up projection). */
int singe_silu_mul_bf16(singe_stream_t stream, void *out, const void *gate, const void *up, size_t input_row_stride,
                        size_t rows, size_t width);

/* Greedy next token (argmax over logits rows, singe/src/generation/mod.rs:352-365): lowest index wins ties;
 * best_index gets index + index_offset (a vocabulary shard reports global ids), best_value the winning logit. */
int singe_argmax_bf16(singe_stream_t stream, float *best_value, int64_t *best_index, const void *logits,
                      size_t row_stride, size_t rows, size_t width, int64_t index_offset);

/* ---- tensor-parallel all-reduce over NVLink peer memory, fused with residual add + RMSNorm ----
 * Replaces, for the decode step's two collectives per layer: Communicator::all_reduce_in_place with
 * ReductionOperator::Sum (singe-nccl/src/communicator/operations/collectives.rs:99-134) followed by the residual
 * add and the next RMSNorm of the pre-norm block (singe-model/src/assembly/decoder.rs:102-126).
 *
 * Peer buffers are plain device allocations shared between the ranks' processes through CUDA IPC handles
 * (SINGE_PEER_HANDLE_BYTES opaque bytes, exchanged by the host's own means, e.g. the NCCL bootstrap store). */
#define SINGE_PEER_HANDLE_BYTES 64
int singe_peer_buffer_create(size_t bytes, void **pointer, void *handle_out); /* zero-filled */
int singe_peer_buffer_open(const void *handle_in, void **pointer);            /* another rank's buffer */
int singe_peer_buffer_close(void *pointer);                                   /* what _open returned */
int singe_peer_buffer_destroy(void *pointer);                                 /* what _create returned */

/* hidden[rows, width] += bf16(sum over ranks of partials[r][rows, width]) (f32 sum in rank order, so every rank
 * gets identical bits), then normed = RMSNorm(hidden) * weight; bf16 throughout, rounding after every op as the
 * reference's tensor ops do.  partials / flags: HOST arrays of `world` device pointers, entry r being rank r's
 * partial buffer / flag array (uint32[world], zero at first use) as mapped into this process; entry `rank` is the
 * local one.  state: local uint32[2], zero at first use.  The call only enqueues; ranks synchronise inside the
 * kernel through the flag arrays (every wait is bounded: on a timeout *status gets SINGE_STATUS_WAIT_TIMEOUT and
 * hidden/normed are left unwritten).  The local partial buffer may be rewritten only after a LATER call of this
 * function (on another partial buffer) has been enqueued behind this one: alternate two buffers. world <= 8,
 * width % 8 == 0, width <= 8192. */
int singe_allreduce_add_rms_norm_bf16(singe_stream_t stream, void *hidden, void *normed, const void *weight,
                                      const void *const *partials, uint32_t *const *flags, uint32_t *state, int rank,
                                      int world, size_t rows, size_t width, float eps, uint32_t *status);

/* The same collective in two phases, for more ranks (the one-shot form reads world x rows x width per rank):
 * rank r owns rows [r * rpr, (r + 1) * rpr), rpr = ceil(rows / world).  Every rank pushes its partial rows into their
 * owners' receive buffers, an owner sums its rows (rank order, f32, rounded to bf16), adds them to ITS rows of the
 * residual stream `hidden` (only the owner keeps a row of the residual up to date), normalises and pushes the
 * normalised rows to every rank; when the kernel has finished, the local `normed` [rows, width] holds all rows.
 * Data crosses NVLink as 8-byte packets {4 bytes data, 4-byte launch epoch}: no flags, fences or atomics.
 *   partial          : local [rows, width], this rank's partial sums (read only)
 *   receive, gather  : HOST arrays of `world` device pointers, entry r being rank r's buffer as mapped into this
 *                      process; receive holds world * rpr * width * 4 bytes, gather (rows + rpr) * width * 4 bytes
 *                      (all normalised rows, then a staging area for the rows this rank owns), both
 *                      zero at first use and owned by the collective (packet format, not for the caller to read)
 *   state            : local uint32[4], zero at first use; state[2] != 0 shortens every wait to state[2] * 1024
 *                      clock cycles (the default is a few seconds).  The one-shot call reads state[2] the same way.
 *   replicated       : 0 as described.  1: every rank owns every row -- each partial row is pushed to ALL ranks, every
 *                      rank sums and normalises all rows itself and keeps the whole residual stream; one NVLink trip
 *                      instead of two at world x the bytes, which pays for two ranks.  receive then holds
 *                      world * rows * width * 4 bytes and gather is unused (pass the same pointers).
 * rows <= 256, width % 8 == 0, width <= 8192.  A wait that runs out writes SINGE_STATUS_WAIT_TIMEOUT to *status, leaves
 * the rows that depended on it unwritten, and the kernel ends.  No reference counterpart beyond the all-reduce itself
 * (singe-nccl/src/communicator/operations/collectives.rs:99-134). */
int singe_allreduce_two_phase_add_rms_norm_bf16(singe_stream_t stream, void *hidden, void *normed, const void *weight,
                                                const void *partial, void *const *receive, void *const *gather,
                                                uint32_t *state, int rank, int world, size_t rows, size_t width,
                                                float eps, int replicated, uint32_t *status);

/* The gate and up projections of GatedMlp (singe/src/nn/layers/feed_forward/mod.rs:58-66) and its activation in one
 * call: rhs [columns, reduction] holds the gate and up weight rows interleaved (row 2j = gate_j, row 2j+1 = up_j),
 * out [rows, columns / 2] = bf16(bf16(silu(g_j)) * u_j) with g, u the bf16-rounded projections: the same roundings as
 * singe_matmul_bf16_bf16 followed by singe_silu_mul_bf16, without writing the projections out.
 * Replaces: two Linear::forward calls + silu + mul of GatedMlp::forward. */
int singe_matmul_bf16_swiglu_bf16(singe_stream_t stream, void *out, const void *lhs, const void *rhs, size_t rows,
                                  size_t columns, size_t reduction, size_t lhs_row_stride, size_t rhs_row_stride,
                                  size_t output_row_stride);

/* Linear::forward (singe/src/nn/layers/linear/mod.rs:49-70): out[rows, columns] = x[rows, reduction] . weight[columns,
 * reduction]^T, bf16 in, f32 accumulate, bf16 out -- singe_matmul_bf16_bf16 with the layer's layout fixed and a `hints`
 * word (SINGE_HINT_STABLE_WEIGHTS).  gated != 0: the SwiGLU epilogue of singe_matmul_bf16_swiglu_bf16 (out is
 * columns / 2 wide). */
int singe_linear_bf16(singe_stream_t stream, void *out, const void *x, const void *weight, size_t rows, size_t columns,
                      size_t reduction, size_t x_row_stride, size_t weight_row_stride, size_t output_row_stride,
                      int gated, unsigned hints);

/* Explicit tile choice for the two GEMM entry points, process-wide: block_n in {32,64,128,256},
 * k_slices_per_stage in {1,2,4,8}; 0 = choose from the problem shape.
 * Replaces: TuningChoice::Explicit(MatmulTuning { tile, .. }) (singe-kernel/src/cuda/matmul.rs:58-77). */
int singe_matmul_set_tuning(int block_n, int k_slices_per_stage);

/* K splits for problems with at most 128 rows (a thread-block cluster of that many CTAs shares one N tile and
 * reduces through distributed shared memory): 0 = choose from the shape, 1 = never split, 2 / 4 / 8 = as given.
 * No reference counterpart: the reference's MatmulTuning (singe-kernel/src/cuda/matmul.rs:57-77) carries a tile and
 * compile options only; this is a tuning knob of the same kind for this library's extra degree of freedom. */
int singe_matmul_set_splits(int k_splits);

/* Staging knobs of the same kind: shared memory one GEMM CTA may take (KB; 0 = choose), and how many KB of a stable
 * weight operand each CTA pulls into L2 ahead of its dependency wait beyond what its ring holds (negative = choose). */
int singe_matmul_set_staging(int shared_kb, int prefetch_kb);

/* L2 warm-ahead: attaches the read-only range [pointer, pointer + bytes) (16-byte aligned) to the NEXT kernel this host
 * thread enqueues through singe_linear_bf16 / singe_matmul_*, singe_paged_kv_decode_step_bf16 and the other
 * *_splitk_* decode calls, singe_add_rms_norm_bf16, singe_rotary_cache_write_bf16 or singe_allreduce_add_rms_norm_bf16;
 * that kernel asks the memory system to pull the range into L2 beside its own work, so that a later kernel (a weight
 * matrix two launches ahead, say) finds it there.  The range must stay allocated until that kernel has finished; it is
 * only read.  A hint: results never depend on it.  No reference counterpart. */
int singe_warm_l2_with_next_launch(const void *pointer, size_t bytes);

/* Frees the current device's decode workspaces (the live one and every one retired by growth) after a device
 * synchronisation.  Only when no captured graph that used them will be replayed again.  No reference
 * counterpart (the reference's operators take all scratch from the caller). */
int singe_release_workspaces(void);

/* Reads and clears the library's sticky device error word for the current device (synchronises the device).
 * 0 = no kernel-side failure; 2 = a bounded device-side wait ran out.  Plays the role of the planner's status
 * word read-back (singe/src/backend/cuda/kernel_plan/mod.rs:192-204) for entry points without a status argument. */
int singe_take_device_error(uint32_t *value);

#ifdef __cplusplus
}
#endif

#endif /* SINGE_KERNEL_SYS_H */
