/*
 * TEST INFRASTRUCTURE ONLY -- a CPU restatement of the reference's CPU kernels for the
 * attention-and-linear hot path.  Nothing in the shipped library links, loads or calls this file;
 * only the test suite, the smoke check and the benchmark's CPU-baseline leg do, and only as the
 * checker / reported baseline.
 *
 * Every function follows one function of the reference (tinrab/singe), cited by file:line above
 * it.  Arithmetic order is kept where it decides bits:
 *   - attention scores and P.V use a fused multiply-add exactly where the Rust uses `mul_add`;
 *   - the GEMM uses a separate multiply and add (the Rust forbids fusing there);
 *   - softmax is three passes (max, sum of exp, weighted values) and the weight is
 *     exp(score - max) / denom, divided before it multiplies the value;
 *   - expf/logf are the C library's, which is what Rust's f32::exp / f32::ln call on Linux.
 * One restructuring is used throughout and changes no bit: the Rust recomputes
 * exp(score - max) / denom once per output feature; that value does not depend on the feature, so
 * it is computed once per key here, and the per-feature accumulation keeps its ascending-key order.
 *
 * Parity pinning: the reference is Rust and no Rust toolchain exists in this build environment, so
 * the reference itself cannot be run.  The restatement is pinned against the known-answer vectors
 * the reference's own tests hold for this path (GQA group mapping, causal-left window, README GEMM
 * example, broadcast-stride GEMM, blocked-vs-naive GEMM equality, paging refusal table, cache-write
 * == index_put).  Beyond those vectors, attention and GEMM numerics on random inputs are
 * "parity unpinned": no reference-generated fixture exists to compare against.
 *
 * Build: see oracle/Makefile (gcc -O2 -ffp-contract=off -fopenmp).  Rows are independent, so the
 * OpenMP loops change no result; `oracle_set_threads` selects how many host threads are used.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_OK 0
#define ORACLE_INDEX_OUT_OF_BOUNDS 1
#define ORACLE_INVALID 2
#define ORACLE_LENGTH_TOO_SHORT 3
#define ORACLE_SIZE_OVERFLOW 4
#define ORACLE_LENGTH_MISMATCH 5

void oracle_set_threads(int threads) {
#ifdef _OPENMP
    if (threads > 0) omp_set_num_threads(threads);
#else
    (void)threads;
#endif
}

int oracle_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* ---- bf16 helpers: round-to-nearest-even as the `half` crate does (Cargo.toml:121) ---- */

uint16_t oracle_f32_to_bf16_bits(float value) {
    uint32_t bits;
    memcpy(&bits, &value, 4);
    if ((bits & 0x7fffffffu) > 0x7f800000u) {
        return (uint16_t)((bits >> 16) | 0x0040u); /* quiet NaN */
    }
    uint32_t round = 0x7fffu + ((bits >> 16) & 1u);
    return (uint16_t)((bits + round) >> 16);
}

float oracle_bf16_bits_to_f32(uint16_t bits) {
    uint32_t wide = (uint32_t)bits << 16;
    float value;
    memcpy(&value, &wide, 4);
    return value;
}

void oracle_round_to_bf16(float *values, size_t count) {
    for (size_t i = 0; i < count; ++i) {
        values[i] = oracle_bf16_bits_to_f32(oracle_f32_to_bf16_bits(values[i]));
    }
}

/* Shared softmax tail: given `count` scaled scores, produce weights[i] = exp(s - max) / denom and
 * return max + ln(denom).  Order of the max fold and of the sum is ascending, as the Rust iterators
 * run. */
static float softmax_weights(const float *scores, float *weights, size_t count, float *denom_out,
                             float *max_out) {
    float max_score = -INFINITY;
    for (size_t i = 0; i < count; ++i) max_score = fmaxf(max_score, scores[i]);
    float denom = 0.0f;
    for (size_t i = 0; i < count; ++i) denom += expf(scores[i] - max_score);
    for (size_t i = 0; i < count; ++i) weights[i] = expf(scores[i] - max_score) / denom;
    if (denom_out) *denom_out = denom;
    if (max_out) *max_out = max_score;
    return max_score + logf(denom);
}

/* singe-kernel/src/cpu/attention.rs:1172-1246  paged_kv_decode_attention_f32 */
void oracle_paged_kv_decode_attention_f32(float *out, const float *query, const float *key_cache,
                                          const float *value_cache, const int32_t *actual_seq_lens,
                                          const uint32_t *block_table, size_t batch, size_t heads,
                                          size_t kv_heads, size_t head_dim, size_t block_size,
                                          size_t block_table_batch_stride, float scale) {
    size_t group = heads / kv_heads;
    size_t token_stride = kv_heads * head_dim;
    size_t block_stride = block_size * token_stride;
    memset(out, 0, batch * heads * head_dim * sizeof(float));
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
    for (size_t b = 0; b < batch; ++b) {
        for (size_t head = 0; head < heads; ++head) {
            size_t seq_len = (size_t)actual_seq_lens[b];
            if (seq_len == 0) continue;
            size_t kv_head = head / group;
            float *scores = (float *)malloc(seq_len * sizeof(float));
            float *weights = (float *)malloc(seq_len * sizeof(float));
            const float *q = query + (b * heads + head) * head_dim;
            for (size_t k = 0; k < seq_len; ++k) {
                size_t block = block_table[b * block_table_batch_stride + k / block_size];
                const float *key =
                    key_cache + block * block_stride + (k % block_size) * token_stride + kv_head * head_dim;
                float score = 0.0f;
                for (size_t d = 0; d < head_dim; ++d) score = fmaf(q[d], key[d], score);
                scores[k] = score * scale;
            }
            softmax_weights(scores, weights, seq_len, NULL, NULL);
            float *o = out + (b * heads + head) * head_dim;
            for (size_t k = 0; k < seq_len; ++k) {
                size_t block = block_table[b * block_table_batch_stride + k / block_size];
                const float *value =
                    value_cache + block * block_stride + (k % block_size) * token_stride + kv_head * head_dim;
                for (size_t d = 0; d < head_dim; ++d) o[d] = fmaf(weights[k], value[d], o[d]);
            }
            free(scores);
            free(weights);
        }
    }
}

/* Shared body of the packed-prefill kernels; `block_table == NULL` selects the ragged layout.
 * singe-kernel/src/cpu/attention.rs:1248-1341 (paged) and :1343-1420 (ragged). */
static void prefill_packed(float *out, float *lse, const float *query, const float *key, const float *value,
                           const int32_t *lens_q, const int32_t *lens_kv, const int32_t *offsets,
                           const uint32_t *block_table, size_t batch, size_t total_query_tokens, size_t heads,
                           size_t kv_heads, size_t head_dim, size_t block_size, size_t table_stride, int causal,
                           float scale) {
    size_t group = heads / kv_heads;
    size_t features = heads * head_dim;
    size_t token_stride = kv_heads * head_dim;
    size_t block_stride = block_size * token_stride;
    memset(out, 0, total_query_tokens * features * sizeof(float));
    memset(lse, 0, total_query_tokens * heads * sizeof(float));
    for (size_t b = 0; b < batch; ++b) {
        size_t len_q = (size_t)lens_q[b];
        size_t len_kv = (size_t)lens_kv[b];
        size_t offset = (size_t)offsets[b];
#pragma omp parallel for collapse(2) schedule(dynamic, 4)
        for (size_t qi = 0; qi < len_q; ++qi) {
            for (size_t head = 0; head < heads; ++head) {
                size_t token = offset + qi;
                size_t kv_head = head / group;
                /* causal hides key_index > query_index, both sequence-local (:1282, :1377) */
                size_t visible = causal ? (qi + 1 < len_kv ? qi + 1 : len_kv) : len_kv;
                if (visible == 0) {
                    lse[token * heads + head] = -1.0e20f; /* :1304, :1397 */
                    continue;
                }
                float *scores = (float *)malloc(visible * sizeof(float));
                float *weights = (float *)malloc(visible * sizeof(float));
                const float *q = query + token * features + head * head_dim;
                for (size_t k = 0; k < visible; ++k) {
                    const float *kp;
                    if (block_table) {
                        size_t block = block_table[b * table_stride + k / block_size];
                        kp = key + block * block_stride + (k % block_size) * token_stride + kv_head * head_dim;
                    } else {
                        kp = key + (offset + k) * token_stride + kv_head * head_dim;
                    }
                    float score = 0.0f;
                    for (size_t d = 0; d < head_dim; ++d) score = fmaf(q[d], kp[d], score);
                    scores[k] = score * scale;
                }
                lse[token * heads + head] = softmax_weights(scores, weights, visible, NULL, NULL);
                float *o = out + token * features + head * head_dim;
                for (size_t k = 0; k < visible; ++k) {
                    const float *vp;
                    if (block_table) {
                        size_t block = block_table[b * table_stride + k / block_size];
                        vp = value + block * block_stride + (k % block_size) * token_stride + kv_head * head_dim;
                    } else {
                        vp = value + (offset + k) * token_stride + kv_head * head_dim;
                    }
                    for (size_t d = 0; d < head_dim; ++d) o[d] = fmaf(weights[k], vp[d], o[d]);
                }
                free(scores);
                free(weights);
            }
        }
    }
}

/* singe-kernel/src/cpu/attention.rs:1248-1341  paged_kv_prefill_attention_f32 */
void oracle_paged_kv_prefill_attention_f32(float *out, float *lse, const float *query, const float *key_cache,
                                           const float *value_cache, const int32_t *actual_seq_lens_q,
                                           const int32_t *actual_seq_lens_kv, const int32_t *actual_seq_offsets,
                                           const uint32_t *block_table, size_t batch, size_t total_query_tokens,
                                           size_t heads, size_t kv_heads, size_t head_dim, size_t block_size,
                                           size_t block_table_batch_stride, int causal, float scale) {
    prefill_packed(out, lse, query, key_cache, value_cache, actual_seq_lens_q, actual_seq_lens_kv,
                   actual_seq_offsets, block_table, batch, total_query_tokens, heads, kv_heads, head_dim,
                   block_size, block_table_batch_stride, causal, scale);
}

/* singe-kernel/src/cpu/attention.rs:1343-1420  ragged_kv_prefill_attention_f32 */
void oracle_ragged_kv_prefill_attention_f32(float *out, float *lse, const float *query, const float *key,
                                            const float *value, const int32_t *actual_seq_lens_q,
                                            const int32_t *actual_seq_lens_kv, const int32_t *actual_seq_offsets,
                                            size_t batch, size_t total_query_tokens, size_t heads, size_t kv_heads,
                                            size_t head_dim, int causal, float scale) {
    prefill_packed(out, lse, query, key, value, actual_seq_lens_q, actual_seq_lens_kv, actual_seq_offsets, NULL,
                   batch, total_query_tokens, heads, kv_heads, head_dim, 1, 0, causal, scale);
}

/* singe-kernel/src/cpu/attention.rs:1758-1833  fmha_prefill_lse_f32
 * query/out [B, L, H, D], key/value [B, S, G, D], lse [B, H, L] (natural log).
 * A row that sees no key (possible only when key_len == 0) gets max = -inf, denom = 0 and
 * lse = -inf + ln 0 = NaN in the Rust; callers never pass key_len == 0, and this port writes the
 * same expression. */
void oracle_fmha_prefill_lse_f32(float *out, float *lse, const float *query, const float *key, const float *value,
                                 size_t batch, size_t query_len, size_t key_len, size_t heads, size_t kv_heads,
                                 size_t head_dim, float scale, int causal) {
    size_t q_features = heads * head_dim;
    size_t kv_features = kv_heads * head_dim;
    size_t group = heads / kv_heads;
    memset(out, 0, batch * query_len * q_features * sizeof(float));
#pragma omp parallel for collapse(3) schedule(dynamic, 4)
    for (size_t b = 0; b < batch; ++b) {
        for (size_t head = 0; head < heads; ++head) {
            for (size_t qi = 0; qi < query_len; ++qi) {
                size_t kv_head = head / group;
                size_t visible = causal ? (qi + 1 < key_len ? qi + 1 : key_len) : key_len;
                float *scores = (float *)malloc((visible + 1) * sizeof(float));
                float *weights = (float *)malloc((visible + 1) * sizeof(float));
                const float *q = query + b * query_len * q_features + qi * q_features + head * head_dim;
                for (size_t k = 0; k < visible; ++k) {
                    const float *kp = key + b * key_len * kv_features + k * kv_features + kv_head * head_dim;
                    float score = 0.0f;
                    for (size_t d = 0; d < head_dim; ++d) score = fmaf(q[d], kp[d], score);
                    scores[k] = score * scale;
                }
                lse[b * heads * query_len + head * query_len + qi] =
                    softmax_weights(scores, weights, visible, NULL, NULL);
                float *o = out + b * query_len * q_features + qi * q_features + head * head_dim;
                for (size_t k = 0; k < visible; ++k) {
                    const float *vp = value + b * key_len * kv_features + k * kv_features + kv_head * head_dim;
                    for (size_t d = 0; d < head_dim; ++d) o[d] = fmaf(weights[k], vp[d], o[d]);
                }
                free(scores);
                free(weights);
            }
        }
    }
}

/* singe-kernel/src/cpu/attention.rs:1087-1170  sliding_window_attention_f32
 * A key is visible when key_abs <= query_abs and key_abs + window > query_abs. */
void oracle_sliding_window_attention_f32(float *out, const float *query, const float *key, const float *value,
                                         size_t batch, size_t query_len, size_t key_len, size_t heads,
                                         size_t kv_heads, size_t head_dim, size_t query_start, size_t key_start,
                                         size_t window, float scale, float output_scale) {
    size_t q_features = heads * head_dim;
    size_t kv_features = kv_heads * head_dim;
    size_t group = heads / kv_heads;
    memset(out, 0, batch * query_len * q_features * sizeof(float));
    for (size_t b = 0; b < batch; ++b) {
        for (size_t qi = 0; qi < query_len; ++qi) {
            size_t query_abs = query_start + qi;
            for (size_t head = 0; head < heads; ++head) {
                size_t kv_head = head / group;
                float *scores = (float *)malloc((key_len + 1) * sizeof(float));
                float *weights = (float *)malloc((key_len + 1) * sizeof(float));
                size_t *index = (size_t *)malloc((key_len + 1) * sizeof(size_t));
                size_t count = 0;
                const float *q = query + b * query_len * q_features + qi * q_features + head * head_dim;
                for (size_t k = 0; k < key_len; ++k) {
                    size_t key_abs = key_start + k;
                    if (key_abs > query_abs || key_abs + window <= query_abs) continue;
                    const float *kp = key + b * key_len * kv_features + k * kv_features + kv_head * head_dim;
                    float score = 0.0f;
                    for (size_t d = 0; d < head_dim; ++d) score = fmaf(q[d], kp[d], score);
                    scores[count] = score * scale;
                    index[count] = k;
                    ++count;
                }
                if (count != 0) {
                    softmax_weights(scores, weights, count, NULL, NULL);
                    float *o = out + b * query_len * q_features + qi * q_features + head * head_dim;
                    for (size_t d = 0; d < head_dim; ++d) {
                        float sum = 0.0f;
                        for (size_t i = 0; i < count; ++i) {
                            const float *vp =
                                value + b * key_len * kv_features + index[i] * kv_features + kv_head * head_dim;
                            sum = fmaf(weights[i], vp[d], sum);
                        }
                        o[d] = sum * output_scale;
                    }
                }
                free(scores);
                free(weights);
                free(index);
            }
        }
    }
}

/* singe-kernel/src/cpu/attention.rs:2157-2193  splitk_reduce_f32
 * attn [B, H, splits, D], lse [B, H, splits] (natural log); out [B, H, D]. */
void oracle_splitk_reduce_f32(float *out, const float *attn, const float *lse, size_t batch, size_t heads,
                              size_t splits, size_t head_dim) {
    for (size_t b = 0; b < batch; ++b) {
        for (size_t head = 0; head < heads; ++head) {
            const float *row_lse = lse + b * heads * splits + head * splits;
            float max_lse = -INFINITY;
            for (size_t s = 0; s < splits; ++s) max_lse = fmaxf(max_lse, row_lse[s]);
            float denom = 0.0f;
            for (size_t s = 0; s < splits; ++s) denom += expf(row_lse[s] - max_lse);
            for (size_t d = 0; d < head_dim; ++d) {
                float sum = 0.0f;
                for (size_t s = 0; s < splits; ++s) {
                    float weight = expf(row_lse[s] - max_lse);
                    sum = fmaf(weight, attn[b * heads * splits * head_dim + head * splits * head_dim + s * head_dim + d],
                               sum);
                }
                out[b * heads * head_dim + head * head_dim + d] = sum / denom;
            }
        }
    }
}

/* singe/src/backend/cpu/normalization/attention.rs:191-276  execute_scaled_dot_product_attention
 * Dense [B, H, L, D] queries over [B, H, S, D] keys/values (the caller has already repeated KV heads,
 * :20-130).  causal: end = min(S, i + 1); window (0 = none): start = (i + 1) saturating_sub window.
 * softcap (0 = none): score = tanh(score / cap) * cap after the scale (:250).  sinks (NULL = none): one logit per
 * head, batch_head % heads, which joins the row's max and its sum of exponentials and weighs no value (:253-263).
 * Mask and key_lengths are not on the hot path and are not restated. */
void oracle_attend_options_f32(float *out, const float *query, const float *key, const float *value,
                               size_t batch_heads, size_t query_len, size_t key_len, size_t head_dim,
                               size_t value_dim, float scale, int causal, size_t window, float softcap,
                               const float *sinks, size_t heads) {
#pragma omp parallel for schedule(dynamic, 8)
    for (size_t row = 0; row < batch_heads * query_len; ++row) {
        size_t batch_head = row / query_len;
        size_t qi = row % query_len;
        const float *q = query + row * head_dim;
        const float *keys = key + batch_head * key_len * head_dim;
        const float *values = value + batch_head * key_len * value_dim;
        size_t end = causal ? (qi + 1 < key_len ? qi + 1 : key_len) : key_len;
        size_t start = window ? (qi + 1 > window ? qi + 1 - window : 0) : 0;
        if (end < start) end = start;
        size_t count = end - start;
        float *o = out + row * value_dim;
        for (size_t f = 0; f < value_dim; ++f) o[f] = 0.0f;
        if (count == 0) continue;
        float *scores = (float *)malloc(count * sizeof(float));
        float max_score = -INFINITY;
        for (size_t k = 0; k < count; ++k) {
            const float *kp = keys + (start + k) * head_dim;
            float score = 0.0f;
            for (size_t d = 0; d < head_dim; ++d) score = fmaf(q[d], kp[d], score);
            score *= scale;
            if (softcap > 0.0f) score = tanhf(score / softcap) * softcap;
            scores[k] = score;
            max_score = fmaxf(max_score, score);
        }
        if (sinks) max_score = fmaxf(max_score, sinks[batch_head % (heads ? heads : 1)]);
        float score_sum = 0.0f;
        for (size_t k = 0; k < count; ++k) score_sum += expf(scores[k] - max_score);
        if (sinks) score_sum += expf(sinks[batch_head % (heads ? heads : 1)] - max_score);
        for (size_t k = 0; k < count; ++k) {
            const float *vp = values + (start + k) * value_dim;
            float weight = expf(scores[k] - max_score) / score_sum;
            for (size_t f = 0; f < value_dim; ++f) o[f] = fmaf(weight, vp[f], o[f]);
        }
        free(scores);
    }
}

void oracle_scaled_dot_product_attention_f32(float *out, const float *query, const float *key, const float *value,
                                             size_t batch_heads, size_t query_len, size_t key_len, size_t head_dim,
                                             size_t value_dim, float scale, int causal, size_t window) {
#pragma omp parallel for schedule(dynamic, 8)
    for (size_t row = 0; row < batch_heads * query_len; ++row) {
        size_t batch_head = row / query_len;
        size_t qi = row % query_len;
        const float *q = query + row * head_dim;
        const float *keys = key + batch_head * key_len * head_dim;
        const float *values = value + batch_head * key_len * value_dim;
        size_t end = causal ? (qi + 1 < key_len ? qi + 1 : key_len) : key_len;
        size_t start = window ? (qi + 1 > window ? qi + 1 - window : 0) : 0;
        if (end < start) end = start;
        size_t count = end - start;
        float *o = out + row * value_dim;
        for (size_t f = 0; f < value_dim; ++f) o[f] = 0.0f;
        if (count == 0) continue;
        float *scores = (float *)malloc(count * sizeof(float));
        float *weights = (float *)malloc(count * sizeof(float));
        for (size_t k = 0; k < count; ++k) {
            const float *kp = keys + (start + k) * head_dim;
            float score = 0.0f;
            for (size_t d = 0; d < head_dim; ++d) score = fmaf(q[d], kp[d], score);
            scores[k] = score * scale;
        }
        softmax_weights(scores, weights, count, NULL, NULL);
        for (size_t k = 0; k < count; ++k) {
            const float *vp = values + (start + k) * value_dim;
            for (size_t f = 0; f < value_dim; ++f) o[f] = fmaf(weights[k], vp[f], o[f]);
        }
        free(scores);
        free(weights);
    }
}

/* singe/src/backend/spec/neural/attention.rs:363-416  check_paged_values
 * Returns ORACLE_INDEX_OUT_OF_BOUNDS where the reference returns Error::IndexOutOfBounds. */
int oracle_check_paged_values(const int64_t *query_offsets, const int64_t *page_offsets, const int64_t *pages,
                              size_t table_len, const int64_t *last_page_lengths, size_t sequences, int64_t tokens,
                              int64_t cache_pages, int64_t page_size) {
    int64_t table = (int64_t)table_len;
    for (size_t s = 0; s < sequences; ++s) {
        int64_t qf = query_offsets[s], ql = query_offsets[s + 1];
        int64_t pf = page_offsets[s], pl = page_offsets[s + 1];
        if (!(0 <= qf && qf <= ql && ql <= tokens)) return ORACLE_INDEX_OUT_OF_BOUNDS;
        if (!(0 <= pf && pf <= pl && pl <= table)) return ORACLE_INDEX_OUT_OF_BOUNDS;
        if (pf == pl) continue; /* a sequence with no pages has no last page */
        if (last_page_lengths[s] < 0 || last_page_lengths[s] > page_size) return ORACLE_INDEX_OUT_OF_BOUNDS;
        for (int64_t i = pf; i < pl; ++i) {
            if (pages[i] < 0 || pages[i] >= cache_pages) return ORACLE_INDEX_OUT_OF_BOUNDS;
        }
    }
    return ORACLE_OK;
}

/* singe/src/backend/cpu/normalization/attention.rs:424-540  attend_paged (f32)
 * query/out [T, H, D], caches [P, S, G, D], FlashInfer-style paging; queries are the LAST tokens of
 * their sequence (position = keys - queries + i, :481-483); lse [T, H] is base 2 and -inf for a row
 * that sees no key (:459, :513-515).  window 0 = none.  softcap 0 = none, else score = tanh(score / cap) * cap
 * after the scale (:445, :500).
 * Note the accumulation here is `out = fma(weight/total, value, out)` per key (:519-523), and the
 * weights are exp(score - largest) kept un-normalised until that division. */
int oracle_attend_paged_options_f32(float *out, float *lse, const float *query, const float *key_cache,
                                    const float *value_cache, const int64_t *query_offsets,
                                    const int64_t *page_offsets, const int64_t *pages, size_t table_len,
                                    const int64_t *last_page_lengths, size_t sequences, size_t tokens, size_t heads,
                                    size_t kv_heads, size_t head_dim, size_t page_size, size_t cache_pages,
                                    float scale, int causal, size_t window, float softcap);

int oracle_attend_paged_f32(float *out, float *lse, const float *query, const float *key_cache,
                            const float *value_cache, const int64_t *query_offsets, const int64_t *page_offsets,
                            const int64_t *pages, size_t table_len, const int64_t *last_page_lengths,
                            size_t sequences, size_t tokens, size_t heads, size_t kv_heads, size_t head_dim,
                            size_t page_size, size_t cache_pages, float scale, int causal, size_t window) {
    return oracle_attend_paged_options_f32(out, lse, query, key_cache, value_cache, query_offsets, page_offsets, pages,
                                           table_len, last_page_lengths, sequences, tokens, heads, kv_heads, head_dim,
                                           page_size, cache_pages, scale, causal, window, 0.0f);
}

int oracle_attend_paged_options_f32(float *out, float *lse, const float *query, const float *key_cache,
                                    const float *value_cache, const int64_t *query_offsets,
                                    const int64_t *page_offsets, const int64_t *pages, size_t table_len,
                                    const int64_t *last_page_lengths, size_t sequences, size_t tokens, size_t heads,
                                    size_t kv_heads, size_t head_dim, size_t page_size, size_t cache_pages,
                                    float scale, int causal, size_t window, float softcap) {
    int status = oracle_check_paged_values(query_offsets, page_offsets, pages, table_len, last_page_lengths,
                                           sequences, (int64_t)tokens, (int64_t)cache_pages, (int64_t)page_size);
    if (status != ORACLE_OK) return status;
    size_t groups = heads / kv_heads;
    memset(out, 0, tokens * heads * head_dim * sizeof(float));
    for (size_t i = 0; i < tokens * heads; ++i) lse[i] = -INFINITY;
    const float ln2 = 0.69314718055994530942f; /* F32_LN_2 */
    for (size_t s = 0; s < sequences; ++s) {
        size_t first_query = (size_t)query_offsets[s], end_query = (size_t)query_offsets[s + 1];
        const int64_t *sequence_pages = pages + page_offsets[s];
        size_t page_count = (size_t)(page_offsets[s + 1] - page_offsets[s]);
        size_t last = last_page_lengths[s] > 0 ? (size_t)last_page_lengths[s] : 0;
        size_t keys = page_count == 0 ? 0 : (page_count - 1) * page_size + last;
        size_t queries = end_query - first_query;
#pragma omp parallel for collapse(2) schedule(dynamic, 4)
        for (size_t token = first_query; token < end_query; ++token) {
            for (size_t head = 0; head < heads; ++head) {
                size_t shifted = keys + token - first_query;
                size_t position = shifted > queries ? shifted - queries : 0;
                size_t end = causal ? (position + 1 < keys ? position + 1 : keys) : keys;
                size_t start = window ? (position + 1 > window ? position + 1 - window : 0) : 0;
                if (end <= start) continue;
                size_t count = end - start;
                size_t kv_head = head / groups;
                const float *row = query + (token * heads + head) * head_dim;
                float *scores = (float *)malloc(count * sizeof(float));
                float largest = -INFINITY;
                for (size_t k = 0; k < count; ++k) {
                    size_t pos = start + k;
                    size_t slot = (size_t)sequence_pages[pos / page_size] * page_size + pos % page_size;
                    const float *kp = key_cache + (slot * kv_heads + kv_head) * head_dim;
                    float score = 0.0f;
                    for (size_t d = 0; d < head_dim; ++d) score = fmaf(row[d], kp[d], score);
                    scores[k] = score * scale;
                    if (softcap > 0.0f) scores[k] = tanhf(scores[k] / softcap) * softcap;
                    largest = fmaxf(largest, scores[k]);
                }
                float total = 0.0f;
                for (size_t k = 0; k < count; ++k) {
                    scores[k] = expf(scores[k] - largest);
                    total += scores[k];
                }
                lse[token * heads + head] = (largest + logf(total)) / ln2;
                float *o = out + (token * heads + head) * head_dim;
                for (size_t k = 0; k < count; ++k) {
                    size_t pos = start + k;
                    size_t slot = (size_t)sequence_pages[pos / page_size] * page_size + pos % page_size;
                    const float *vp = value_cache + (slot * kv_heads + kv_head) * head_dim;
                    float weight = scores[k] / total;
                    for (size_t d = 0; d < head_dim; ++d) o[d] = fmaf(weight, vp[d], o[d]);
                }
                free(scores);
            }
        }
    }
    return ORACLE_OK;
}

/* singe-kernel/src/cpu/matmul/mod.rs:12-45  matmul_f32 -- the naive reference-order GEMM.
 * sum += lhs * rhs with separate rounding, ascending k. */
void oracle_matmul_f32(float *out, const float *lhs, const float *rhs, size_t rows, size_t columns,
                       size_t reduction, size_t lhs_row_stride, size_t rhs_row_stride, int transpose_lhs,
                       int transpose_rhs) {
#pragma omp parallel for schedule(static)
    for (size_t row = 0; row < rows; ++row) {
        for (size_t column = 0; column < columns; ++column) {
            float sum = 0.0f;
            for (size_t k = 0; k < reduction; ++k) {
                size_t li = transpose_lhs ? k * lhs_row_stride + row : row * lhs_row_stride + k;
                size_t ri = transpose_rhs ? column * rhs_row_stride + k : k * rhs_row_stride + column;
                float product = lhs[li] * rhs[ri];
                sum = sum + product;
            }
            out[row * columns + column] = sum;
        }
    }
}

static int validate_span(size_t values, size_t rows, size_t columns, size_t s0, size_t s1, size_t *minimum) {
    /* singe-kernel/src/cpu/matmul/blocked.rs:3-25 */
    if (rows == 0 || columns == 0) return ORACLE_OK;
    size_t a, b, c;
    if (__builtin_mul_overflow(rows - 1, s0, &a)) return ORACLE_SIZE_OVERFLOW;
    if (__builtin_mul_overflow(columns - 1, s1, &b)) return ORACLE_SIZE_OVERFLOW;
    if (__builtin_add_overflow(a, b, &c)) return ORACLE_SIZE_OVERFLOW;
    if (__builtin_add_overflow(c, (size_t)1, &c)) return ORACLE_SIZE_OVERFLOW;
    if (minimum) *minimum = c;
    if (c > values) return ORACLE_LENGTH_TOO_SHORT;
    return ORACLE_OK;
}

/* singe-kernel/src/cpu/matmul/blocked.rs:27-95  matmul_strided_f32 -- the blocked GEMM the Tensor
 * surface calls.  Tiles 16 rows x 64 columns x 32 deep when the right operand has unit column
 * stride, else per-element dot products; either way each output sees ascending k. */
int oracle_matmul_strided_f32(const float *lhs, size_t lhs_len, const float *rhs, size_t rhs_len, float *output,
                              size_t output_len, size_t rows, size_t columns, size_t reduction, size_t ls0,
                              size_t ls1, size_t rs0, size_t rs1) {
    size_t count;
    if (__builtin_mul_overflow(rows, columns, &count)) return ORACLE_SIZE_OVERFLOW;
    if (output_len != count) return ORACLE_LENGTH_MISMATCH;
    if (count == 0) return ORACLE_OK;
    int status = validate_span(lhs_len, rows, reduction, ls0, ls1, NULL);
    if (status) return status;
    status = validate_span(rhs_len, reduction, columns, rs0, rs1, NULL);
    if (status) return status;
    for (size_t i = 0; i < count; ++i) output[i] = 0.0f;
    if (rs1 != 1) {
#pragma omp parallel for schedule(static)
        for (size_t row = 0; row < rows; ++row) {
            for (size_t column = 0; column < columns; ++column) {
                float sum = 0.0f;
                for (size_t k = 0; k < reduction; ++k) {
                    float product = lhs[row * ls0 + k * ls1] * rhs[k * rs0 + column * rs1];
                    sum = sum + product;
                }
                output[row * columns + column] = sum;
            }
        }
        return ORACLE_OK;
    }
    for (size_t row_start = 0; row_start < rows; row_start += 16) {
        for (size_t column_start = 0; column_start < columns; column_start += 64) {
            size_t column_end = columns < column_start + 64 ? columns : column_start + 64;
            for (size_t k_start = 0; k_start < reduction; k_start += 32) {
                size_t row_end = rows < row_start + 16 ? rows : row_start + 16;
                size_t k_end = reduction < k_start + 32 ? reduction : k_start + 32;
                for (size_t row = row_start; row < row_end; ++row) {
                    float *o = output + row * columns;
                    for (size_t k = k_start; k < k_end; ++k) {
                        float a = lhs[row * ls0 + k * ls1];
                        const float *b = rhs + k * rs0;
                        for (size_t column = column_start; column < column_end; ++column) {
                            float product = a * b[column];
                            o[column] = o[column] + product;
                        }
                    }
                }
            }
        }
    }
    return ORACLE_OK;
}

/* singe/src/backend/cpu/binary/matmul.rs:18-43 + Linear::forward (singe/src/nn/layers/linear/mod.rs:49-70):
 * Y[M, N] = X[M, K] . W[N, K]^T with bf16 operands widened to f32, multiplied by matmul_strided_f32
 * with rhs strides [1, K] (so the transposed branch runs), and rounded ONCE to bf16.
 * `x_bits`, `w_bits` and `y_bits` are raw bf16 bit patterns. */
void oracle_linear_bf16(uint16_t *y_bits, const uint16_t *x_bits, const uint16_t *w_bits, size_t m, size_t n,
                        size_t k) {
#pragma omp parallel for schedule(static)
    for (size_t row = 0; row < m; ++row) {
        float *x = (float *)malloc(k * sizeof(float));
        for (size_t i = 0; i < k; ++i) x[i] = oracle_bf16_bits_to_f32(x_bits[row * k + i]);
        for (size_t column = 0; column < n; ++column) {
            const uint16_t *w = w_bits + column * k;
            float sum = 0.0f;
            for (size_t i = 0; i < k; ++i) {
                float product = x[i] * oracle_bf16_bits_to_f32(w[i]);
                sum = sum + product;
            }
            y_bits[row * n + column] = oracle_f32_to_bf16_bits(sum);
        }
        free(x);
    }
}

/* Same product kept in f32 (the singe-kernel surface: matmul_bf16_f32, singe-kernel/src/cuda/matmul.rs:1302-1339
 * checked against cpu::matmul_f32). */
void oracle_linear_bf16_f32(float *y, const uint16_t *x_bits, const uint16_t *w_bits, size_t m, size_t n, size_t k) {
#pragma omp parallel for schedule(static)
    for (size_t row = 0; row < m; ++row) {
        float *x = (float *)malloc(k * sizeof(float));
        for (size_t i = 0; i < k; ++i) x[i] = oracle_bf16_bits_to_f32(x_bits[row * k + i]);
        for (size_t column = 0; column < n; ++column) {
            const uint16_t *w = w_bits + column * k;
            float sum = 0.0f;
            for (size_t i = 0; i < k; ++i) {
                float product = x[i] * oracle_bf16_bits_to_f32(w[i]);
                sum = sum + product;
            }
            y[row * n + column] = sum;
        }
        free(x);
    }
}

/* KvCache::write (singe/src/nn/decode/cache.rs:97-101) = index_put_ at (write_pages, write_slots),
 * restating index_write / plan (singe/src/backend/cpu/shape/multi_index.rs:95-125, 204-236):
 * a negative index wraps by its extent, anything still outside refuses the whole write before a
 * byte moves, rows are copied in index order so the last duplicate wins.
 * cache [P, S, row_bytes], rows [T, row_bytes] as raw bytes. */
int oracle_kv_cache_write(uint8_t *cache, const uint8_t *rows, const int64_t *write_pages, const int64_t *write_slots,
                          size_t tokens, size_t pages, size_t page_size, size_t row_bytes) {
    size_t *positions = (size_t *)malloc((tokens ? tokens : 1) * sizeof(size_t));
    for (size_t t = 0; t < tokens; ++t) {
        int64_t page = write_pages[t] < 0 ? write_pages[t] + (int64_t)pages : write_pages[t];
        int64_t slot = write_slots[t] < 0 ? write_slots[t] + (int64_t)page_size : write_slots[t];
        if (page < 0 || page >= (int64_t)pages || slot < 0 || slot >= (int64_t)page_size) {
            free(positions);
            return ORACLE_INDEX_OUT_OF_BOUNDS;
        }
        positions[t] = (size_t)page * page_size + (size_t)slot;
    }
    for (size_t t = 0; t < tokens; ++t) memcpy(cache + positions[t] * row_bytes, rows + t * row_bytes, row_bytes);
    free(positions);
    return ORACLE_OK;
}

/* ------------------------------------------------------------------------------------------------
 * Decode-step glue (Llama block), f32 math on bf16-rounded tensors as the reference's widened CPU
 * kernels do (singe/src/backend/kernels.rs:662-705: narrower floats are cast to f32, computed, cast back).
 * ------------------------------------------------------------------------------------------------ */

/* RmsNorm: singe-kernel/src/cpu/normalization/standard.rs:43-60  x * rsqrt(mean(x^2) + eps) * w in f32. */
void oracle_rms_norm_f32(float *out, const float *input, const float *weight, size_t rows, size_t width, float eps) {
    for (size_t r = 0; r < rows; ++r) {
        const float *x = input + r * width;
        float sum = 0.0f;
        for (size_t i = 0; i < width; ++i) sum += x[i] * x[i];
        float inv = 1.0f / sqrtf(sum / (float)width + eps);
        for (size_t i = 0; i < width; ++i) out[r * width + i] = x[i] * inv * weight[i];
    }
}
