// Decode-step glue around the attention and GEMM kernels, bf16 tensors with f32 arithmetic inside:
// embedding lookup, RMSNorm (alone and fused with the residual add), half-split rotary embedding fused with
// the slot-mapped KV-cache write, SwiGLU activation, and the last-row argmax.
//
// Meaning follows the reference's Llama block (singe/src/nn/layers/blocks/mod.rs:56-83):
//   h += o_proj(attn(norm(h)));  h += down(silu(gate(norm h)) * up(norm h))
// with RmsNorm = x * 1/sqrt(mean(x^2) + eps) * w in f32 (singe/src/backend/cpu/normalization/standard.rs:43-60),
// the half-split rotation of RotaryAngles::rotate_pairs (singe/src/nn/layers/positional/rotary.rs:274-304) and
// KvCache::write (singe/src/nn/decode/cache.rs:97-101).  The reference runs these as separate bf16 tensor ops, each
// rounding its result to bf16; the fused kernels here keep those roundings (product, then sum) so results match
// the unfused chain.  All of them move a few hundred KB per step: one CTA per row, 128-bit accesses.
#include "common.cuh"

namespace singe {
namespace {

bool aligned16(const void *pointer) { return (reinterpret_cast<uintptr_t>(pointer) & 15u) == 0; }

__device__ __forceinline__ float round_bf16(float value) { return __bfloat162float(__float2bfloat16_rn(value)); }

__device__ __forceinline__ float block_sum(float value, float *scratch) {
    value = warp_sum(value);
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    if (lane == 0) scratch[warp] = value;
    __syncthreads();
    float total = 0.0f;
    const int warps = (blockDim.x + 31) >> 5;
    for (int i = 0; i < warps; ++i) total += scratch[i];
    __syncthreads();
    return total;
}

// ---- 128-bit helpers: eight bf16 per access ----
struct Vec8 {
    float v[8];
};

__device__ __forceinline__ Vec8 load8(const __nv_bfloat16 *pointer) {
    const uint4 raw = *reinterpret_cast<const uint4 *>(pointer);
    const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
    Vec8 out;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        out.v[2 * i] = __uint_as_float(words[i] << 16);
        out.v[2 * i + 1] = __uint_as_float(words[i] & 0xffff0000u);
    }
    return out;
}

__device__ __forceinline__ void store8(__nv_bfloat16 *pointer, const Vec8 &value) {
    uint4 raw;
    raw.x = pack2<__nv_bfloat16>(value.v[0], value.v[1]);
    raw.y = pack2<__nv_bfloat16>(value.v[2], value.v[3]);
    raw.z = pack2<__nv_bfloat16>(value.v[4], value.v[5]);
    raw.w = pack2<__nv_bfloat16>(value.v[6], value.v[7]);
    *reinterpret_cast<uint4 *>(pointer) = raw;
}

// VEC = 8: rows are multiples of eight bf16 and every pointer is 16-byte aligned; VEC = 1 otherwise.
template <typename Index, int VEC>
__global__ void embedding_kernel(__nv_bfloat16 *out, const __nv_bfloat16 *table, const Index *ids, int width,
                                 long long vocab, uint32_t *status) {
    grid_launch_dependents();
    grid_dependency_wait();
    const int row = blockIdx.x;
    long long id = static_cast<long long>(ids[row]);
    if (id < 0) id += vocab;  // negative indices wrap, as index_select does
    const bool valid = id >= 0 && id < vocab;
    if (!valid && threadIdx.x == 0) report_status(status, kStatusIndexOutOfBounds);
    __nv_bfloat16 *target = out + static_cast<size_t>(row) * width;
    const __nv_bfloat16 *source = table + static_cast<size_t>(valid ? id : 0) * width;
    for (int c = threadIdx.x * VEC; c < width; c += blockDim.x * VEC) {
        if (VEC == 8) {
            *reinterpret_cast<uint4 *>(target + c) =
                valid ? *reinterpret_cast<const uint4 *>(source + c) : make_uint4(0u, 0u, 0u, 0u);
        } else {
            target[c] = valid ? source[c] : __float2bfloat16_rn(0.0f);
        }
    }
}

// hidden (+)= delta (rounded to bf16, as Tensor::add does), then normed = rms_norm(hidden) * weight.
// delta == nullptr: plain RMSNorm of `hidden`.  normed == nullptr: residual add only.
// One CTA per row; with VEC = 8 a thread keeps up to kHeld chunks of eight values in registers between the
// sum-of-squares pass and the scaling pass, so rows up to blockDim * 8 * kHeld wide are read once.
constexpr int kHeld = 4;

template <int VEC>
__global__ void add_rms_norm_kernel(__nv_bfloat16 *hidden, const __nv_bfloat16 *delta, __nv_bfloat16 *normed,
                                    const __nv_bfloat16 *weight, int width, float eps, const WarmRange warm) {
    grid_launch_dependents();
    if (threadIdx.x < 32) warm_l2(warm, blockIdx.x, gridDim.x, threadIdx.x);
    grid_dependency_wait();
    __shared__ float scratch[32];
    const size_t base = static_cast<size_t>(blockIdx.x) * width;
    float square = 0.0f;
    if (VEC == 8) {
        Vec8 held[kHeld];
        const int stride = blockDim.x * 8;
#pragma unroll
        for (int h = 0; h < kHeld; ++h) {
            const int c = threadIdx.x * 8 + h * stride;
            if (c < width) {
                held[h] = load8(hidden + base + c);
                if (delta != nullptr) {
                    const Vec8 other = load8(delta + base + c);
#pragma unroll
                    for (int i = 0; i < 8; ++i) held[h].v[i] = round_bf16(held[h].v[i] + other.v[i]);
                    store8(hidden + base + c, held[h]);
                }
#pragma unroll
                for (int i = 0; i < 8; ++i) square = square_chain(square, held[h].v[i]);
            }
        }
        for (int c = threadIdx.x * 8 + kHeld * stride; c < width; c += stride) {  // rows wider than the held part
            Vec8 value = load8(hidden + base + c);
            if (delta != nullptr) {
                const Vec8 other = load8(delta + base + c);
#pragma unroll
                for (int i = 0; i < 8; ++i) value.v[i] = round_bf16(value.v[i] + other.v[i]);
                store8(hidden + base + c, value);
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) square = square_chain(square, value.v[i]);
        }
        if (normed == nullptr) return;
        const float total = block_sum(square, scratch);
        const float scale = 1.0f / sqrtf(total / static_cast<float>(width) + eps);
#pragma unroll
        for (int h = 0; h < kHeld; ++h) {
            const int c = threadIdx.x * 8 + h * stride;
            if (c < width) {
                const Vec8 gain = load8(weight + c);
                Vec8 result;
#pragma unroll
                for (int i = 0; i < 8; ++i) result.v[i] = held[h].v[i] * scale * gain.v[i];
                store8(normed + base + c, result);
            }
        }
        for (int c = threadIdx.x * 8 + kHeld * stride; c < width; c += stride) {
            const Vec8 value = load8(hidden + base + c);
            const Vec8 gain = load8(weight + c);
            Vec8 result;
#pragma unroll
            for (int i = 0; i < 8; ++i) result.v[i] = value.v[i] * scale * gain.v[i];
            store8(normed + base + c, result);
        }
        return;
    }
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float value = __bfloat162float(hidden[base + c]);
        if (delta != nullptr) {
            value = round_bf16(value + __bfloat162float(delta[base + c]));
            hidden[base + c] = __float2bfloat16_rn(value);
        }
        square = square_chain(square, value);
    }
    if (normed == nullptr) return;
    const float total = block_sum(square, scratch);
    const float scale = 1.0f / sqrtf(total / static_cast<float>(width) + eps);
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float value = __bfloat162float(hidden[base + c]);
        normed[base + c] = __float2bfloat16_rn(value * scale * __bfloat162float(weight[c]));
    }
}

// One CTA per token.  qkv row = [heads*D | kv_heads*D | kv_heads*D].  Rotates Q into q_out and K into the cache at
// (write_pages[t], write_slots[t]); V is copied into the cache.  Rounding follows the tensor-op chain of
// rotate_pairs: first' = bf16(bf16(first*cos) - bf16(second*sin)), second' = bf16(bf16(second*cos) + bf16(first*sin)).
// With VEC = 8 a thread rotates eight adjacent pairs (head_dim/2 is then a multiple of eight).
// Per-head RMSNorm before the rotation (RotationNorm, query_norm / key_norm of RotaryCacheInputs,
// singe/src/backend/cuda/kernel_plan/source/rotary_cache.rs:25-52): each head's D values are scaled by
// 1 / sqrt(mean(x^2) + eps) and its gain, rounded to bf16 as the separate RmsNorm op would return them, then rotated.
// The threads of one head are adjacent lanes of one warp, so the head's sum of squares is a few shuffles.
struct HeadNorms {
    const __nv_bfloat16 *query_weight;  // [head_dim] gain, or nullptr for none
    const __nv_bfloat16 *key_weight;
    int query;                          // 1: normalise the query heads
    int key;                            // 1: normalise the key heads
    float eps;
};

template <typename Index, int VEC>
__global__ void rotary_cache_write_kernel(__nv_bfloat16 *q_out, const __nv_bfloat16 *qkv, long long qkv_stride,
                                          const __nv_bfloat16 *cos_table, const __nv_bfloat16 *sin_table,
                                          const Index *positions, __nv_bfloat16 *key_cache,
                                          __nv_bfloat16 *value_cache, const Index *write_pages,
                                          const Index *write_slots, int heads, int kv_heads, int head_dim,
                                          long long pages, long long page_size, long long capacity,
                                          uint32_t *status, const WarmRange warm, const HeadNorms norms) {
    grid_launch_dependents();
    if (threadIdx.x < 32) warm_l2(warm, blockIdx.x, gridDim.x, threadIdx.x);
    grid_dependency_wait();
    const int token = blockIdx.x;
    const int half = head_dim >> 1;
    long long position = static_cast<long long>(positions[token]);
    if (position < 0) position += capacity;
    long long page = static_cast<long long>(write_pages[token]);
    long long slot = static_cast<long long>(write_slots[token]);
    if (page < 0) page += pages;
    if (slot < 0) slot += page_size;
    const bool position_ok = position >= 0 && position < capacity;
    const bool slot_ok = page >= 0 && page < pages && slot >= 0 && slot < page_size;
    if ((!position_ok || !slot_ok) && threadIdx.x == 0) report_status(status, kStatusIndexOutOfBounds);
    if (!position_ok) return;
    const __nv_bfloat16 *row = qkv + static_cast<size_t>(token) * qkv_stride;
    const __nv_bfloat16 *cos_row = cos_table + static_cast<size_t>(position) * half;
    const __nv_bfloat16 *sin_row = sin_table + static_cast<size_t>(position) * half;
    const size_t cache_row = (static_cast<size_t>(page) * page_size + slot) * kv_heads * head_dim;
    const int rotated_heads = heads + kv_heads;
    const int per_head = half / VEC;   // threads of one head: adjacent lanes (a power of two <= 32 when a norm is asked for)
    const bool any_norm = norms.query != 0 || norms.key != 0;
    const int items = rotated_heads * per_head;
    // With a norm every lane of a warp must reach the shuffles: the loop runs in whole warps.
    const int bound = any_norm ? (items + 31) / 32 * 32 : items;
    for (int item = threadIdx.x; item < bound; item += blockDim.x) {
        const bool live = item < items;
        const int head = live ? item / per_head : 0;
        const int i = live ? (item - head * per_head) * VEC : 0;
        const __nv_bfloat16 *source = row + static_cast<size_t>(head) * head_dim;
        __nv_bfloat16 *target = nullptr;
        if (live && head < heads) {
            target = q_out + (static_cast<size_t>(token) * heads + head) * head_dim;
        } else if (live && slot_ok) {
            target = key_cache + cache_row + static_cast<size_t>(head - heads) * head_dim;
        }
        const bool normalise = live && (head < heads ? norms.query != 0 : norms.key != 0);
        const __nv_bfloat16 *gain = head < heads ? norms.query_weight : norms.key_weight;
        if (VEC == 8) {
            Vec8 first, second;
            if (live) {
                first = load8(source + i);
                second = load8(source + i + half);
            }
            if (any_norm) {
                float squares = 0.0f;
                if (normalise) {
#pragma unroll
                    for (int e = 0; e < 8; ++e) squares += first.v[e] * first.v[e] + second.v[e] * second.v[e];
                }
                for (int offset = 1; offset < per_head; offset <<= 1) {
                    squares += __shfl_xor_sync(0xffffffffu, squares, offset);
                }
                if (normalise) {
                    const float scale = 1.0f / sqrtf(squares / static_cast<float>(head_dim) + norms.eps);
                    Vec8 gain_first, gain_second;
#pragma unroll
                    for (int e = 0; e < 8; ++e) gain_first.v[e] = gain_second.v[e] = 1.0f;
                    if (gain != nullptr) {
                        gain_first = load8(gain + i);
                        gain_second = load8(gain + i + half);
                    }
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        first.v[e] = round_bf16(first.v[e] * scale * gain_first.v[e]);
                        second.v[e] = round_bf16(second.v[e] * scale * gain_second.v[e]);
                    }
                }
            }
            if (target == nullptr) continue;
            const Vec8 c = load8(cos_row + i), s = load8(sin_row + i);
            Vec8 out_first, out_second;
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                out_first.v[e] = round_bf16(first.v[e] * c.v[e]) - round_bf16(second.v[e] * s.v[e]);
                out_second.v[e] = round_bf16(second.v[e] * c.v[e]) + round_bf16(first.v[e] * s.v[e]);
            }
            store8(target + i, out_first);
            store8(target + i + half, out_second);
        } else {
            float first = live ? __bfloat162float(source[i]) : 0.0f;
            float second = live ? __bfloat162float(source[i + half]) : 0.0f;
            if (any_norm) {
                float squares = normalise ? first * first + second * second : 0.0f;
                for (int offset = 1; offset < per_head; offset <<= 1) {
                    squares += __shfl_xor_sync(0xffffffffu, squares, offset);
                }
                if (normalise) {
                    const float scale = 1.0f / sqrtf(squares / static_cast<float>(head_dim) + norms.eps);
                    const float g_first = gain != nullptr ? __bfloat162float(gain[i]) : 1.0f;
                    const float g_second = gain != nullptr ? __bfloat162float(gain[i + half]) : 1.0f;
                    first = round_bf16(first * scale * g_first);
                    second = round_bf16(second * scale * g_second);
                }
            }
            if (target == nullptr) continue;
            const float c = __bfloat162float(cos_row[i]);
            const float s = __bfloat162float(sin_row[i]);
            target[i] = __float2bfloat16_rn(round_bf16(first * c) - round_bf16(second * s));
            target[i + half] = __float2bfloat16_rn(round_bf16(second * c) + round_bf16(first * s));
        }
    }
    if (slot_ok) {
        const __nv_bfloat16 *values = row + static_cast<size_t>(heads + kv_heads) * head_dim;
        for (int c = threadIdx.x * VEC; c < kv_heads * head_dim; c += blockDim.x * VEC) {
            if (VEC == 8) {
                *reinterpret_cast<uint4 *>(value_cache + cache_row + c) = *reinterpret_cast<const uint4 *>(values + c);
            } else {
                value_cache[cache_row + c] = values[c];
            }
        }
    }
}

// out = bf16(bf16(silu(gate)) * up), the two roundings of activation-then-mul in GatedMlp
// (singe/src/nn/layers/feed_forward/mod.rs:58-66).  Elementwise: grid (column chunks, rows).
template <int VEC>
__global__ void silu_mul_kernel(__nv_bfloat16 *out, const __nv_bfloat16 *gate, const __nv_bfloat16 *up,
                                long long in_stride, int width) {
    grid_launch_dependents();
    grid_dependency_wait();
    const size_t in_base = static_cast<size_t>(blockIdx.y) * in_stride;
    const size_t out_base = static_cast<size_t>(blockIdx.y) * width;
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * VEC;
    if (c >= width) return;
    if (VEC == 8) {
        const Vec8 g = load8(gate + in_base + c), u = load8(up + in_base + c);
        Vec8 result;
#pragma unroll
        for (int i = 0; i < 8; ++i) result.v[i] = round_bf16(silu_fast(g.v[i])) * u.v[i];
        store8(out + out_base + c, result);
    } else {
        const float g = __bfloat162float(gate[in_base + c]);
        const float u = __bfloat162float(up[in_base + c]);
        out[out_base + c] = __float2bfloat16_rn(round_bf16(silu_fast(g)) * u);
    }
}

// Row-wise argmax; ties go to the lowest index.  Writes the winning value (f32) and index (int64, plus
// `index_offset` so that a vocabulary shard reports global token ids).  NaN logits never win.
template <int VEC>
__global__ void argmax_kernel(float *best_value, long long *best_index, const __nv_bfloat16 *logits,
                              long long stride, int width, long long index_offset) {
    grid_launch_dependents();
    grid_dependency_wait();
    __shared__ float values[32];
    __shared__ int indices[32];
    const __nv_bfloat16 *row = logits + static_cast<size_t>(blockIdx.x) * stride;
    float best = -INFINITY;
    int where = 0x7fffffff;
    for (int c = threadIdx.x * VEC; c < width; c += blockDim.x * VEC) {
        if (VEC == 8) {
            const Vec8 chunk = load8(row + c);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                if (chunk.v[i] > best) {  // ascending scan: a later equal value never replaces an earlier one
                    best = chunk.v[i];
                    where = c + i;
                }
            }
        } else {
            const float value = __bfloat162float(row[c]);
            if (value > best) {
                best = value;
                where = c;
            }
        }
    }
    for (int offset = 16; offset > 0; offset >>= 1) {
        const float other = __shfl_xor_sync(0xffffffffu, best, offset);
        const int other_where = __shfl_xor_sync(0xffffffffu, where, offset);
        if (other > best || (other == best && other_where < where)) {
            best = other;
            where = other_where;
        }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) {
        values[warp] = best;
        indices[warp] = where;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        const int warps = (blockDim.x + 31) >> 5;
        for (int i = 1; i < warps; ++i) {
            if (values[i] > best || (values[i] == best && indices[i] < where)) {
                best = values[i];
                where = indices[i];
            }
        }
        best_value[blockIdx.x] = best;
        best_index[blockIdx.x] = static_cast<long long>(where) + index_offset;
    }
}

}  // namespace
}  // namespace singe

using namespace singe;

extern "C" {

int singe_embedding_bf16(singe_stream_t stream, void *out, const void *table, const void *ids, int index_width,
                         size_t tokens, size_t width, size_t vocab, uint32_t *status) {
    if (tokens == 0 || width == 0 || vocab == 0) return SINGE_ERR_INVALID_LENGTH;
    if (!fits_i32(tokens) || !fits_i32(width) || !fits_i32(vocab)) return SINGE_ERR_LENGTH_EXCEEDS_I32;
    if (out == nullptr || table == nullptr || ids == nullptr) return SINGE_ERR_NULL_POINTER;
    if (index_width != 4 && index_width != 8) return SINGE_ERR_INVALID_ARGUMENT;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool wide = width % 8 == 0 && aligned16(out) && aligned16(table);
#define SINGE_EMBED(Index, VEC)                                                                              \
    launch_dependent(embedding_kernel<Index, VEC>, dim3(static_cast<unsigned>(tokens)), dim3(256), 0, s, kLaunchGlue, 1,  \
        static_cast<__nv_bfloat16 *>(out), static_cast<const __nv_bfloat16 *>(table),                        \
        static_cast<const Index *>(ids), static_cast<int>(width), static_cast<long long>(vocab), status)
    if (index_width == 8) {
        if (wide) SINGE_EMBED(long long, 8); else SINGE_EMBED(long long, 1);
    } else {
        if (wide) SINGE_EMBED(int, 8); else SINGE_EMBED(int, 1);
    }
#undef SINGE_EMBED
    return launch_status();
}

int singe_add_rms_norm_bf16(singe_stream_t stream, void *hidden, const void *delta, void *normed, const void *weight,
                            size_t rows, size_t width, float eps) {
    if (rows == 0 || width == 0) return SINGE_ERR_INVALID_LENGTH;
    if (!fits_i32(rows) || !fits_i32(width)) return SINGE_ERR_LENGTH_EXCEEDS_I32;
    if (hidden == nullptr || (normed != nullptr && weight == nullptr) || (normed == nullptr && delta == nullptr)) {
        return SINGE_ERR_NULL_POINTER;
    }
    const bool wide = width % 8 == 0 && aligned16(hidden) && aligned16(delta) && aligned16(normed) && aligned16(weight);
    const WarmRange warm = take_pending_warm();
    if (wide) {
        int threads = static_cast<int>((width / 8 + 31) / 32 * 32);
        if (threads > 512) threads = 512;
        launch_dependent(add_rms_norm_kernel<8>, dim3(static_cast<unsigned>(rows)), dim3(threads), 0,
                         static_cast<cudaStream_t>(stream), kLaunchGlue, 1,
            static_cast<__nv_bfloat16 *>(hidden), static_cast<const __nv_bfloat16 *>(delta),
            static_cast<__nv_bfloat16 *>(normed), static_cast<const __nv_bfloat16 *>(weight),
            static_cast<int>(width), eps, warm);
    } else {
        launch_dependent(add_rms_norm_kernel<1>, dim3(static_cast<unsigned>(rows)), dim3(256), 0,
                         static_cast<cudaStream_t>(stream), kLaunchGlue, 1,
            static_cast<__nv_bfloat16 *>(hidden), static_cast<const __nv_bfloat16 *>(delta),
            static_cast<__nv_bfloat16 *>(normed), static_cast<const __nv_bfloat16 *>(weight),
            static_cast<int>(width), eps, warm);
    }
    return launch_status();
}

static int rotary_cache_write(singe_stream_t stream, void *q_out, const void *qkv, size_t qkv_row_stride,
                              const void *cos_table, const void *sin_table, const void *positions, void *key_cache,
                              void *value_cache, const void *write_pages, const void *write_slots, int index_width,
                              size_t tokens, size_t heads, size_t kv_heads, size_t head_dim, size_t pages,
                              size_t page_size, size_t capacity, uint32_t *status, const HeadNorms &norms) {
    if (tokens == 0 || heads == 0 || kv_heads == 0 || head_dim == 0 || head_dim % 2 != 0 || pages == 0 ||
        page_size == 0 || capacity == 0 || qkv_row_stride < (heads + 2 * kv_heads) * head_dim) {
        return SINGE_ERR_INVALID_LENGTH;
    }
    if (!fits_i32(tokens) || !fits_i32(heads) || !fits_i32(kv_heads) || !fits_i32(head_dim) || !fits_i32(pages) ||
        !fits_i32(page_size) || !fits_i32(capacity)) {
        return SINGE_ERR_LENGTH_EXCEEDS_I32;
    }
    if (q_out == nullptr || qkv == nullptr || cos_table == nullptr || sin_table == nullptr || positions == nullptr ||
        key_cache == nullptr || value_cache == nullptr || write_pages == nullptr || write_slots == nullptr) {
        return SINGE_ERR_NULL_POINTER;
    }
    if (index_width != 4 && index_width != 8) return SINGE_ERR_INVALID_ARGUMENT;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool wide = (head_dim / 2) % 8 == 0 && qkv_row_stride % 8 == 0 && aligned16(q_out) && aligned16(qkv) &&
                      aligned16(cos_table) && aligned16(sin_table) && aligned16(key_cache) && aligned16(value_cache) &&
                      aligned16(norms.query_weight) && aligned16(norms.key_weight);
    if (norms.query != 0 || norms.key != 0) {
        // a head's threads must be adjacent lanes of one warp
        const size_t per_head = wide ? head_dim / 16 : head_dim / 2;
        if (per_head > 32 || (per_head & (per_head - 1)) != 0 || !(norms.eps == norms.eps)) {
            return SINGE_ERR_UNSUPPORTED_CONFIGURATION;
        }
    }
#define SINGE_ROTARY(Index, VEC)                                                                                     \
    launch_dependent(rotary_cache_write_kernel<Index, VEC>, dim3(static_cast<unsigned>(tokens)), dim3(256), 0, s, kLaunchGlue, 1, \
        static_cast<__nv_bfloat16 *>(q_out), static_cast<const __nv_bfloat16 *>(qkv),                                \
        static_cast<long long>(qkv_row_stride), static_cast<const __nv_bfloat16 *>(cos_table),                       \
        static_cast<const __nv_bfloat16 *>(sin_table), static_cast<const Index *>(positions),                        \
        static_cast<__nv_bfloat16 *>(key_cache), static_cast<__nv_bfloat16 *>(value_cache),                          \
        static_cast<const Index *>(write_pages), static_cast<const Index *>(write_slots), static_cast<int>(heads),   \
        static_cast<int>(kv_heads), static_cast<int>(head_dim), static_cast<long long>(pages),                       \
        static_cast<long long>(page_size), static_cast<long long>(capacity), status, warm, norms)
    const WarmRange warm = take_pending_warm();
    if (index_width == 8) {
        if (wide) SINGE_ROTARY(long long, 8); else SINGE_ROTARY(long long, 1);
    } else {
        if (wide) SINGE_ROTARY(int, 8); else SINGE_ROTARY(int, 1);
    }
#undef SINGE_ROTARY
    return launch_status();
}

int singe_rotary_cache_write_bf16(singe_stream_t stream, void *q_out, const void *qkv, size_t qkv_row_stride,
                                  const void *cos_table, const void *sin_table, const void *positions,
                                  void *key_cache, void *value_cache, const void *write_pages,
                                  const void *write_slots, int index_width, size_t tokens, size_t heads,
                                  size_t kv_heads, size_t head_dim, size_t pages, size_t page_size, size_t capacity,
                                  uint32_t *status) {
    const HeadNorms none = {nullptr, nullptr, 0, 0, 0.0f};
    return rotary_cache_write(stream, q_out, qkv, qkv_row_stride, cos_table, sin_table, positions, key_cache,
                              value_cache, write_pages, write_slots, index_width, tokens, heads, kv_heads, head_dim,
                              pages, page_size, capacity, status, none);
}

int singe_rotary_norm_cache_write_bf16(singe_stream_t stream, void *q_out, const void *qkv, size_t qkv_row_stride,
                                       const void *cos_table, const void *sin_table, const void *positions,
                                       void *key_cache, void *value_cache, const void *write_pages,
                                       const void *write_slots, int index_width, size_t tokens, size_t heads,
                                       size_t kv_heads, size_t head_dim, size_t pages, size_t page_size,
                                       size_t capacity, int normalise_query, const void *query_norm_weight,
                                       int normalise_key, const void *key_norm_weight, float eps, uint32_t *status) {
    const HeadNorms norms = {static_cast<const __nv_bfloat16 *>(query_norm_weight),
                             static_cast<const __nv_bfloat16 *>(key_norm_weight), normalise_query != 0 ? 1 : 0,
                             normalise_key != 0 ? 1 : 0, eps};
    return rotary_cache_write(stream, q_out, qkv, qkv_row_stride, cos_table, sin_table, positions, key_cache,
                              value_cache, write_pages, write_slots, index_width, tokens, heads, kv_heads, head_dim,
                              pages, page_size, capacity, status, norms);
}

int singe_silu_mul_bf16(singe_stream_t stream, void *out, const void *gate, const void *up, size_t input_row_stride,
                        size_t rows, size_t width) {
    if (rows == 0 || width == 0 || input_row_stride < width) return SINGE_ERR_INVALID_LENGTH;
    if (!fits_i32(rows) || !fits_i32(width)) return SINGE_ERR_LENGTH_EXCEEDS_I32;
    if (out == nullptr || gate == nullptr || up == nullptr) return SINGE_ERR_NULL_POINTER;
    if (rows > 65535) return SINGE_ERR_UNSUPPORTED_CONFIGURATION;
    const bool wide = width % 8 == 0 && input_row_stride % 8 == 0 && aligned16(out) && aligned16(gate) && aligned16(up);
    if (wide) {
        dim3 grid(static_cast<unsigned>((width / 8 + 255) / 256), static_cast<unsigned>(rows));
        launch_dependent(silu_mul_kernel<8>, grid, dim3(256), 0, static_cast<cudaStream_t>(stream), kLaunchGlue, 1,
            static_cast<__nv_bfloat16 *>(out), static_cast<const __nv_bfloat16 *>(gate),
            static_cast<const __nv_bfloat16 *>(up), static_cast<long long>(input_row_stride), static_cast<int>(width));
    } else {
        dim3 grid(static_cast<unsigned>((width + 255) / 256), static_cast<unsigned>(rows));
        launch_dependent(silu_mul_kernel<1>, grid, dim3(256), 0, static_cast<cudaStream_t>(stream), kLaunchGlue, 1,
            static_cast<__nv_bfloat16 *>(out), static_cast<const __nv_bfloat16 *>(gate),
            static_cast<const __nv_bfloat16 *>(up), static_cast<long long>(input_row_stride), static_cast<int>(width));
    }
    return launch_status();
}

int singe_argmax_bf16(singe_stream_t stream, float *best_value, int64_t *best_index, const void *logits,
                      size_t row_stride, size_t rows, size_t width, int64_t index_offset) {
    if (rows == 0 || width == 0 || row_stride < width) return SINGE_ERR_INVALID_LENGTH;
    if (!fits_i32(rows) || !fits_i32(width)) return SINGE_ERR_LENGTH_EXCEEDS_I32;
    if (best_value == nullptr || best_index == nullptr || logits == nullptr) return SINGE_ERR_NULL_POINTER;
    const bool wide = width % 8 == 0 && row_stride % 8 == 0 && aligned16(logits);
    if (wide) {
        launch_dependent(argmax_kernel<8>, dim3(static_cast<unsigned>(rows)), dim3(1024), 0,
                         static_cast<cudaStream_t>(stream), kLaunchGlue, 1,
            best_value, reinterpret_cast<long long *>(best_index), static_cast<const __nv_bfloat16 *>(logits),
            static_cast<long long>(row_stride), static_cast<int>(width), static_cast<long long>(index_offset));
    } else {
        launch_dependent(argmax_kernel<1>, dim3(static_cast<unsigned>(rows)), dim3(1024), 0,
                         static_cast<cudaStream_t>(stream), kLaunchGlue, 1,
            best_value, reinterpret_cast<long long *>(best_index), static_cast<const __nv_bfloat16 *>(logits),
            static_cast<long long>(row_stride), static_cast<int>(width), static_cast<long long>(index_offset));
    }
    return launch_status();
}

}  // extern "C"
