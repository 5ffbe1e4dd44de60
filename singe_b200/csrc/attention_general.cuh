// General attention kernel: one warp per (query row, head), lanes split the head dimension, online
// softmax in f32.  It serves every attention surface of the path for shapes and dtypes the specialised
// kernels do not take (f32 everywhere; any head_dim / page size), the way the reference keeps
// singe_paged_attention_general beside its tiled kernels
// (singe/src/backend/cuda/kernel_plan/source/paged_general.rs:73-247).
//
// A Policy describes one surface: how a row finds its query, its visible key range and the address of
// key `pos`.  Policies return false / -1 for anything that would address outside a buffer; the row is
// then skipped and the status word set, so bad paging values never fault.
#pragma once

#include "common.cuh"

namespace singe {

enum class LseKind : int { None = 0, Natural = 1, Base2 = 2 };

template <typename T>
struct RowPlan {
    const T *query;    // head_dim values
    T *out;            // head_dim values
    float *lse;        // one value or nullptr
    int start;         // first visible key
    int end;           // one past the last visible key
    int kv_head;
    long long handle;  // policy-specific (sequence index, table offset, ...)
    long long aux;
    float sink;        // a logit that takes part in the row's softmax and weighs no value, or -inf for none
                       // (sinks of Tensor::attend, singe/src/backend/cpu/normalization/attention.rs:253-263)
};

constexpr int kMaxPerLane = 8;  // head_dim <= 256

template <typename T, typename Policy>
__global__ void __launch_bounds__(128) attention_general_kernel(Policy policy, size_t rows, int head_dim, float scale,
                                                                LseKind lse_kind, float empty_lse,
                                                                uint32_t *status, float softcap) {
    // Launched as a programmatic dependent: its CTAs may become resident while the kernel before still runs, and
    // read or write nothing before that kernel has finished.
    grid_launch_dependents();
    grid_dependency_wait();
    const int lane = threadIdx.x & 31;
    const size_t row = static_cast<size_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) {
        return;
    }
    RowPlan<T> plan;
    plan.sink = -INFINITY;
    const int located = policy.locate(row, plan);
    if (located == 0) {
        return;  // the row belongs to no sequence: nothing is written
    }
    if (located < 0) {
        if (lane == 0) report_status(status, kStatusIndexOutOfBounds);
        return;
    }
    const int per_lane = (head_dim + 31) >> 5;
    float q[kMaxPerLane];
    float acc[kMaxPerLane];
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
        const int d = lane + 32 * i;
        q[i] = (i < per_lane && d < head_dim) ? to_float<T>(plan.query[d]) * scale : 0.0f;
        acc[i] = 0.0f;
    }
    // a sink starts the online softmax as one key of weight exp(sink - sink) = 1 and value zero
    float running_max = plan.sink;
    float running_sum = plan.sink == -INFINITY ? 0.0f : 1.0f;
    bool failed = false;
    for (int pos = plan.start; pos < plan.end; pos += 4) {
        float score[4];
        long long offset[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            score[j] = 0.0f;
            offset[j] = -2;
            if (pos + j < plan.end) {
                offset[j] = policy.key_offset(plan, pos + j);
                if (offset[j] < 0) {
                    failed = true;
                } else {
                    const T *key = policy.key_base() + offset[j];
#pragma unroll
                    for (int i = 0; i < kMaxPerLane; ++i) {
                        const int d = lane + 32 * i;
                        if (i < per_lane && d < head_dim) {
                            score[j] = fmaf(q[i], to_float<T>(key[d]), score[j]);
                        }
                    }
                }
            }
        }
        if (failed) {
            break;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            score[j] = warp_sum(score[j]);
            // AttentionOptions::softcap: the scaled score is capped as cap * tanh(score / cap)
            // (singe/src/backend/cpu/normalization/attention.rs:250,500)
            if (softcap > 0.0f) score[j] = softcap * tanhf(score[j] / softcap);
            if (pos + j >= plan.end) score[j] = -INFINITY;
        }
        const float tile_max = fmaxf(fmaxf(score[0], score[1]), fmaxf(score[2], score[3]));
        const float next_max = fmaxf(running_max, tile_max);
        const float correction = __expf(running_max - next_max);  // exp(-inf) = 0 on the first tile
        float weight[4];
        float tile_sum = 0.0f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            weight[j] = (pos + j < plan.end) ? expf(score[j] - next_max) : 0.0f;
            tile_sum += weight[j];
        }
        running_sum = running_sum * correction + tile_sum;
        running_max = next_max;
#pragma unroll
        for (int i = 0; i < kMaxPerLane; ++i) {
            acc[i] *= correction;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (pos + j < plan.end) {
                const T *value = policy.value_base() + offset[j];
#pragma unroll
                for (int i = 0; i < kMaxPerLane; ++i) {
                    const int d = lane + 32 * i;
                    if (i < per_lane && d < head_dim) {
                        acc[i] = fmaf(weight[j], to_float<T>(value[d]), acc[i]);
                    }
                }
            }
        }
    }
    if (failed) {
        if (lane == 0) report_status(status, kStatusIndexOutOfBounds);
        return;
    }
    const bool empty = plan.end <= plan.start && plan.sink == -INFINITY;
    const float inverse = empty ? 0.0f : 1.0f / running_sum;
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
        const int d = lane + 32 * i;
        if (i < per_lane && d < head_dim) {
            plan.out[d] = from_float<T>(acc[i] * inverse);
        }
    }
    if (lane == 0 && plan.lse != nullptr && lse_kind != LseKind::None) {
        float value = empty ? empty_lse : running_max + logf(running_sum);
        if (lse_kind == LseKind::Base2 && !empty) {
            value *= 1.4426950408889634f;
        }
        *plan.lse = value;
    }
}

template <typename T, typename Policy>
int launch_attention_general(cudaStream_t stream, const Policy &policy, size_t rows, size_t head_dim, float scale,
                             LseKind lse_kind, float empty_lse, uint32_t *status, float softcap = 0.0f) {
    if (head_dim > 32 * kMaxPerLane) {
        return SINGE_ERR_UNSUPPORTED_WIDTH;
    }
    if (rows == 0) {
        return SINGE_OK;
    }
    const size_t blocks = (rows + 3) / 4;
    if (blocks > 0x7fffffffull) {
        return SINGE_ERR_LENGTH_EXCEEDS_I32;
    }
    SINGE_CUDA_TRY(launch_dependent(attention_general_kernel<T, Policy>, dim3(static_cast<unsigned>(blocks)), dim3(128), 0,
                                    stream, kLaunchGlue, 1, policy, rows, static_cast<int>(head_dim), scale, lse_kind,
                                    empty_lse, status, softcap));
    return launch_status();
}

}  // namespace singe
