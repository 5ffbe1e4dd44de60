// Tensor-parallel all-reduce over NVLink peer memory, fused with the residual add and RMSNorm that follow it in the
// Llama decode step.
//
// Meaning: the reference sums the row-sharded o_proj / down_proj outputs of all ranks with a singe-nccl all-reduce
// (Communicator::all_reduce_in_place, singe-nccl/src/communicator/operations/collectives.rs:99-134, operator Sum)
// and then runs the residual add and the next RMSNorm of the pre-norm block as separate tensor ops
// (singe-model/src/assembly/decoder.rs:102-126).  Here one kernel does all three: every rank reads the partial rows
// of all ranks straight out of their HBM over NVLink (one-shot all-reduce: world x rows x width bf16 per rank, 4 MB
// at world 8 for a 64 x 4096 step), sums them in f32 in rank order (so every rank computes bit-identical results),
// rounds the sum to bf16 (the all-reduce's result type), adds it to the residual stream and normalises.  At decode
// sizes the collective is pure latency; this removes two kernel launches and the NCCL protocol per collective.
//
// Synchronisation (no host involvement, CUDA-graph replayable):
//   * every rank owns a flag array flags[world] in peer-mapped memory; slot r is written only by rank r.
//   * a launch has an epoch (a counter in local memory, advanced by the last CTA of the launch).  CTA 0 stores the
//     epoch into slot `rank` of every rank's array with release semantics at system scope: the partial rows were
//     written by the GEMM kernel that precedes this launch on the stream, so they are visible before the flag.
//   * every CTA waits (acquire loads at system scope, bounded by a cycle count) until all slots of the local array
//     have reached the epoch, then reads the peers' rows with loads that bypass L1.
//   * a rank may overwrite a partial buffer again only after a later all-reduce has passed its entry wait: the
//     decode step alternates two partial buffers (o_proj, down_proj), and passing the entry wait of the down_proj
//     all-reduce proves that every peer has finished the o_proj all-reduce, i.e. has finished reading that buffer.
// Peer buffers are plain cudaMalloc allocations shared through CUDA IPC handles; no multicast object is involved.
#include "common.cuh"

namespace singe {
namespace {

constexpr int kMaxPeers = 8;
constexpr int kReduceThreads = 512;
constexpr long long kPeerWaitCycles = 1ll << 33;  // a few seconds: ranks reach a collective at different times

struct PeerParams {
    const __nv_bfloat16 *partial[kMaxPeers];  // this call's partial buffer of every rank (own included)
    uint32_t *flags[kMaxPeers];               // the flag array of every rank (own included)
    uint32_t *state;                          // local: [0] epoch of the last finished launch, [1] finished CTAs
    __nv_bfloat16 *hidden;                    // local residual stream, updated in place
    __nv_bfloat16 *normed;                    // local output
    const __nv_bfloat16 *weight;
    uint32_t *status;
    int rank;
    int world;
    int width;
    float eps;
    WarmRange warm;  // pulled into L2 while the ranks wait for one another
};

__device__ __forceinline__ void store_release_system(uint32_t *address, uint32_t value) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(address), "r"(value) : "memory");
}

__device__ __forceinline__ uint32_t load_acquire_system(const uint32_t *address) {
    uint32_t value;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(value) : "l"(address) : "memory");
    return value;
}

// 16 bytes from a peer's memory, not served from this SM's L1 (an earlier launch read the same addresses).
__device__ __forceinline__ uint4 load_peer(const void *address) {
    uint4 value;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(value.x), "=r"(value.y), "=r"(value.z), "=r"(value.w)
                 : "l"(address)
                 : "memory");
    return value;
}

__device__ __forceinline__ float round_to_bf16(float value) { return __bfloat162float(__float2bfloat16_rn(value)); }

__global__ void __launch_bounds__(kReduceThreads)
    allreduce_add_rms_norm_kernel(const PeerParams p) {
    __shared__ uint32_t shared_epoch;
    __shared__ int shared_ok;
    __shared__ float scratch[kReduceThreads / 32];
    const int tid = threadIdx.x;
    grid_launch_dependents();
    if (tid < 32) warm_l2(p.warm, blockIdx.x, gridDim.x, tid);
    grid_dependency_wait();  // the GEMM before this launch has written this rank's partial rows
    if (tid == 0) {
        shared_epoch = p.state[0] + 1;
        shared_ok = 1;
    }
    __syncthreads();
    const uint32_t epoch = shared_epoch;
    if (blockIdx.x == 0 && tid < p.world) {
        store_release_system(p.flags[tid] + p.rank, epoch);  // "my partial rows are written"
    }
    if (tid < p.world) {
        const uint32_t *slot = p.flags[p.rank] + tid;
        const long long start = clock64();
        while (static_cast<int32_t>(load_acquire_system(slot) - epoch) < 0) {
            if (clock64() - start > kPeerWaitCycles) {
                shared_ok = 0;
                break;
            }
        }
    }
    __syncthreads();
    const bool ok = shared_ok != 0;
    if (ok) {
        const size_t base = static_cast<size_t>(blockIdx.x) * p.width;
        constexpr int kHeld = 2;  // rows up to 512 * 8 * 2 = 8192 wide are held in registers between the passes
        float held[kHeld][8];
        float square = 0.0f;
        const int stride = kReduceThreads * 8;
#pragma unroll
        for (int h = 0; h < kHeld; ++h) {
            const int c = tid * 8 + h * stride;
            if (c < p.width) {
                float sum[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
                uint4 raw[kMaxPeers];
#pragma unroll
                for (int r = 0; r < kMaxPeers; ++r) {
                    if (r < p.world) raw[r] = load_peer(p.partial[r] + base + c);  // all loads in flight together
                }
#pragma unroll
                for (int r = 0; r < kMaxPeers; ++r) {
                    if (r < p.world) {
                        const uint32_t words[4] = {raw[r].x, raw[r].y, raw[r].z, raw[r].w};
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            sum[2 * i] += __uint_as_float(words[i] << 16);
                            sum[2 * i + 1] += __uint_as_float(words[i] & 0xffff0000u);
                        }
                    }
                }
                const uint4 residual = *reinterpret_cast<const uint4 *>(p.hidden + base + c);
                const uint32_t words[4] = {residual.x, residual.y, residual.z, residual.w};
                uint4 updated;
                uint32_t *out_words = &updated.x;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float low = round_to_bf16(__uint_as_float(words[i] << 16) + round_to_bf16(sum[2 * i]));
                    const float high =
                        round_to_bf16(__uint_as_float(words[i] & 0xffff0000u) + round_to_bf16(sum[2 * i + 1]));
                    held[h][2 * i] = low;
                    held[h][2 * i + 1] = high;
                    square += low * low + high * high;
                    out_words[i] = pack2<__nv_bfloat16>(low, high);
                }
                *reinterpret_cast<uint4 *>(p.hidden + base + c) = updated;
            }
        }
        float total = warp_sum(square);
        if ((tid & 31) == 0) scratch[tid >> 5] = total;
        __syncthreads();
        total = 0.0f;
#pragma unroll
        for (int i = 0; i < kReduceThreads / 32; ++i) total += scratch[i];
        const float scale = 1.0f / sqrtf(total / static_cast<float>(p.width) + p.eps);
#pragma unroll
        for (int h = 0; h < kHeld; ++h) {
            const int c = tid * 8 + h * stride;
            if (c < p.width) {
                const uint4 gain = *reinterpret_cast<const uint4 *>(p.weight + c);
                const uint32_t words[4] = {gain.x, gain.y, gain.z, gain.w};
                uint4 result;
                uint32_t *out_words = &result.x;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    out_words[i] = pack2<__nv_bfloat16>(held[h][2 * i] * scale * __uint_as_float(words[i] << 16),
                                                        held[h][2 * i + 1] * scale *
                                                            __uint_as_float(words[i] & 0xffff0000u));
                }
                *reinterpret_cast<uint4 *>(p.normed + base + c) = result;
            }
        }
    } else if (tid == 0) {
        report_status(p.status, kStatusWaitTimeout);
    }
    // The last CTA to finish advances the epoch: every CTA of this launch has read the old value by then.
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        const uint32_t finished = atomicAdd(p.state + 1, 1u);
        if (finished == gridDim.x - 1) {
            p.state[1] = 0;
            __threadfence();
            p.state[0] = epoch;
        }
    }
}

}  // namespace
}  // namespace singe

extern "C" {

// A peer-shareable device buffer: a cudaMalloc allocation, zero-filled, with the CUDA IPC handle other processes
// open it by.
int singe_peer_buffer_create(size_t bytes, void **pointer, void *handle_out) {
    if (pointer == nullptr || handle_out == nullptr) return SINGE_ERR_NULL_POINTER;
    if (bytes == 0) return SINGE_ERR_INVALID_LENGTH;
    void *memory = nullptr;
    SINGE_CUDA_TRY(cudaMalloc(&memory, bytes));
    cudaError_t error = cudaMemset(memory, 0, bytes);
    cudaIpcMemHandle_t handle;
    if (error == cudaSuccess) error = cudaIpcGetMemHandle(&handle, memory);
    if (error == cudaSuccess) error = cudaDeviceSynchronize();
    if (error != cudaSuccess) {
        cudaFree(memory);
        return singe::cuda_status(error);
    }
    static_assert(sizeof(cudaIpcMemHandle_t) == SINGE_PEER_HANDLE_BYTES, "handle size");
    memcpy(handle_out, &handle, sizeof(handle));
    *pointer = memory;
    return SINGE_OK;
}

int singe_peer_buffer_open(const void *handle_in, void **pointer) {
    if (pointer == nullptr || handle_in == nullptr) return SINGE_ERR_NULL_POINTER;
    cudaIpcMemHandle_t handle;
    memcpy(&handle, handle_in, sizeof(handle));
    SINGE_CUDA_TRY(cudaIpcOpenMemHandle(pointer, handle, cudaIpcMemLazyEnablePeerAccess));
    return SINGE_OK;
}

int singe_peer_buffer_close(void *pointer) {
    if (pointer == nullptr) return SINGE_ERR_NULL_POINTER;
    SINGE_CUDA_TRY(cudaIpcCloseMemHandle(pointer));
    return SINGE_OK;
}

int singe_peer_buffer_destroy(void *pointer) {
    if (pointer == nullptr) return SINGE_ERR_NULL_POINTER;
    SINGE_CUDA_TRY(cudaFree(pointer));
    return SINGE_OK;
}

int singe_allreduce_add_rms_norm_bf16(singe_stream_t stream, void *hidden, void *normed, const void *weight,
                                      const void *const *partials, uint32_t *const *flags, uint32_t *state, int rank,
                                      int world, size_t rows, size_t width, float eps, uint32_t *status) {
    if (hidden == nullptr || normed == nullptr || weight == nullptr || partials == nullptr || flags == nullptr ||
        state == nullptr) {
        return SINGE_ERR_NULL_POINTER;
    }
    if (world < 1 || world > singe::kMaxPeers || rank < 0 || rank >= world) return SINGE_ERR_INVALID_ARGUMENT;
    if (rows == 0 || width == 0 || width % 8 != 0 || width > static_cast<size_t>(singe::kReduceThreads) * 8 * 2) {
        return SINGE_ERR_INVALID_LENGTH;
    }
    if (rows > 0x7fffffffull) return SINGE_ERR_LENGTH_EXCEEDS_I32;
    singe::PeerParams params;
    for (int r = 0; r < singe::kMaxPeers; ++r) {
        params.partial[r] = r < world ? static_cast<const __nv_bfloat16 *>(partials[r]) : nullptr;
        params.flags[r] = r < world ? flags[r] : nullptr;
        if (r < world && (params.partial[r] == nullptr || params.flags[r] == nullptr)) return SINGE_ERR_NULL_POINTER;
        if (r < world && (reinterpret_cast<uintptr_t>(params.partial[r]) & 15u) != 0) return SINGE_ERR_INVALID_ARGUMENT;
    }
    if (((reinterpret_cast<uintptr_t>(hidden) | reinterpret_cast<uintptr_t>(normed) |
          reinterpret_cast<uintptr_t>(weight)) & 15u) != 0) {
        return SINGE_ERR_INVALID_ARGUMENT;
    }
    params.state = state;
    params.hidden = static_cast<__nv_bfloat16 *>(hidden);
    params.normed = static_cast<__nv_bfloat16 *>(normed);
    params.weight = static_cast<const __nv_bfloat16 *>(weight);
    params.status = status != nullptr ? status : singe::device_error_word();
    params.rank = rank;
    params.world = world;
    params.width = static_cast<int>(width);
    params.eps = eps;
    params.warm = singe::take_pending_warm();
    SINGE_CUDA_TRY(singe::launch_dependent(singe::allreduce_add_rms_norm_kernel, dim3(static_cast<unsigned>(rows)),
                                           dim3(singe::kReduceThreads), 0, static_cast<cudaStream_t>(stream),
                                           singe::kLaunchReduce, 1,
                                           params));
    return singe::launch_status();
}

}  // extern "C"
