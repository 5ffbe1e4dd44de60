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
    uint32_t *state;                          // local: [0] epoch of the last finished launch, [1] finished CTAs,
                                              // [2] wait limit in units of 1024 cycles (0 = kPeerWaitCycles)
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
    const uint32_t short_limit = p.state[2];  // 0: the default below; else the wait limit in units of 1024 cycles
    const long long wait_cycles = short_limit != 0 ? static_cast<long long>(short_limit) << 10 : kPeerWaitCycles;
    if (blockIdx.x == 0 && tid < p.world) {
        store_release_system(p.flags[tid] + p.rank, epoch);  // "my partial rows are written"
    }
    if (tid < p.world) {
        const uint32_t *slot = p.flags[p.rank] + tid;
        const long long start = clock64();
        while (static_cast<int32_t>(load_acquire_system(slot) - epoch) < 0) {
            if (clock64() - start > wait_cycles) {
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
                    square = square_chain(square_chain(square, low), high);
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


// ---------------------------------------------------------------------------------------------------------------
// Two-phase form: reduce-scatter by rows, then all-gather of the normalised rows, both by PUSHING flagged packets.
//
// The one-shot kernel above waits for a flag and then PULLS world x rows x width over NVLink: at 8 ranks every rank
// reads 3.5 MB per collective behind a remote-load latency, and every rank repeats all the norms.  Here rank r owns
// rows [r * rpr, (r + 1) * rpr), and nothing ever waits for a round trip or an acknowledgement: data travels as
// 8-byte packets {4 bytes of data, 4-byte epoch} (two per 16-byte store; an aligned 8-byte store arrives whole), so
// a receiver that reads the current epoch in a packet holds valid data -- no flag behind a fence, no atomics.
//   phase 1  every rank pushes each of its partial rows into the owner's receive buffer (slot = sender);
//   phase 2  the threads of an owner's CTA poll their own packets of all `world` slots, sum them in rank order in
//            f32, round to bf16 (the all-reduce's result type), add the residual (only the owner keeps a row of the
//            residual stream up to date), normalise, and leave the normalised row as packets in a local staging area;
//   phase 2b CTA (r, j) of every rank takes owned row r out of the staging area and pushes it to rank j: the rows of
//            one collective are 0.9 MB at eight ranks, which eight owner CTAs alone took 3 us to issue -- an SM
//            pushes about 45 GB/s over NVLink -- so the push is spread over all CTAs of the launch;
//   phase 3  every rank unpacks the normalised rows it received into the plain buffer the next GEMM reads.
// Per rank and collective 2 x 7/8 x 1 MB leave (packets double the bytes) instead of 3.5 MB arriving behind a
// load latency.  The epoch only grows and lives on the device, so the kernel replays inside a CUDA graph; packets of
// an earlier launch carry an older epoch, so nothing is ever cleared.  Buffers are safe to reuse by the next launch:
// a rank starts the next launch only after it has unpacked every normalised row of this one, which the owners sent
// after they had consumed every packet of this launch's first phase.
// Every wait is bounded; a wait that runs out sets status 2, the thread skips what depended on it, the kernel ends.
// (A first version signalled with release atomics at system scope behind plain pushes: each release waits for the
// acknowledgement of the stores before it, two of those per collective; at two ranks it cost 15 us more than the
// one-shot kernel.)
// ---------------------------------------------------------------------------------------------------------------
struct TwoPhaseParams {
    const __nv_bfloat16 *partial;   // local [rows, width]: this rank's partial sums
    uint4 *receive[kMaxPeers];      // rank j's receive packets [world][rpr][width / 4] (16 bytes carry 4 values)
    uint4 *gather[kMaxPeers];       // rank j's packets of normalised rows [rows][width / 4], followed by rank j's own
                                    // staging area [rpr][width / 4] (see phase 2b)
    uint4 *stage;                   // local: gather[rank] + rows * width / 4
    uint32_t *state;                // local: [0] finished launches, [1] finished CTAs, [2] wait limit / 1024 cycles
    __nv_bfloat16 *hidden;          // local residual stream; only the owned rows are kept up to date
    __nv_bfloat16 *normed;          // local [rows, width]: all normalised rows, plain
    const __nv_bfloat16 *weight;
    uint32_t *status;
    int rank, world, rows, rpr, width;
    int replicated;  // 1: every rank owns every row -- each partial row is pushed to all ranks, every rank sums and
                     // normalises all rows itself, and there is no second phase (one NVLink trip; for two ranks)
    float eps;
    WarmRange warm;
};

__device__ __forceinline__ void store_packets(uint4 *address, uint32_t first, uint32_t second, uint32_t epoch) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(address), "r"(first), "r"(epoch),
                 "r"(second), "r"(epoch)
                 : "memory");
}

constexpr int kTwoPhaseThreads = 1024;  // one 16-byte packet pair (four values) per thread for rows 4096 wide

__device__ __forceinline__ bool packets_ready(const uint4 &value, uint32_t epoch) {
    return value.y == epoch && value.w == epoch;
}

// Polls one 16-byte pair of packets until both carry `epoch`; false when the limit ran out.
__device__ __forceinline__ bool poll_packets(const uint4 *address, uint32_t epoch, long long limit, uint4 &value) {
    value = load_peer(address);
    if (!packets_ready(value, epoch)) {
        const long long start = clock64();
        do {
            if (clock64() - start > limit) return false;
            value = load_peer(address);
        } while (!packets_ready(value, epoch));
    }
    return true;
}

__global__ void __launch_bounds__(kTwoPhaseThreads)
    allreduce_two_phase_kernel(const TwoPhaseParams p) {
    __shared__ uint32_t shared_epoch;
    __shared__ long long shared_limit;
    __shared__ int shared_failed;
    __shared__ float scratch[16];
    __shared__ float chunk_sums[kTwoPhaseThreads / 2];
    const int tid = threadIdx.x;
    const int c = blockIdx.x;
    grid_launch_dependents();
    if (tid < 32) warm_l2(p.warm, blockIdx.x, gridDim.x, tid);
    grid_dependency_wait();  // the GEMM before this launch has written this rank's partial rows
    if (tid == 0) {
        shared_epoch = p.state[0] + 1;
        const uint32_t limit = p.state[2];
        shared_limit = limit != 0 ? static_cast<long long>(limit) << 10 : kPeerWaitCycles;
        shared_failed = 0;
    }
    __syncthreads();
    const uint32_t epoch = shared_epoch;
    const long long limit = shared_limit;
    const int quads = p.width >> 2;            // 16-byte packet pairs per row (4 values each)
    constexpr int kHeld = 2;                   // rows up to 1024 * 2 * 4 = 8192 wide

    // ---- phase 1: row c of this rank's partial goes to its owner (replicated: to every rank) ----
    {
        const int owner = p.replicated ? 0 : c / p.rpr;
        const size_t at = (static_cast<size_t>(p.rank) * p.rpr + (c - owner * p.rpr)) * quads;
        const uint2 *source = reinterpret_cast<const uint2 *>(p.partial + static_cast<size_t>(c) * p.width);
        for (int q = tid; q < quads; q += kTwoPhaseThreads) {
            uint2 value;
            asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(value.x), "=r"(value.y) : "l"(source + q));
            if (p.replicated) {
#pragma unroll
                for (int r = 0; r < kMaxPeers; ++r) {
                    if (r < p.world) store_packets(p.receive[r] + at + q, value.x, value.y, epoch);
                }
            } else {
                store_packets(p.receive[owner] + at + q, value.x, value.y, epoch);
            }
        }
    }

    // ---- phase 2: the first `owned` CTAs each finish one owned row ----
    const int first_owned = p.replicated ? 0 : p.rank * p.rpr;
    const int owned = p.replicated ? p.rows : max(0, min(p.rows, first_owned + p.rpr) - first_owned);
    if (c < owned) {
        const int row = first_owned + c;
        float held[kHeld][4];
        bool ok = true;
#pragma unroll
        for (int h = 0; h < kHeld; ++h) {
            const int q = tid + h * kTwoPhaseThreads;
            held[h][0] = held[h][1] = held[h][2] = held[h][3] = 0.0f;
            if (q < quads) {
                // All slots are requested together; only those that have not arrived yet are asked for again.
                const uint4 *slot = p.receive[p.rank] + static_cast<size_t>(c) * quads + q;
                const size_t slot_stride = static_cast<size_t>(p.rpr) * quads;
                uint4 packet[kMaxPeers];
#pragma unroll
                for (int r = 0; r < kMaxPeers; ++r) {
                    if (r < p.world) packet[r] = load_peer(slot + r * slot_stride);
                }
                bool pending = false;
#pragma unroll
                for (int r = 0; r < kMaxPeers; ++r) {
                    if (r < p.world && !packets_ready(packet[r], epoch)) pending = true;
                }
                if (pending && ok) {
#pragma unroll
                    for (int r = 0; r < kMaxPeers; ++r) {
                        if (r < p.world && ok && !packets_ready(packet[r], epoch)) {
                            ok = poll_packets(slot + r * slot_stride, epoch, limit, packet[r]);
                        }
                    }
                }
                float sum[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                for (int r = 0; r < kMaxPeers; ++r) {  // rank order: every owner adds in the same order
                    if (r < p.world) {
                        sum[0] += __uint_as_float(packet[r].x << 16);
                        sum[1] += __uint_as_float(packet[r].x & 0xffff0000u);
                        sum[2] += __uint_as_float(packet[r].z << 16);
                        sum[3] += __uint_as_float(packet[r].z & 0xffff0000u);
                    }
                }
                const uint2 residual =
                    *reinterpret_cast<const uint2 *>(p.hidden + static_cast<size_t>(row) * p.width + q * 4);
                held[h][0] = round_to_bf16(__uint_as_float(residual.x << 16) + round_to_bf16(sum[0]));
                held[h][1] = round_to_bf16(__uint_as_float(residual.x & 0xffff0000u) + round_to_bf16(sum[1]));
                held[h][2] = round_to_bf16(__uint_as_float(residual.y << 16) + round_to_bf16(sum[2]));
                held[h][3] = round_to_bf16(__uint_as_float(residual.y & 0xffff0000u) + round_to_bf16(sum[3]));
            }
        }
        if (!ok) shared_failed = 1;
        // Sum of squares in the library's one order (see square_chain): a chunk of eight values is held by a pair of
        // adjacent threads, so the chain runs through the even thread's four values, then the odd thread's, chunk
        // after chunk; the pair's total then plays the part of one of 512 virtual threads.
        const int lane = tid & 31;
        float carry = 0.0f;
#pragma unroll
        for (int h = 0; h < kHeld; ++h) {
            float chain = carry;
#pragma unroll
            for (int i = 0; i < 4; ++i) chain = square_chain(chain, held[h][i]);     // meaningful on even lanes
            chain = __shfl_sync(0xffffffffu, chain, lane & ~1);
#pragma unroll
            for (int i = 0; i < 4; ++i) chain = square_chain(chain, held[h][i]);     // meaningful on odd lanes
            carry = __shfl_sync(0xffffffffu, chain, lane | 1);
        }
        if ((tid & 1) == 0) chunk_sums[tid >> 1] = carry;
        __syncthreads();
        if (tid < 512) {
            const float folded = warp_sum(chunk_sums[tid]);
            if (lane == 0) scratch[tid >> 5] = folded;
        }
        __syncthreads();
        if (shared_failed == 0) {  // the whole row arrived: only now is anything written
            float total = 0.0f;
#pragma unroll
            for (int i = 0; i < 16; ++i) total += scratch[i];
            const float scale = 1.0f / sqrtf(total / static_cast<float>(p.width) + p.eps);
#pragma unroll
            for (int h = 0; h < kHeld; ++h) {
                const int q = tid + h * kTwoPhaseThreads;
                if (q < quads) {
                    *reinterpret_cast<uint2 *>(p.hidden + static_cast<size_t>(row) * p.width + q * 4) = make_uint2(
                        pack2<__nv_bfloat16>(held[h][0], held[h][1]), pack2<__nv_bfloat16>(held[h][2], held[h][3]));
                    const uint2 gain = *reinterpret_cast<const uint2 *>(p.weight + q * 4);
                    const uint32_t first = pack2<__nv_bfloat16>(held[h][0] * scale * __uint_as_float(gain.x << 16),
                                                                held[h][1] * scale * __uint_as_float(gain.x & 0xffff0000u));
                    const uint32_t second = pack2<__nv_bfloat16>(held[h][2] * scale * __uint_as_float(gain.y << 16),
                                                                 held[h][3] * scale * __uint_as_float(gain.y & 0xffff0000u));
                    if (p.replicated) {
                        *reinterpret_cast<uint2 *>(p.normed + static_cast<size_t>(row) * p.width + q * 4) =
                            make_uint2(first, second);
                    } else {
                        store_packets(p.stage + static_cast<size_t>(c) * quads + q, first, second, epoch);
                    }
                }
            }
        }
    }

    // ---- phase 2b: owned row r goes to rank j, one (r, j) pair per CTA ----
    if (!p.replicated) {
        bool ok = true;
        for (int pair = c; pair < p.rpr * p.world && ok; pair += gridDim.x) {
            const int r = pair % p.rpr;
            const int j = pair / p.rpr;
            if (r >= owned) continue;
            const size_t row = static_cast<size_t>(first_owned + r);
            for (int q = tid; q < quads; q += kTwoPhaseThreads) {
                if (shared_failed != 0) break;  // the owner's wait ran out: the row will not come
                uint4 packet;
                ok = poll_packets(p.stage + static_cast<size_t>(r) * quads + q, epoch, limit, packet);
                if (!ok) break;
                store_packets(p.gather[j] + row * quads + q, packet.x, packet.z, epoch);
            }
        }
        if (!ok) shared_failed = 1;
    }

    // ---- phase 3: unpack normalised row c ----
    if (!p.replicated) {
        bool ok = true;
        for (int q = tid; q < quads; q += kTwoPhaseThreads) {
            if (shared_failed != 0) break;  // an owner's wait ran out on this rank: do not sit through another one
            uint4 packet;
            ok = poll_packets(p.gather[p.rank] + static_cast<size_t>(c) * quads + q, epoch, limit, packet);
            if (!ok) break;
            *reinterpret_cast<uint2 *>(p.normed + static_cast<size_t>(c) * p.width + q * 4) = make_uint2(packet.x, packet.z);
        }
        if (!ok) shared_failed = 1;
    }
    __syncthreads();
    if (shared_failed != 0 && tid == 0) report_status(p.status, kStatusWaitTimeout);
    // The last CTA to finish advances the epoch: every CTA of this launch has read the old value by then.
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

int singe_allreduce_two_phase_add_rms_norm_bf16(singe_stream_t stream, void *hidden, void *normed, const void *weight,
                                                const void *partial, void *const *receive, void *const *gather,
                                                uint32_t *state, int rank, int world, size_t rows, size_t width,
                                                float eps, int replicated, uint32_t *status) {
    if (hidden == nullptr || normed == nullptr || weight == nullptr || partial == nullptr || receive == nullptr ||
        gather == nullptr || state == nullptr) {
        return SINGE_ERR_NULL_POINTER;
    }
    if (world < 1 || world > singe::kMaxPeers || rank < 0 || rank >= world) return SINGE_ERR_INVALID_ARGUMENT;
    if (rows == 0 || width == 0 || width % 8 != 0 || width > static_cast<size_t>(singe::kTwoPhaseThreads) * 2 * 4) {
        return SINGE_ERR_INVALID_LENGTH;
    }
    // One CTA per row, and CTAs wait for one another's pushes: all of them must be resident at once (two CTAs of 1024
    // threads fit an SM).
    if (rows > 256) return SINGE_ERR_UNSUPPORTED_CONFIGURATION;
    singe::TwoPhaseParams params;
    for (int r = 0; r < singe::kMaxPeers; ++r) {
        params.receive[r] = r < world ? static_cast<uint4 *>(receive[r]) : nullptr;
        params.gather[r] = r < world ? static_cast<uint4 *>(gather[r]) : nullptr;
        if (r < world && (params.receive[r] == nullptr || params.gather[r] == nullptr)) return SINGE_ERR_NULL_POINTER;
        if (r < world && ((reinterpret_cast<uintptr_t>(params.receive[r]) |
                           reinterpret_cast<uintptr_t>(params.gather[r])) & 15u) != 0) {
            return SINGE_ERR_INVALID_ARGUMENT;
        }
    }
    if (((reinterpret_cast<uintptr_t>(hidden) | reinterpret_cast<uintptr_t>(partial) | reinterpret_cast<uintptr_t>(normed) |
          reinterpret_cast<uintptr_t>(weight)) & 15u) != 0) {
        return SINGE_ERR_INVALID_ARGUMENT;
    }
    params.partial = static_cast<const __nv_bfloat16 *>(partial);
    params.state = state;
    params.stage = params.gather[rank] + rows * (width / 4);
    params.hidden = static_cast<__nv_bfloat16 *>(hidden);
    params.normed = static_cast<__nv_bfloat16 *>(normed);
    params.weight = static_cast<const __nv_bfloat16 *>(weight);
    params.status = status != nullptr ? status : singe::device_error_word();
    params.rank = rank;
    params.world = world;
    params.rows = static_cast<int>(rows);
    params.replicated = replicated != 0 ? 1 : 0;
    params.rpr = params.replicated ? static_cast<int>(rows)
                                   : static_cast<int>((rows + static_cast<size_t>(world) - 1) / static_cast<size_t>(world));
    params.width = static_cast<int>(width);
    params.eps = eps;
    params.warm = singe::take_pending_warm();
    SINGE_CUDA_TRY(singe::launch_dependent(singe::allreduce_two_phase_kernel, dim3(static_cast<unsigned>(rows)),
                                           dim3(singe::kTwoPhaseThreads), 0, static_cast<cudaStream_t>(stream),
                                           singe::kLaunchReduce, 1, params));
    return singe::launch_status();
}

}  // extern "C"
