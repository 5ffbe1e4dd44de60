// Shared device/host helpers for the sm_100a kernels: status codes, bounded mbarrier waits,
// TMA (cp.async.bulk.tensor) wrappers, tensor-map encoding through the driver entry point,
// and the warp-level MMA / ldmatrix wrappers used by the HBM-bound attention kernels.
#pragma once

#include <cuda.h>
#include <cudaTypedefs.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#include "../../include/singe_kernel_sys.h"

namespace singe {

// ---------------------------------------------------------------------------------------------
// Host-side helpers
// ---------------------------------------------------------------------------------------------

inline int cuda_status(cudaError_t error) {
    return error == cudaSuccess ? SINGE_OK : SINGE_ERR_CUDA_BASE + static_cast<int>(error);
}

#define SINGE_CUDA_TRY(expr)                                  \
    do {                                                      \
        cudaError_t singe_cuda_error_ = (expr);               \
        if (singe_cuda_error_ != cudaSuccess) {               \
            return ::singe::cuda_status(singe_cuda_error_);   \
        }                                                     \
    } while (0)

#define SINGE_TRY(expr)                           \
    do {                                          \
        int singe_status_ = (expr);               \
        if (singe_status_ != SINGE_OK) {          \
            return singe_status_;                 \
        }                                         \
    } while (0)

inline bool fits_i32(size_t value) { return value <= static_cast<size_t>(INT32_MAX); }

inline int launch_status() { return cuda_status(cudaGetLastError()); }

// What the Tensor-surface paged attention hands the tiled decode kernel when a call is a plain decode batch: the
// page list as the caller gave it, and what the planning kernel of the same call wrote into the workspace.
struct RaggedDecode {
    const void *pages;         // [table_len] page ids, 32- or 64-bit
    const long long *first;    // [sequences] index of each sequence's first page in `pages`
    const int *control;        // [0] 0 = plain decode batch (tiled kernel runs), else the general kernel runs; [1] tokens per split
    int index_width;           // 4 or 8
    float *lse_out;            // [tokens, heads] base-2 LSE
    float softcap;             // 0: none; else the scaled scores are capped as softcap * tanh(score / softcap)
    const int *hidden;         // nullptr, or [sequences]: keys at the front of the sequence's first page that a sliding
                               // window hides (the planning kernel has already dropped the whole pages before it)
};

// What the tiled decode kernel needs to rotate its queries itself (singe_rotary_paged_kv_decode_attention_bf16).
struct QueryRotation {
    const void *cos;        // [capacity, head_dim / 2] in the cache dtype
    const void *sin;
    const void *positions;  // [batch], int32 or int64
    int index_width;
    int capacity;
    const void *gain;       // per-head RMSNorm gain [head_dim] or nullptr
    int normalise;
    float eps;
};

// What the tiled decode kernel needs to take a whole decode step's attention part (see FUSED in paged_decode.cu):
// the step's un-rotated projections and where the new K/V rows go.  Index width and capacity come with the
// QueryRotation of the same call.
struct FusedStep {
    const void *qkv;          // [batch, qkv_stride]
    long long qkv_stride;     // elements
    const void *write_pages;  // [batch]
    const void *write_slots;  // [batch]
};

// Programmatic dependent launch.  Every kernel of the decode path is launched with the attribute that lets it start
// while the kernels before it on the stream are still running: its CTAs do whatever does not depend on earlier work
// (barriers, tensor memory, tensor-map prefetch and -- where the caller has said that an operand is stable, see
// SINGE_HINT_* -- the first loads of that operand) and then block in grid_dependency_wait() until the earlier kernels
// have completed and their writes are visible.  The wait comes before any access to global memory that another kernel
// may have written or may still read, so stream order is preserved; without the attribute the wait returns at once.
// A step of nine short launches per layer otherwise pays a launch ramp and a cold pipeline per kernel.
// Measured on B200 (config-2 decode and the Llama decode step): every kind gains.  The split-K combine does so only
// because the decode kernel releases its dependents late, after its key loop: released at the top, the combine's
// thousand small CTAs took warp slots from the decode kernel's last wave (-4 % on the headline).
enum LaunchKind : unsigned { kLaunchGlue = 1, kLaunchGemm = 2, kLaunchDecode = 4, kLaunchCombine = 8, kLaunchReduce = 16 };

constexpr int kMaxDevices = 64;

// Index of the current device in the library's per-device tables, or -1.
inline int device_slot() {
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) return -1;
    return device;
}

// Raises a kernel's dynamic shared-memory limit once per device (the attribute belongs to the device's copy of the
// function, so a process that drives several GPUs sets it on each).  `done` is the launch site's own table.
template <typename Kernel>
inline cudaError_t ensure_dynamic_shared(Kernel kernel, int bytes, int (&done)[kMaxDevices]) {
    const int slot = device_slot();
    if (slot >= 0 && done[slot] >= bytes) return cudaSuccess;
    const cudaError_t error = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (error == cudaSuccess && slot >= 0) done[slot] = bytes;
    return error;
}

template <typename... Parameters, typename... Arguments>
inline cudaError_t launch_dependent(void (*kernel)(Parameters...), dim3 grid, dim3 block, size_t shared_bytes,
                                    cudaStream_t stream, unsigned kind, unsigned cluster, Arguments... arguments) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = shared_bytes;
    config.stream = stream;
    cudaLaunchAttribute attributes[2];
    unsigned count = 0;
    (void)kind;
    attributes[count].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attributes[count].val.programmaticStreamSerializationAllowed = 1;
    ++count;
    if (cluster > 1) {
        attributes[count].id = cudaLaunchAttributeClusterDimension;
        attributes[count].val.clusterDim.x = cluster;
        attributes[count].val.clusterDim.y = 1;
        attributes[count].val.clusterDim.z = 1;
        ++count;
    }
    config.attrs = attributes;
    config.numAttrs = count;
    return cudaLaunchKernelEx(&config, kernel, static_cast<Parameters>(arguments)...);
}

// cuTensorMapEncodeTiled through the runtime's driver entry point (no link against libcuda).
inline PFN_cuTensorMapEncodeTiled_v12000 tensor_map_encoder() {
    static PFN_cuTensorMapEncodeTiled_v12000 encoder = [] {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult query;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &query) != cudaSuccess ||
            query != cudaDriverEntryPointSuccess) {
            fn = nullptr;
        }
        return reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
    }();
    return encoder;
}

// Encodes a tiled tensor map of `rank` dimensions (innermost first).  `strides_bytes[i]` is the
// stride of dimension i+1.  Returns a SINGE status.
inline int encode_tensor_map(CUtensorMap *map, CUtensorMapDataType type, uint32_t rank, const void *base,
                             const uint64_t *dims, const uint64_t *strides_bytes, const uint32_t *box,
                             CUtensorMapSwizzle swizzle, CUtensorMapL2promotion promotion) {
    PFN_cuTensorMapEncodeTiled_v12000 encode = tensor_map_encoder();
    if (encode == nullptr) {
        return SINGE_ERR_UNSUPPORTED_CONFIGURATION;
    }
    cuuint64_t global_dims[5];
    cuuint64_t global_strides[4];
    cuuint32_t box_dims[5];
    cuuint32_t element_strides[5];
    for (uint32_t i = 0; i < rank; ++i) {
        global_dims[i] = dims[i];
        box_dims[i] = box[i];
        element_strides[i] = 1;
        if (i + 1 < rank) {
            global_strides[i] = strides_bytes[i];
        }
    }
    CUresult result = encode(map, type, rank, const_cast<void *>(base), global_dims, global_strides, box_dims,
                             element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, promotion,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return result == CUDA_SUCCESS ? SINGE_OK : SINGE_ERR_UNSUPPORTED_CONFIGURATION;
}

template <typename T>
struct TensorMapType;
template <>
struct TensorMapType<__nv_bfloat16> {
    static constexpr CUtensorMapDataType value = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
};
template <>
struct TensorMapType<__half> {
    static constexpr CUtensorMapDataType value = CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
};
template <>
struct TensorMapType<float> {
    static constexpr CUtensorMapDataType value = CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
};

// L2 warm-ahead.  A decode step is a chain of short kernels, each of which streams a weight matrix once; whatever a
// kernel finds in L2 when its turn comes it does not have to wait for HBM for.  A caller that knows what the kernels
// after the next one will read (singe_warm_l2_with_next_launch) attaches that range to the next launch: the kernel's
// CTAs ask the memory system to pull it into L2 (cp.async.bulk.prefetch, no registers, no shared memory, no
// completion to wait for) next to their own work.  The range must stay allocated until the kernel has finished and
// is only read.
struct WarmRange {
    const void *pointer;
    unsigned long long bytes;
};
// The range attached to this host thread's next launch (runtime.cu); taking it clears it.
WarmRange take_pending_warm();

// Device address of the library's sticky error word on the current device (runtime.cu): kernels record
// their first internal failure there (2 = a bounded wait ran out).  nullptr if it cannot be resolved.
uint32_t *device_error_word();

// SM count of the current device (cached per device).
inline int device_sm_count() {
    static int counts[kMaxDevices] = {0};
    const int slot = device_slot();
    if (slot >= 0 && counts[slot] > 0) return counts[slot];
    int value = 0;
    if (slot < 0 || cudaDeviceGetAttribute(&value, cudaDevAttrMultiProcessorCount, slot) != cudaSuccess || value <= 0) {
        return 148;
    }
    counts[slot] = value;
    return value;
}

// ---------------------------------------------------------------------------------------------
// Device-side helpers
// ---------------------------------------------------------------------------------------------
#if defined(__CUDACC__)

// Device-side status word codes (match the reference's status word: 1 = index out of bounds).
constexpr uint32_t kStatusIndexOutOfBounds = 1;
// Set when a bounded wait ran out; the kernel abandons its work instead of hanging.
constexpr uint32_t kStatusWaitTimeout = 2;

// See launch_dependent(): blocks until the kernels this launch depends on have completed and flushed.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// Lets the next kernel on the stream begin launching (it still waits for this one to complete before it reads).
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ void report_status(uint32_t *status, uint32_t code) {
    if (status != nullptr) {
        atomicCAS(status, 0u, code);
    }
}

__device__ __forceinline__ uint32_t smem_u32(const void *pointer) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(pointer));
}

__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t value;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(value));
    return value;
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}

__device__ __forceinline__ void mbar_init_fence() {
    // Makes barrier initialisation visible to the async proxy (TMA / tcgen05 completions).
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done != 0;
}

// Waits for the phase with `parity` to complete, for at most `kWaitLimitCycles` SM clock cycles
// (about half a second at full clock).  Returns false when the limit ran out, so callers can flag the
// failure and leave instead of spinning for ever.  The SM cycle counter is used because it is
// monotonic for a resident thread; the global nanosecond timer can jump when the GPU leaves idle.
constexpr long long kWaitLimitCycles = 1ll << 30;

__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) {
        return true;
    }
    const long long start = clock64();
    while (!mbar_try_wait(bar, parity)) {
        if (clock64() - start > kWaitLimitCycles) {
            return false;
        }
    }
    return true;
}

// After a bounded wait has run out, copies that were issued may still be landing in the CTA's shared memory.  The
// threads that gave up stay for a bounded while (about half a millisecond) before the CTA ends, so that the memory is
// not handed to another CTA with those copies still in flight.
__device__ __forceinline__ void linger_after_timeout() {
    const long long start = clock64();
    while (clock64() - start < (1ll << 20)) {
    }
}

__device__ __forceinline__ void fence_proxy_async_shared() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void prefetch_tensor_map(const CUtensorMap *map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// TMA tiled loads global -> shared, completing `bytes` on the mbarrier.  The innermost coordinate
// times the element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int32_t c0,
                                            int32_t c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1)
        : "memory");
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int32_t c0,
                                            int32_t c1, int32_t c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int32_t c0,
                                            int32_t c1, int32_t c2, int32_t c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], "
        "[%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}

// Asks the memory system to bring a tile into L2; nothing lands in shared memory and nothing signals completion.
__device__ __forceinline__ void tma_prefetch_2d(const CUtensorMap *map, int32_t c0, int32_t c1) {
    asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global [%0, {%1, %2}];"
                 ::"l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1)
                 : "memory");
}

__device__ __forceinline__ void tma_prefetch_4d(const CUtensorMap *map, int32_t c0, int32_t c1, int32_t c2, int32_t c3) {
    asm volatile("cp.async.bulk.prefetch.tensor.4d.L2.global [%0, {%1, %2, %3, %4}];"
                 ::"l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
                 : "memory");
}

// One warp of each CTA calls this: the CTAs of the grid split the range into 4 KB pieces.
__device__ __forceinline__ void warm_l2(const WarmRange &range, unsigned cta, unsigned ctas, unsigned lane) {
    constexpr unsigned long long kPiece = 4096;
    if (range.bytes == 0) return;
    const unsigned long long pieces = range.bytes / kPiece;
    const char *start = static_cast<const char *>(range.pointer);
    for (unsigned long long i = static_cast<unsigned long long>(lane) * ctas + cta; i < pieces; i += 32ull * ctas) {
        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(start + i * kPiece), "r"(4096u) : "memory");
    }
}

__device__ __forceinline__ void tma_store_2d(const CUtensorMap *map, uint32_t src, int32_t c0, int32_t c1) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(reinterpret_cast<uint64_t>(map)), "r"(src), "r"(c0), "r"(c1)
                 : "memory");
}

__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }

template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

template <int N>
__device__ __forceinline__ void tma_store_wait() {
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ bool elect_one() {
    uint32_t elected;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "elect.sync _|p, 0xffffffff;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(elected));
    return elected != 0;
}

// ldmatrix: four 8x8 b16 matrices; lane i supplies the row address of matrix i/8, row i%8.
__device__ __forceinline__ void ldmatrix_x4(uint32_t address, uint32_t &r0, uint32_t &r1, uint32_t &r2,
                                            uint32_t &r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(address));
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t address, uint32_t &r0, uint32_t &r1, uint32_t &r2,
                                                  uint32_t &r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(address));
}

// Warp-level m16n8k16 MMA with f32 accumulation; the operand type selects the bf16 or f16 form.
template <typename T>
__device__ __forceinline__ void mma_m16n8k16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1);

template <>
__device__ __forceinline__ void mma_m16n8k16<__nv_bfloat16>(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                                            uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <>
__device__ __forceinline__ void mma_m16n8k16<__half>(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                                     uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <typename T>
__device__ __forceinline__ uint32_t pack2(float low, float high);

template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float low, float high) {
    __nv_bfloat162 pair = __floats2bfloat162_rn(low, high);
    return *reinterpret_cast<uint32_t *>(&pair);
}

template <>
__device__ __forceinline__ uint32_t pack2<__half>(float low, float high) {
    __half2 pair = __floats2half2_rn(low, high);
    return *reinterpret_cast<uint32_t *>(&pair);
}

template <typename T>
__device__ __forceinline__ float to_float(T value);
template <>
__device__ __forceinline__ float to_float<float>(float value) {
    return value;
}
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 value) {
    return __bfloat162float(value);
}
template <>
__device__ __forceinline__ float to_float<__half>(__half value) {
    return __half2float(value);
}

template <typename T>
__device__ __forceinline__ T from_float(float value);
template <>
__device__ __forceinline__ float from_float<float>(float value) {
    return value;
}
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float value) {
    return __float2bfloat16_rn(value);
}
template <>
__device__ __forceinline__ __half from_float<__half>(float value) {
    return __float2half_rn(value);
}

// silu(x) = x / (1 + exp(-x)) with the special-function unit's exponential and reciprocal (a handful of instructions;
// the IEEE division it replaces costs about twenty, which shows in epilogues that run one warp per scheduler).  Every
// kernel that applies the activation uses this one form, so fused and unfused paths agree bit for bit; against the
// exact f32 value the error is a few ulp, far inside the bf16 rounding that follows.
__device__ __forceinline__ float silu_fast(float x) { return __fdividef(x, 1.0f + __expf(-x)); }

// Sum of squares of a row, the way every RMSNorm in the library takes it, so that the fused and unfused paths agree
// bit for bit: rows are cut into chunks of eight adjacent values; "virtual thread" t of 512 owns chunks t, t + 512, ...
// and runs one fused-multiply-add chain over their values in order; the 32 virtual threads of a warp are folded with
// the xor butterfly of warp_sum, and the warp totals are added in warp order.
__device__ __forceinline__ float square_chain(float sum, float value) { return __fmaf_rn(value, value, sum); }

__device__ __forceinline__ float warp_sum(float value) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
        value += __shfl_xor_sync(0xffffffffu, value, offset);
    }
    return value;
}

__device__ __forceinline__ float warp_max(float value) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
        value = fmaxf(value, __shfl_xor_sync(0xffffffffu, value, offset));
    }
    return value;
}

#endif  // __CUDACC__

}  // namespace singe
