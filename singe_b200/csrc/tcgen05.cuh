// Inline-PTX wrappers for the 5th-generation tensor core (tcgen05) of sm_100a: tensor-memory
// allocation, shared-memory matrix descriptors, the instruction descriptor of kind::f16, MMA issue,
// commit to an mbarrier, and tensor-memory loads/stores for epilogues.
//
// Layout facts these wrappers rely on:
//   * An operand tile is staged by TMA with SWIZZLE_128B as rows of 128 bytes; eight rows form a
//     1024-byte swizzle atom, so tiles start on 1024-byte boundaries.
//   * K-major operand (rows = M or N, 64 bf16 of K per row): descriptor SBO = 1024 bytes (next group
//     of eight rows), LBO unused; stepping K by 16 elements advances the start address by 32 bytes.
//   * MN-major operand (rows = K, 64 bf16 of M/N per row): eight K rows x 64 MN elements form one
//     atom; LBO = byte distance to the next 64 MN elements, SBO = byte distance to the next eight K
//     rows; stepping K by 16 elements advances the start address by two SBO strides.
//   * With M = 128 and cta_group::1 the accumulator occupies 128 tensor-memory lanes (lane = row)
//     and N consecutive 32-bit columns; warp w of a warpgroup may touch lanes 32*(w%4) .. +31.
#pragma once

#include "common.cuh"

namespace singe {
#if defined(__CUDACC__)

__device__ __forceinline__ void tmem_alloc(uint32_t smem_holder, uint32_t columns) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_holder), "r"(columns)
                 : "memory");
}

__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t address, uint32_t columns) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(address), "r"(columns) : "memory");
}

__device__ __forceinline__ void tcgen05_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tcgen05_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// All prior tcgen05 operations of this thread arrive (once) on the mbarrier when they complete.
__device__ __forceinline__ void tcgen05_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

constexpr uint64_t kSwizzle128 = 2;  // descriptor layout type of SWIZZLE_128B

// Shared-memory matrix descriptor: start address, leading/stride byte offsets (16-byte units),
// descriptor version 1 (Blackwell) and the swizzle mode.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t address, uint32_t leading_bytes, uint32_t stride_bytes) {
    uint64_t desc = 0;
    desc |= static_cast<uint64_t>((address & 0x3ffffu) >> 4);
    desc |= static_cast<uint64_t>((leading_bytes >> 4) & 0x3fffu) << 16;
    desc |= static_cast<uint64_t>((stride_bytes >> 4) & 0x3fffu) << 32;
    desc |= 1ull << 46;
    desc |= kSwizzle128 << 61;
    return desc;
}

// Instruction descriptor of tcgen05.mma kind::f16 with bf16 (or f16) operands and f32 accumulation.
// a_mn_major / b_mn_major: 0 = K-major, 1 = MN-major.
__host__ __device__ constexpr uint32_t make_instr_desc(uint32_t m, uint32_t n, bool bf16, uint32_t a_mn_major,
                                                       uint32_t b_mn_major) {
    return (1u << 4) |                      // D format: f32
           ((bf16 ? 1u : 0u) << 7) |        // A format
           ((bf16 ? 1u : 0u) << 10) |       // B format
           (a_mn_major << 15) | (b_mn_major << 16) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread.
__device__ __forceinline__ void umma_ss(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(tmem_d),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// D[tmem] (+)= A[tmem] * B[smem]; A is read from tensor memory (packed 16-bit pairs per column).
__device__ __forceinline__ void umma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
        "}\n" ::"r"(tmem_d),
        "r"(tmem_a), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Waits for this thread's tensor-memory loads and ties the wait to the registers of the newest one, so the
// compiler cannot move a use of those registers above the wait (a load may still be in flight while an older
// buffer is being consumed).
__device__ __forceinline__ void tmem_wait_ld_into(uint32_t (&r)[32]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                   "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]),
                   "+r"(r[15]), "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]),
                   "+r"(r[22]), "+r"(r[23]), "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]),
                   "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
                 :
                 : "memory");
}

// 32 lanes x 32-bit, 32 consecutive columns: thread `lane` receives row (lane base + lane), columns c .. c+31.
__device__ __forceinline__ void tmem_ld_x32(uint32_t address, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(address));
}

__device__ __forceinline__ void tmem_ld_x16(uint32_t address, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(address));
}

__device__ __forceinline__ void tmem_st_x32(uint32_t address, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(address),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
        "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
        "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}

__device__ __forceinline__ void tmem_st_x16(uint32_t address, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(address),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}

#endif  // __CUDACC__
}  // namespace singe
