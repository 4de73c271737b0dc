// tcgen05 / tensor-memory plumbing shared by the kernels that issue 5th-generation tensor-core MMAs:
// fences, commit, the kind::f16 MMA with shared-memory operand descriptors, accumulator read-back,
// and the two operand layouts used here (both with the 128-byte swizzle):
//   K-major  : a row of the tile holds 64 consecutive k (128 bytes); 8-row groups are SBO bytes apart
//              (what TMA writes for a [rows][k] matrix); 16 more k = +32 bytes in the start address;
//   MN-major : a row holds 64 consecutive m (or n) of ONE k; 8-k groups are SBO bytes apart, the next 64
//              m / n are LBO bytes apart; 16 more k = +2 * SBO in the start address.
// In both, the 16-byte chunk c of row r sits at chunk position c ^ (r % 8) (tile base 1024-byte aligned).
#pragma once

#include <cstdint>

namespace q35 {

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

// Shared-memory matrix descriptor, 128-byte swizzle, descriptor version 1.  lbo / sbo in bytes.
__device__ __forceinline__ uint64_t smem_desc_sw128_ex(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    uint64_t d = 0;
    d |= (uint64_t)((addr >> 4) & 0x3FFF);
    d |= (uint64_t)((lbo >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sbo >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;                  // descriptor version
    d |= (uint64_t)2 << 61;                  // SWIZZLE_128B
    return d;
}
// K-major tile of 128-byte rows, 8-row groups 1024 bytes apart (the leading offset is unused there)
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) { return smem_desc_sw128_ex(addr, 16, 1024); }

// kind::f16 instruction descriptor: D = f32, A = B = bf16, N >> 3 at bit 17, M >> 4 at bit 24;
// a_mn / b_mn = 1: that operand is MN-major (bits 15 / 16), else K-major.
__host__ __device__ constexpr uint32_t instr_desc(int m, int n, int a_mn = 0, int b_mn = 0) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)a_mn << 15) | ((uint32_t)b_mn << 16) |
           ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// 32 consecutive accumulator columns of this thread's tensor-memory lane (warp w reads lanes 32 (w % 4) ..)
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
}

}  // namespace q35
