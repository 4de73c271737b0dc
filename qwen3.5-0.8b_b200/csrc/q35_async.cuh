// Asynchronous-copy plumbing shared by the kernels: shared-memory addresses, the nanosecond clock,
// mbarrier helpers with BOUNDED waits (a wait polls for about one second, then reports failure; the
// caller raises the engine's status word and leaves without touching anything further), bulk and
// tensor copies, and the driver entry point that encodes tensor maps.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace q35 {

constexpr unsigned long long kWaitLimitNs = 1000000000ull;      // one second

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}

// Spin on the barrier's phase (try_wait suspends the thread for a hardware-chosen time); false on expiry.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    unsigned long long t0 = 0;
    for (int it = 0;; ++it) {
        uint32_t ok;
        asm volatile(
            "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
            " selp.u32 %0, 1, 0, p;\n}\n"
            : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
        if (it == 0) t0 = global_ns();
        else if (global_ns() - t0 > kWaitLimitNs) return false;
    }
}

// The same for waits every thread of a CTA takes part in: test, sleep 20 ns, test again.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity) {
    const unsigned long long t0 = global_ns();
    for (;;) {
        uint32_t ok;
        asm volatile(
            "{\n .reg .pred p;\n mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
            " selp.u32 %0, 1, 0, p;\n}\n"
            : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
        if (global_ns() - t0 > kWaitLimitNs) return false;
        __nanosleep(20);
    }
}

// global -> shared bulk copy (16-byte aligned addresses, size a multiple of 16), completing on `bar`
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
        ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
// 2-D tensor copy of one box at element coordinates (c0 innermost, c1); no multicast anywhere
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1) : "memory");
}

// cuTensorMapEncodeTiled through the runtime's driver entry point (no link against libcuda)
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
inline EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    return fn;
}

}  // namespace q35
