// umma.cuh — the pieces every tcgen05 kernel of this library shares: mbarrier and bulk-copy wrappers, the shared-memory
// and instruction descriptors of tcgen05.mma, and the host-side lookup of the tensor-map encoder.
#pragma once
#include <cuda.h>  // the CUtensorMap type and enums only: the encoder is looked up through the runtime, nothing links to the driver library

#include <cstdint>

#include <cuda_runtime.h>

namespace {

constexpr int kTileBytes = 128 * 128;  // an MMA operand tile: 128 rows x 64 fp16, K-major, 128-byte swizzle

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_arrive(unsigned bar) {
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
// Bounded wait; false when the barrier did not complete the phase in time (or the CTA is aborting). try_wait suspends
// the thread for a hardware-bounded time instead of spinning: 17 warps share 4 schedulers, and warps that spin on a
// barrier take issue slots from the warps they are waiting for.
constexpr int kWaitPolls = 1 << 20;
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity, volatile int* abort_flag = nullptr, int polls = kWaitPolls) {
    for (int i = 0; i < polls; i++) {
        unsigned ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}\n"
            : "=r"(ok)
            : "r"(bar), "r"(parity)
            : "memory");
        if (ok) return true;
        if (abort_flag && *abort_flag) return false;
    }
    return false;
}

// The same bounded wait, polling with test_wait (which never suspends the thread): for hand-offs on a kernel's critical path
// between a few warps, where the time a suspended thread takes to come back shows in every tile.
__device__ __forceinline__ bool mbar_wait_spin(unsigned bar, unsigned parity, volatile int* abort_flag = nullptr, int polls = kWaitPolls * 16) {
    for (int i = 0; i < polls; i++) {
        unsigned ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}\n"
            : "=r"(ok)
            : "r"(bar), "r"(parity)
            : "memory");
        if (ok) return true;
        if ((i & 63) == 63 && abort_flag && *abort_flag) return false;
    }
    return false;
}

// K-major, 128-byte swizzle, 8-row groups 1024 bytes apart (cute/arch/mma_sm100_desc.hpp SmemDescriptor: start>>4 [0,14),
// LBO>>4 [16,30), SBO>>4 [32,46), version 1 at [46,48), layout type SWIZZLE_128B = 2 at [61,64)).
__device__ __forceinline__ uint64_t umma_desc(unsigned smem_addr) {
    return (uint64_t)((smem_addr >> 4) & 0x3FFFu) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}

// fp32 accumulate, f16 x f16, both K-major, M=128, N = 128 or 256 (InstrDescriptor: c_format [4,6), n>>3 [17,23), m>>4 [24,29)).
__host__ __device__ constexpr unsigned idesc_for(unsigned n) { return (1u << 4) | ((n >> 3) << 17) | ((128u >> 4) << 24); }

__device__ __forceinline__ void umma_f16(unsigned tmem_d, uint64_t adesc, uint64_t bdesc, unsigned idesc, unsigned accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(unsigned bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(unsigned bar, unsigned bytes) {
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t}\n" ::"r"(bar), "r"(bytes) : "memory");
}
// global -> shared bulk copy by the copy engine (no multicast); completion is counted in bytes on the mbarrier.
// Both addresses 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_g2s(unsigned dst, const void* src, unsigned bytes, unsigned bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(dst), "l"(src),
                 "r"(bytes), "r"(bar)
                 : "memory");
}

// 2-D tiled copy by the copy engine (no multicast): box of the tensor map at (x, y) -> shared memory. x * element size
// must be a multiple of 16 bytes.
__device__ __forceinline__ void tensor_g2s_2d(unsigned dst, const CUtensorMap* map, int x, int y, unsigned bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::"r"(dst),
                 "l"(map), "r"(x), "r"(y), "r"(bar)
                 : "memory");
}


typedef CUresult (*tensor_map_encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                         const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                         CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled, reached through the runtime's driver-entry-point lookup; nullptr when this driver lacks it.
inline tensor_map_encode_fn tensor_map_encoder() {
    static tensor_map_encode_fn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<tensor_map_encode_fn>(p);
    }();
    return fn;
}

}  // namespace
