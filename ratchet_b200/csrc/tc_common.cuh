// Pieces shared by the tcgen05 GEMM kernels: mbarrier / TMA helpers (bulk_async.cuh), the
// shared-memory matrix descriptor for 128-byte-swizzled K-major tiles, fences, commit and the
// tensor-memory load used by the epilogues.
#pragma once
#include <cuda.h>

#include "bulk_async.cuh"   // mbarrier + tensor-map helpers

namespace tc {

using gemvq8::mbar_arrive;
using gemvq8::mbar_expect_tx;
using gemvq8::mbar_init;
using gemvq8::mbar_wait;
using gemvq8::mbar_wait_spin;
using gemvq8::smem_u32;
using gemvq8::tma_load_2d;
using gemvq8::tma_load_3d;

constexpr int TM = 128;          // tokens per tile (UMMA M)
constexpr int TK = 64;           // K per stage: 64 f16 = 128 bytes = one swizzle row
constexpr int kStages = 4;
constexpr int kThreadsTc = 192;  // 6 warps

// 64-bit shared-memory matrix descriptor, K-major operand, 128-byte swizzle:
// rows of 128 bytes, 8-row groups 1024 bytes apart (SBO), descriptor version 1 (sm_100).
__device__ __forceinline__ uint64_t umma_desc_sw128(const void* smem_ptr) {
    const uint32_t addr = smem_u32(smem_ptr);
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFF) >> 4);            // start address, 16-byte units
    d |= (uint64_t)0 << 16;                            // leading byte offset: unused for swizzled K-major
    d |= (uint64_t)(1024 >> 4) << 32;                  // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                            // descriptor version
    d |= (uint64_t)2 << 61;                            // SWIZZLE_128B
    return d;
}

// 32-bit instruction descriptor, kind::f16: f16 A and B (both K-major), f32 D, M x N tile.
__host__ __device__ constexpr uint32_t umma_idesc_f16(int m, int n) {
    return (1u << 4)                      // D format f32
           | (0u << 7) | (0u << 10)       // A, B format f16
           | (0u << 15) | (0u << 16)      // A, B K-major
           | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// arrive on `bar` once every tcgen05.mma issued so far by this thread has finished
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// 32 lanes x 32 consecutive f32 columns of tensor memory -> 32 registers per thread
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, float* v) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}


}  // namespace tc
