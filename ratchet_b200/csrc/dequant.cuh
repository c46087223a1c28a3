// Register-level dequantisation of ratchet's Q8_0 and Q4_K codes to f16, shared by the dequantise
// kernels and by the tensor-core GEMM that converts weight tiles in shared memory.  The arithmetic is
// the CPU dequantiser's: Q8_0 w = fp16(q * d) (quant.rs:121-125), Q4_K w = fma(q, delta, -min) in f16
// with one rounding (ops/matmul/quantized.rs:207-230).  Integer codes become f16 values through
// the exponent trick (code bits under the exponent of 1024, then an exact subtraction) instead of
// integer-to-float conversions.
#pragma once
#include <cuda_fp16.h>

#include <cstdint>

namespace rcu_dequant {

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}
__device__ __forceinline__ __half2 as_h2(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }
__device__ __forceinline__ uint32_t as_u32(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }

// 8 consecutive int8 (two packed words) -> 8 f16 weights q * d.  byte ^ 0x80 under exponent byte 0x64
// is the half 1024 + (q + 128); subtracting 1152 gives q exactly, and the f16 product q * d is the f32
// product rounded once (quant.rs:121-125 on f16 scales).
__device__ __forceinline__ uint4 dequant8_q8(uint32_t w0, uint32_t w1, __half2 d2) {
    const __half2 off = __float2half2_rn(1152.0f);
    const uint32_t x0 = w0 ^ 0x80808080u, x1 = w1 ^ 0x80808080u;
    uint4 o;
    o.x = as_u32(__hmul2_rn(__hsub2_rn(as_h2(prmt(x0, 0x64646464u, 0x4140u)), off), d2));
    o.y = as_u32(__hmul2_rn(__hsub2_rn(as_h2(prmt(x0, 0x64646464u, 0x4342u)), off), d2));
    o.z = as_u32(__hmul2_rn(__hsub2_rn(as_h2(prmt(x1, 0x64646464u, 0x4140u)), off), d2));
    o.w = as_u32(__hmul2_rn(__hsub2_rn(as_h2(prmt(x1, 0x64646464u, 0x4342u)), off), d2));
    return o;
}

// 8 consecutive 4-bit codes (the low nibbles of two words already shifted for the sub-block) ->
// fma(q, delta, -min) in f16 with a single rounding (quantized.rs:230).
__device__ __forceinline__ uint4 dequant8_q4(uint32_t x0, uint32_t x1, __half2 delta2, __half2 negmin2) {
    const __half2 k1024 = __float2half2_rn(1024.0f);
    uint4 o;
    {
        const uint32_t p02 = (x0 & 0x000F000Fu) | 0x64006400u, p13 = ((x0 >> 8) & 0x000F000Fu) | 0x64006400u;
        o.x = as_u32(__hfma2(__hsub2_rn(as_h2(prmt(p02, p13, 0x5410u)), k1024), delta2, negmin2));
        o.y = as_u32(__hfma2(__hsub2_rn(as_h2(prmt(p02, p13, 0x7632u)), k1024), delta2, negmin2));
    }
    {
        const uint32_t p02 = (x1 & 0x000F000Fu) | 0x64006400u, p13 = ((x1 >> 8) & 0x000F000Fu) | 0x64006400u;
        o.z = as_u32(__hfma2(__hsub2_rn(as_h2(prmt(p02, p13, 0x5410u)), k1024), delta2, negmin2));
        o.w = as_u32(__hfma2(__hsub2_rn(as_h2(prmt(p02, p13, 0x7632u)), k1024), delta2, negmin2));
    }
    return o;
}

// byte i (0..11) of a 12-byte pack held in three registers (selects, no indexed register array)
__device__ __forceinline__ uint32_t pack_byte(const uint32_t* w, int i) {
    const uint32_t word = i < 4 ? w[0] : (i < 8 ? w[1] : w[2]);
    return (word >> (8 * (i & 3))) & 0xFFu;
}

}  // namespace rcu_dequant
