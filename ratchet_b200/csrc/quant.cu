// Device-side dequantisation of ratchet's quantised buffers, bit-identical with the CPU routine
// `dequantize` (ratchet-core/src/quant.rs:101-164) for Q8_0 and with the Q4_K decode arithmetic of
// ops/matmul/quantized.rs:158-266 on the segment layout of ratchet-loader/src/gguf/dtype.rs:39-125.
#include "common.cuh"

namespace {

// 16 int8 per thread: one 16-byte load, one scale, 16 products rounded in the scale type.
template <class ScaleT>
__global__ void __launch_bounds__(256)
dequant_q8_kernel(const uint4* __restrict__ q, const ScaleT* __restrict__ d, ScaleT* __restrict__ out, size_t n16) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += stride) {
        const uint4 w = q[i];
        const float sc = to_f32<ScaleT>(d[i >> 1]);
        const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
        ScaleT* o = out + i * 16;
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int v = (int)(ws[a] << (8 * (3 - j))) >> 24;   // quant.rs:121-125
                o[a * 4 + j] = from_f32<ScaleT>((float)v * sc);
            }
    }
}

// one thread per (super-block, 32-weight sub-block)
template <class FP>
__global__ void __launch_bounds__(256)
dequant_q4k_kernel(const uint8_t* __restrict__ qs, const uint8_t* __restrict__ scales, const FP* __restrict__ dmin,
                   const FP* __restrict__ d, FP* __restrict__ out, size_t nsub) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < nsub; i += stride) {
        const size_t b = i >> 3;
        const int j = (int)(i & 7);
        const uint8_t* sc = scales + b * 12;
        uint32_t s, m;
        if (j < 4) {
            s = sc[j] & 63u;
            m = sc[j + 4] & 63u;
        } else {
            s = (sc[j + 4] & 0xFu) | ((uint32_t)(sc[j - 4] >> 6) << 4);
            m = (uint32_t)(sc[j + 4] >> 4) | ((uint32_t)(sc[j] >> 6) << 4);
        }
        const float delta = rnd<FP>((float)s * to_f32<FP>(d[b]));
        const float mn = rnd<FP>((float)m * to_f32<FP>(dmin[b]));
        const uint8_t* qb = qs + b * 128 + (j >> 1) * 32;
        FP* o = out + b * 256 + j * 32;
        const int shift = (j & 1) * 4;
#pragma unroll 8
        for (int l = 0; l < 32; ++l) o[l] = from_f32<FP>(fmaf((float)((qb[l] >> shift) & 0xF), delta, -mn));
    }
}

}  // namespace

extern "C" rcu_status rcu_dequantize(rcu_device* dev, const rcu_tensor* src, rcu_tensor* dst) {
    if (!dev) return RCU_ERR_INVALID_ARG;
    RCU_REQUIRE(dev, t_valid(src) && t_valid(dst), "dequantize: invalid tensor descriptor");
    RCU_REQUIRE(dev, dt_is_quant(src->dt), "Unsupported dtype %d", src->dt);
    RCU_REQUIRE(dev, dst->dt == rcu_activation_dtype(src->dt) && t_numel(dst) == t_numel(src), "dequantize: dst must be the activation dtype with the same shape");
    const size_t n = t_numel(src);
    DevGuard g(dev->ordinal);
    uint64_t off[4];
    rcu_dtype_segments(src->dt, n, off);
    const char* base = (const char*)src->data;
    const int cap = dev->sm_count * 8;
    if (dt_is_q8(src->dt)) {
        RCU_REQUIRE(dev, n % 32 == 0, "dequantize: Q8_0 needs a multiple of 32 elements");   // quant.rs:102-103
        const size_t n16 = n / 16;
        const int grid = (int)std::min<size_t>((n16 + 255) / 256, (size_t)cap);
        if (src->dt == RCU_Q8_0F) dequant_q8_kernel<float><<<grid, 256, 0, dev->stream>>>((const uint4*)base, (const float*)(base + off[1]), (float*)dst->data, n16);
        else dequant_q8_kernel<__half><<<grid, 256, 0, dev->stream>>>((const uint4*)base, (const __half*)(base + off[1]), (__half*)dst->data, n16);
    } else {
        RCU_REQUIRE(dev, n % 256 == 0, "dequantize: Q4_K needs a multiple of 256 elements");
        const size_t nsub = n / 32;
        const int grid = (int)std::min<size_t>((nsub + 255) / 256, (size_t)cap);
        if (src->dt == RCU_Q4_KF) dequant_q4k_kernel<float><<<grid, 256, 0, dev->stream>>>((const uint8_t*)base, (const uint8_t*)base + off[1], (const float*)(base + off[2]), (const float*)(base + off[3]), (float*)dst->data, nsub);
        else dequant_q4k_kernel<__half><<<grid, 256, 0, dev->stream>>>((const uint8_t*)base, (const uint8_t*)base + off[1], (const __half*)(base + off[2]), (const __half*)(base + off[3]), (__half*)dst->data, nsub);
    }
    RCU_LAUNCH_CHECK(dev);
    return RCU_OK;
}
