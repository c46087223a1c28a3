// Device-side dequantisation of ratchet's quantised buffers, bit-identical with the CPU routine
// `dequantize` (ratchet-core/src/quant.rs:101-164) for Q8_0 and with the Q4_K decode arithmetic of
// ops/matmul/quantized.rs:158-266 on the segment layout of ratchet-loader/src/gguf/dtype.rs:39-125.
#include "common.cuh"
#include "dequant.cuh"

namespace {

template <class T> struct Pack8;
template <> struct Pack8<__half> {
    __device__ static __forceinline__ void store(__half* dst, const float* v) {
        __align__(16) __half h[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) h[i] = __float2half_rn(v[i]);
        *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(h);
    }
};
template <> struct Pack8<float> {
    __device__ static __forceinline__ void store(float* dst, const float* v) {
        reinterpret_cast<float4*>(dst)[0] = make_float4(v[0], v[1], v[2], v[3]);
        reinterpret_cast<float4*>(dst)[1] = make_float4(v[4], v[5], v[6], v[7]);
    }
};

// 8 int8 per thread: one 8-byte load, one scale, products rounded once in the scale type, one
// 16-byte (f16) or two 16-byte (f32) stores; consecutive threads write consecutive vectors.
template <class ScaleT>
__global__ void __launch_bounds__(256)
dequant_q8_kernel(const uint2* __restrict__ q, const ScaleT* __restrict__ d, ScaleT* __restrict__ out, size_t n8) {
    rcu_kernel_entry();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += stride) {
        const uint2 w = q[i];
        if (sizeof(ScaleT) == 2) {   // f16: exponent-trick conversion and a native f16 multiply (same rounding)
            const __half dh = reinterpret_cast<const __half*>(d)[i >> 2];
            *reinterpret_cast<uint4*>(out + i * 8) = rcu_dequant::dequant8_q8(w.x, w.y, __half2half2(dh));
            continue;
        }
        const float sc = to_f32<ScaleT>(d[i >> 2]);
        const uint32_t ws[2] = {w.x, w.y};
        float v[8];
#pragma unroll
        for (int a = 0; a < 2; ++a)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int qv = (int)(ws[a] << (8 * (3 - j))) >> 24;   // quant.rs:121-125
                v[a * 4 + j] = rnd<ScaleT>((float)qv * sc);
            }
        Pack8<ScaleT>::store(out + i * 8, v);
    }
}

using rcu_dequant::pack_byte;

// Thread = (super-block b, 32-byte chunk c, quarter q of the chunk): one 8-byte load of nibble bytes
// yields 8 weights of sub-block 2c (low nibbles) and 8 of sub-block 2c+1 (high nibbles), each stored
// as one 16-byte vector; four neighbouring lanes fill 64 consecutive bytes of each sub-block.  The pack
// of 6-bit codes is read as three words, d and dmin once.
template <class FP>
__global__ void __launch_bounds__(256)
dequant_q4k_kernel(const uint8_t* __restrict__ qs, const uint8_t* __restrict__ scales, const FP* __restrict__ dmin,
                   const FP* __restrict__ d, FP* __restrict__ out, size_t nthreads) {
    rcu_kernel_entry();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < nthreads; i += stride) {
        const size_t b = i >> 4;
        const int c = (int)(i >> 2) & 3, q = (int)i & 3;
        const uint2 qw = *reinterpret_cast<const uint2*>(qs + b * 128 + c * 32 + q * 8);
        const uint32_t* pk = reinterpret_cast<const uint32_t*>(scales + b * 12);
        const uint32_t w[3] = {pk[0], pk[1], pk[2]};
        const float df = to_f32<FP>(d[b]), mf = to_f32<FP>(dmin[b]);
#pragma unroll
        for (int hi = 0; hi < 2; ++hi) {
            const int j = 2 * c + hi;
            uint32_t s, m;
            if (j < 4) {
                s = pack_byte(w, j) & 63u;
                m = pack_byte(w, j + 4) & 63u;
            } else {
                s = (pack_byte(w, j + 4) & 0xFu) | ((pack_byte(w, j - 4) >> 6) << 4);
                m = (pack_byte(w, j + 4) >> 4) | ((pack_byte(w, j) >> 6) << 4);
            }
            const float delta = rnd<FP>((float)s * df);
            const float mn = rnd<FP>((float)m * mf);
            FP* o = out + b * 256 + j * 32 + q * 8;
            if (sizeof(FP) == 2) {   // f16: fma(q, delta, -min) with one rounding is the native half2 fma
                const __half2 d2 = __float2half2_rn(delta), n2 = __float2half2_rn(-mn);   // both exact f16 values
                *reinterpret_cast<uint4*>(o) = rcu_dequant::dequant8_q4(qw.x >> (4 * hi), qw.y >> (4 * hi), d2, n2);
                continue;
            }
            const uint32_t ws[2] = {qw.x, qw.y};
            float v[8];
#pragma unroll
            for (int a = 0; a < 2; ++a)
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    v[a * 4 + e] = rnd<FP>(fmaf((float)((ws[a] >> (8 * e + 4 * hi)) & 0xF), delta, -mn));
            Pack8<FP>::store(o, v);
        }
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
        const size_t n8 = n / 8;
        const int grid = (int)std::min<size_t>((n8 + 255) / 256, (size_t)cap);
        if (src->dt == RCU_Q8_0F) rcu_launch(dev, dequant_q8_kernel<float>, grid, 256, 0, (const uint2*)base, (const float*)(base + off[1]), (float*)dst->data, n8);
        else rcu_launch(dev, dequant_q8_kernel<__half>, grid, 256, 0, (const uint2*)base, (const __half*)(base + off[1]), (__half*)dst->data, n8);
    } else {
        RCU_REQUIRE(dev, n % 256 == 0, "dequantize: Q4_K needs a multiple of 256 elements");
        const size_t nsub = n / 16;
        const int grid = (int)std::min<size_t>((nsub + 255) / 256, (size_t)cap);
        if (src->dt == RCU_Q4_KF) rcu_launch(dev, dequant_q4k_kernel<float>, grid, 256, 0, (const uint8_t*)base, (const uint8_t*)base + off[1], (const float*)(base + off[2]), (const float*)(base + off[3]), (float*)dst->data, nsub);
        else rcu_launch(dev, dequant_q4k_kernel<__half>, grid, 256, 0, (const uint8_t*)base, (const uint8_t*)base + off[1], (const __half*)(base + off[2]), (const __half*)(base + off[3]), (__half*)dst->data, nsub);
    }
    RCU_LAUNCH_CHECK(dev);
    return RCU_OK;
}
