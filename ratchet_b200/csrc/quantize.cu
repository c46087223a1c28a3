// Q8_0 quantiser: ratchet-core/src/quant.rs:19-99 (quantize_inner / quantize) as a library routine,
// on the host (rcu_quantize) and on the device (rcu_quantize_device).
//
// Per 32 consecutive elements (dtype/blocks.rs:180-198: GROUP_SIZE 32, PACK_SIZE 4, SF 127):
//     d   = max|x| / 127                                  stored as the tensor's float type
//     q_j = round_half_away(x_j / d) & 0xFF               four codes per u32, code j at bits 8 j
// and the buffer is the code segment followed by the scale segment, each padded to 256 bytes
// (quant.rs:7-17, gpu/align.rs).  Q8_0F quantises f32 input with f32 arithmetic; Q8_0H quantises f16
// input with every operation rounded to f16, which is what the `half` crate's operators do.  The
// conversions to integer follow Rust's `as i32`: saturating, NaN -> 0 — so an all-zero block
// (d = 0, x / d = NaN) gets zero codes, and `max` ignores a NaN operand as f32::max does.
//
// The Q4_K arms of the reference's quantize() emit an absmax 4-bit layout that is not the Q4_K segment
// layout its loader and kernels use (ratchet-loader/src/gguf/dtype.rs:83-125); they are refused here.
// Q4_K buffers come from GGUF files through rcu_gguf_transcode.
#include <algorithm>
#include <cmath>
#include <cstring>
#include <thread>

#include "common.cuh"

namespace {

inline float half_bits_to_float(uint16_t h) {
    __half v;
    std::memcpy(&v, &h, 2);
    return __half2float(v);
}
inline uint16_t float_to_half_bits(float f) {
    const __half v = __float2half_rn(f);
    uint16_t h;
    std::memcpy(&h, &v, 2);
    return h;
}

// `f32 as i32` of Rust
inline int32_t saturating_i32(float v) {
    if (std::isnan(v)) return 0;
    if (v >= 2147483648.0f) return INT32_MAX;
    if (v <= -2147483648.0f) return INT32_MIN;
    return (int32_t)v;
}

// blocks [b0, b1) of a Q8_0F buffer from f32 input
void quantize_blocks_f32(const float* x, uint64_t b0, uint64_t b1, uint32_t* codes, float* scales) {
    for (uint64_t b = b0; b < b1; ++b) {
        const float* xb = x + b * 32;
        float amax = 0.f;
        for (int j = 0; j < 32; ++j) amax = std::fmax(amax, std::fabs(xb[j]));
        const float d = amax / 127.0f;
        scales[b] = d;
        for (int w = 0; w < 8; ++w) {
            int32_t packed = 0;
            for (int j = 0; j < 4; ++j) packed |= (saturating_i32(std::round(xb[4 * w + j] / d)) & 0xFF) << (8 * j);
            codes[b * 8 + w] = (uint32_t)packed;
        }
    }
}

// blocks [b0, b1) of a Q8_0H buffer from f16 input: f16 arithmetic = f32 operation, then round to nearest even
void quantize_blocks_f16(const uint16_t* x, uint64_t b0, uint64_t b1, uint32_t* codes, uint16_t* scales) {
    for (uint64_t b = b0; b < b1; ++b) {
        const uint16_t* xb = x + b * 32;
        float amax = 0.f;
        for (int j = 0; j < 32; ++j) amax = std::fmax(amax, std::fabs(half_bits_to_float(xb[j])));
        const uint16_t dh = float_to_half_bits(amax / 127.0f);
        const float d = half_bits_to_float(dh);
        scales[b] = dh;
        for (int w = 0; w < 8; ++w) {
            int32_t packed = 0;
            for (int j = 0; j < 4; ++j) {
                const float ratio = half_bits_to_float(float_to_half_bits(half_bits_to_float(xb[4 * w + j]) / d));
                const float r = half_bits_to_float(float_to_half_bits(std::round(ratio)));
                packed |= (saturating_i32(r) & 0xFF) << (8 * j);
            }
            codes[b * 8 + w] = (uint32_t)packed;
        }
    }
}

template <class Fn>
void for_block_ranges(uint64_t n_blocks, const Fn& fn) {
    const unsigned hw = std::max(1u, std::thread::hardware_concurrency());
    const uint64_t n_threads = std::min<uint64_t>(hw, std::max<uint64_t>(1, n_blocks / 4096));
    if (n_threads <= 1) {
        fn(0, n_blocks);
        return;
    }
    std::vector<std::thread> pool;
    for (uint64_t t = 0; t < n_threads; ++t)
        pool.emplace_back([&, t] { fn(t * n_blocks / n_threads, (t + 1) * n_blocks / n_threads); });
    for (auto& th : pool) th.join();
}

// One thread per packed word; the eight threads of a block share its maximum through shuffles.
template <bool HALF>
__global__ void quantize_q8_kernel(const void* __restrict__ src, uint64_t n_words, uint32_t* __restrict__ codes, void* __restrict__ scales) {
    rcu_kernel_entry();
    const uint64_t w = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const bool live = w < n_words;
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    if (live) {
        if (HALF) {
            const uint2 raw = reinterpret_cast<const uint2*>(src)[w];
            const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
            const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
            v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
        } else {
            const float4 raw = reinterpret_cast<const float4*>(src)[w];
            v[0] = raw.x; v[1] = raw.y; v[2] = raw.z; v[3] = raw.w;
        }
    }
    float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));   // fmaxf drops a NaN operand, as f32::max
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
    if (!live) return;
    float d = __fdiv_rn(amax, 127.0f);
    if (HALF) d = __half2float(__float2half_rn(d));
    if ((w & 7) == 0) {
        if (HALF) reinterpret_cast<__half*>(scales)[w >> 3] = __float2half_rn(d);
        else reinterpret_cast<float*>(scales)[w >> 3] = d;
    }
    uint32_t packed = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        float r = __fdiv_rn(v[j], d);
        if (HALF) r = __half2float(__float2half_rn(r));
        r = roundf(r);                                    // half away from zero; exact in f16 at these magnitudes
        packed |= ((uint32_t)__float2int_rz(r) & 0xFFu) << (8 * j);   // saturating, NaN -> 0
    }
    codes[w] = packed;
}

}  // namespace

extern "C" {

rcu_status rcu_quantize(int32_t dt, const void* src, uint64_t numel, void* host_out, uint64_t out_bytes) {
    if (!src || !host_out) return RCU_ERR_INVALID_ARG;
    if (dt != RCU_Q8_0F && dt != RCU_Q8_0H) return RCU_ERR_UNSUPPORTED;
    if (numel % 32 != 0) return RCU_ERR_INVALID_ARG;                   // quant.rs:20-21
    if (out_bytes < rcu_dtype_nbytes(dt, numel)) return RCU_ERR_INVALID_ARG;
    uint64_t off[4];
    rcu_dtype_segments(dt, numel, off);
    std::memset(host_out, 0, rcu_dtype_nbytes(dt, numel));              // the padding of both segments is zero
    uint32_t* codes = reinterpret_cast<uint32_t*>(host_out);
    void* scales = reinterpret_cast<char*>(host_out) + off[1];
    const uint64_t n_blocks = numel / 32;
    if (dt == RCU_Q8_0F)
        for_block_ranges(n_blocks, [&](uint64_t b0, uint64_t b1) { quantize_blocks_f32((const float*)src, b0, b1, codes, (float*)scales); });
    else
        for_block_ranges(n_blocks, [&](uint64_t b0, uint64_t b1) { quantize_blocks_f16((const uint16_t*)src, b0, b1, codes, (uint16_t*)scales); });
    return RCU_OK;
}

rcu_status rcu_quantize_device(rcu_device* dev, const rcu_tensor* src, rcu_tensor* dst) {
    if (!dev) return RCU_ERR_INVALID_ARG;
    RCU_REQUIRE(dev, t_valid(src) && t_valid(dst) && t_same_shape(src, dst), "quantize: src and dst must have the same shape");
    const bool half = dst->dt == RCU_Q8_0H;
    if (!dt_is_q8(dst->dt))
        return rcu_fail(dev, RCU_ERR_UNSUPPORTED, "quantize: only Q8_0F / Q8_0H are produced (Q4_K buffers come from GGUF files)");
    RCU_REQUIRE(dev, src->dt == (half ? RCU_F16 : RCU_F32), "quantize: Q8_0F takes f32 input, Q8_0H takes f16 input (quant.rs:52-76)");
    const uint64_t numel = t_numel(src);
    RCU_REQUIRE(dev, numel % 32 == 0, "quantize: %llu elements are not whole 32-element blocks", (unsigned long long)numel);
    DevGuard g(dev->ordinal);
    uint64_t off[4];
    rcu_dtype_segments(dst->dt, numel, off);
    RCU_CUDA(dev, cudaMemsetAsync(dst->data, 0, rcu_dtype_nbytes(dst->dt, numel), dev->stream));
    const uint64_t n_words = numel / 4;
    if (n_words == 0) return RCU_OK;
    const unsigned grid = (unsigned)((n_words + 255) / 256);
    uint32_t* codes = reinterpret_cast<uint32_t*>(dst->data);
    void* scales = reinterpret_cast<char*>(dst->data) + off[1];
    if (half) rcu_launch(dev, quantize_q8_kernel<true>, grid, 256, 0, src->data, n_words, codes, scales);
    else rcu_launch(dev, quantize_q8_kernel<false>, grid, 256, 0, src->data, n_words, codes, scales);
    RCU_LAUNCH_CHECK(dev);
    return RCU_OK;
}

}  // extern "C"
