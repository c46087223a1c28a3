// Decode GEMV: y[N] = W[N,K] . x[K] (+ bias), W in ratchet's Q8_0 segment layout or plain f16/f32.
//
// Takes the place of ratchet-core's subgroup_gemv / workgroup_gemv WGSL kernels
// (ops/matmul/subgroup_gemv.rs:89-309, ops/matmul/workgroup_gemv.rs:221-371) for the case
// Matmul::select_kernel (ops/matmul/mod.rs:716-748) routes to them: rhs is a vector and lhs is not
// transposed.
//
// The kernel is HBM-bound: every weight byte is read exactly once.  Layout of the work:
//   * persistent CTAs (a multiple of the SM count), 8 warps each; the activation vector is staged
//     once per CTA in shared memory;
//   * rows are dealt to warps as contiguous ranges (balanced to one row), so there is no tail wave;
//   * a warp walks K in 512-element chunks, each lane owning 16 consecutive int8 (one 16-byte
//     streaming load per row per chunk), ROWS rows at a time so that ROWS x UNROLL loads are in
//     flight per lane and the activation registers are reused ROWS times;
//   * int8 -> f16 conversion is exact (byte ^ 0x80 placed in the mantissa of 1024.0h, minus 1152),
//     products are accumulated in f32 with the sm_100 mixed-precision fma (f16 x f16 + f32), one
//     f32 multiply by the block scale per 16 elements, warp-shuffle reduction at the end;
//   * small N: KSPLIT warps share a row range and split K, combined through shared memory.
#include "common.cuh"

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}

// f32 += f16 * f16 (exact product, f32 accumulate); sm_100 mixed-precision fma.
__device__ __forceinline__ float fma_mixed(uint16_t a, uint16_t b, float c) {
    float d;
    asm("fma.rn.f32.f16 %0, %1, %2, %3;" : "=f"(d) : "h"(a), "h"(b), "f"(c));
    return d;
}
__device__ __forceinline__ void split_h2(uint32_t v, uint16_t& lo, uint16_t& hi) {
    asm("mov.b32 {%0, %1}, %2;" : "=h"(lo), "=h"(hi) : "r"(v));
}

// four packed int8 -> two half2 holding the exact integer values
__device__ __forceinline__ void i8x4_to_h2x2(uint32_t w, uint32_t& h01, uint32_t& h23) {
    const uint32_t t = w ^ 0x80808080u;                 // q + 128 in each byte
    const uint32_t a = prmt(t, 0x64646464u, 0x4140u);   // {1024 + b0, 1024 + b1}
    const uint32_t b = prmt(t, 0x64646464u, 0x4342u);   // {1024 + b2, 1024 + b3}
    const __half2 k = __halves2half2(__ushort_as_half(0x6480), __ushort_as_half(0x6480));  // 1152
    __half2 ha = __hsub2(*reinterpret_cast<const __half2*>(&a), k);
    __half2 hb = __hsub2(*reinterpret_cast<const __half2*>(&b), k);
    h01 = *reinterpret_cast<uint32_t*>(&ha);
    h23 = *reinterpret_cast<uint32_t*>(&hb);
}

// dot of 16 int8 (one uint4) with 16 activations
template <class ActT> struct Dot16;

template <> struct Dot16<__half> {
    uint32_t x[8];  // 16 halves
    __device__ __forceinline__ void load(const __half* xs, int k) {
        const uint4 a = *reinterpret_cast<const uint4*>(xs + k);
        const uint4 b = *reinterpret_cast<const uint4*>(xs + k + 8);
        x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w;
        x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
    }
    __device__ __forceinline__ float dot(const uint4& w) const {
        const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
        float p0 = 0.f, p1 = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            uint32_t h01, h23;
            i8x4_to_h2x2(ws[i], h01, h23);
            uint16_t q0, q1, q2, q3, x0, x1, x2, x3;
            split_h2(h01, q0, q1);
            split_h2(h23, q2, q3);
            split_h2(x[2 * i], x0, x1);
            split_h2(x[2 * i + 1], x2, x3);
            p0 = fma_mixed(q0, x0, p0);
            p1 = fma_mixed(q1, x1, p1);
            p0 = fma_mixed(q2, x2, p0);
            p1 = fma_mixed(q3, x3, p1);
        }
        return p0 + p1;
    }
};

template <> struct Dot16<float> {
    float x[16];
    __device__ __forceinline__ void load(const float* xs, int k) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float4 v = *reinterpret_cast<const float4*>(xs + k + 4 * i);
            x[4 * i] = v.x; x[4 * i + 1] = v.y; x[4 * i + 2] = v.z; x[4 * i + 3] = v.w;
        }
    }
    __device__ __forceinline__ float dot(const uint4& w) const {
        const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
        float p0 = 0.f, p1 = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            // byte j of (w ^ 0x80..) in the mantissa of 2^23: value 8388608 + q + 128, exact
            const uint32_t t = ws[i] ^ 0x80808080u;
            const float q0 = __uint_as_float(prmt(t, 0x4B000000u, 0x7440u)) - 8388736.f;
            const float q1 = __uint_as_float(prmt(t, 0x4B000000u, 0x7441u)) - 8388736.f;
            const float q2 = __uint_as_float(prmt(t, 0x4B000000u, 0x7442u)) - 8388736.f;
            const float q3 = __uint_as_float(prmt(t, 0x4B000000u, 0x7443u)) - 8388736.f;
            p0 = fmaf(q0, x[4 * i], p0);
            p1 = fmaf(q1, x[4 * i + 1], p1);
            p0 = fmaf(q2, x[4 * i + 2], p0);
            p1 = fmaf(q3, x[4 * i + 3], p1);
        }
        return p0 + p1;
    }
};

template <class ScaleT> __device__ __forceinline__ float ld_scale(const ScaleT* p);
template <> __device__ __forceinline__ float ld_scale<float>(const float* p) { return __ldg(p); }
template <> __device__ __forceinline__ float ld_scale<__half>(const __half* p) {
    return __half2float(__ushort_as_half(__ldg(reinterpret_cast<const unsigned short*>(p))));
}

// Dequantised weights of the reference are rounded to the scale type (f16 for Q8_0H): w = fp(q*d).
// y = sum_k w_k x_k is evaluated here as sum over blocks of d * (sum q x), which differs from the
// reference only by f32/f16 rounding of individual products (inside the 1e-2 matmul tolerance).

template <class ScaleT, class ActT, int ROWS, int KSPLIT, int UNROLL>
__global__ void __launch_bounds__(kThreads)
gemv_q8_kernel(const int8_t* __restrict__ qs, const ScaleT* __restrict__ scales, const ActT* __restrict__ x,
               const ActT* __restrict__ bias, ActT* __restrict__ y, int N, int K) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    ActT* xs = reinterpret_cast<ActT*>(smem_raw);
    float* red = reinterpret_cast<float*>(smem_raw + (size_t)K * sizeof(ActT));  // [kWarps][ROWS]

    const int tid = threadIdx.x;
    {   // stage the activation vector, 16 bytes per thread per step (K % 32 == 0)
        const int vec = 16 / (int)sizeof(ActT);
        const uint4* src = reinterpret_cast<const uint4*>(x);
        uint4* dst = reinterpret_cast<uint4*>(xs);
        for (int i = tid; i < K / vec; i += kThreads) dst[i] = __ldg(src + i);
    }
    __syncthreads();

    const int warp = tid >> 5, lane = tid & 31;
    constexpr int RG = kWarps / KSPLIT;          // row groups (independent row ranges) per CTA
    const int rg = warp / KSPLIT, ks = warp % KSPLIT;
    const long long gw = (long long)blockIdx.x * RG + rg;   // global row-group index
    const long long W = (long long)gridDim.x * RG;
    const int row_begin = (int)((gw * N) / W);
    const int row_end = (int)(((gw + 1) * N) / W);
    const int kblocks = K >> 5;                  // scales per row
    const int nchunks = (K + 511) >> 9;          // 512-element chunks per row
    const int kl = lane << 4;                    // lane offset inside a chunk

    for (int r0 = row_begin; r0 < row_end; r0 += ROWS) {
        float acc[ROWS];
        const int8_t* wrow[ROWS];
        const ScaleT* srow[ROWS];
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            acc[r] = 0.f;
            const int row = min(r0 + r, row_end - 1);   // duplicate the last row; its result is dropped
            wrow[r] = qs + (size_t)row * K;
            srow[r] = scales + (size_t)row * kblocks;
        }
        for (int c0 = ks; c0 < nchunks; c0 += KSPLIT * UNROLL) {
            uint4 w[UNROLL][ROWS];
            float sc[UNROLL][ROWS];
            bool live[UNROLL];
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                const int k = ((c0 + u * KSPLIT) << 9) + kl;
                live[u] = k < K;
#pragma unroll
                for (int r = 0; r < ROWS; ++r) {
                    if (live[u]) {
                        w[u][r] = ld_stream_v4(wrow[r] + k);
                        sc[u][r] = ld_scale<ScaleT>(srow[r] + (k >> 5));
                    } else {
                        w[u][r] = make_uint4(0x0, 0x0, 0x0, 0x0);
                        sc[u][r] = 0.f;
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                if (!live[u]) continue;
                const int k = ((c0 + u * KSPLIT) << 9) + kl;
                Dot16<ActT> d16;
                d16.load(xs, k);
#pragma unroll
                for (int r = 0; r < ROWS; ++r) acc[r] = fmaf(d16.dot(w[u][r]), sc[u][r], acc[r]);
            }
        }
#pragma unroll
        for (int r = 0; r < ROWS; ++r) acc[r] = warp_sum(acc[r]);

        if (KSPLIT > 1) {
            // combine the K-splits of this row group through shared memory
            if (lane == 0) {
#pragma unroll
                for (int r = 0; r < ROWS; ++r) red[warp * ROWS + r] = acc[r];
            }
            asm volatile("bar.sync %0, %1;" ::"r"(1 + rg), "r"(KSPLIT * 32) : "memory");
            if (ks == 0 && lane < ROWS) {
                float s = 0.f;
#pragma unroll
                for (int j = 0; j < KSPLIT; ++j) s += red[(rg * KSPLIT + j) * ROWS + lane];
                const int row = r0 + lane;
                if (row < row_end) {
                    if (bias) s += to_f32<ActT>(bias[row]);
                    y[row] = from_f32<ActT>(s);
                }
            }
            asm volatile("bar.sync %0, %1;" ::"r"(1 + rg), "r"(KSPLIT * 32) : "memory");
        } else {
            if (lane == 0) {
#pragma unroll
                for (int r = 0; r < ROWS; ++r) {
                    const int row = r0 + r;
                    if (row < row_end) {
                        float s = acc[r];
                        if (bias) s += to_f32<ActT>(bias[row]);
                        y[row] = from_f32<ActT>(s);
                    }
                }
            }
        }
    }
}

// Plain f16 / f32 weights: same work layout, 16 bytes (8 halves / 4 floats) per lane per step.
template <class T, int ROWS, int KSPLIT, int UNROLL>
__global__ void __launch_bounds__(kThreads)
gemv_float_kernel(const T* __restrict__ Wm, const T* __restrict__ x, const T* __restrict__ bias, T* __restrict__ y,
                  int N, int K) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    T* xs = reinterpret_cast<T*>(smem_raw);
    float* red = reinterpret_cast<float*>(smem_raw + (((size_t)K * sizeof(T) + 15) / 16) * 16);
    const int tid = threadIdx.x;
    for (int i = tid; i < K; i += kThreads) xs[i] = x[i];
    __syncthreads();
    constexpr int VEC = 16 / (int)sizeof(T);
    const int warp = tid >> 5, lane = tid & 31;
    constexpr int RG = kWarps / KSPLIT;
    const int rg = warp / KSPLIT, ks = warp % KSPLIT;
    const long long gw = (long long)blockIdx.x * RG + rg;
    const long long W = (long long)gridDim.x * RG;
    const int row_begin = (int)((gw * N) / W);
    const int row_end = (int)(((gw + 1) * N) / W);
    constexpr int CH = 32 * VEC;                  // elements per warp step
    const int nchunks = (K + CH - 1) / CH;
    const bool vec_ok = (K % VEC) == 0;           // rows stay 16-byte aligned

    for (int r0 = row_begin; r0 < row_end; r0 += ROWS) {
        float acc[ROWS];
#pragma unroll
        for (int r = 0; r < ROWS; ++r) acc[r] = 0.f;
        if (vec_ok) {
            for (int c0 = ks; c0 < nchunks; c0 += KSPLIT * UNROLL) {
                uint4 w[UNROLL][ROWS];
                bool live[UNROLL];
#pragma unroll
                for (int u = 0; u < UNROLL; ++u) {
                    const int k = (c0 + u * KSPLIT) * CH + lane * VEC;
                    live[u] = k < K;
#pragma unroll
                    for (int r = 0; r < ROWS; ++r) {
                        const int row = min(r0 + r, row_end - 1);
                        w[u][r] = live[u] ? ld_stream_v4(Wm + (size_t)row * K + k) : make_uint4(0, 0, 0, 0);
                    }
                }
#pragma unroll
                for (int u = 0; u < UNROLL; ++u) {
                    if (!live[u]) continue;
                    const int k = (c0 + u * KSPLIT) * CH + lane * VEC;
                    float xv[VEC];
#pragma unroll
                    for (int j = 0; j < VEC; ++j) xv[j] = to_f32<T>(xs[k + j]);
#pragma unroll
                    for (int r = 0; r < ROWS; ++r) {
                        const T* wv = reinterpret_cast<const T*>(&w[u][r]);
#pragma unroll
                        for (int j = 0; j < VEC; ++j) acc[r] = fmaf(to_f32<T>(wv[j]), xv[j], acc[r]);
                    }
                }
            }
        } else {
            for (int k = ks * 32 + lane; k < K; k += KSPLIT * 32) {
                const float xv = to_f32<T>(xs[k]);
#pragma unroll
                for (int r = 0; r < ROWS; ++r) {
                    const int row = min(r0 + r, row_end - 1);
                    acc[r] = fmaf(to_f32<T>(Wm[(size_t)row * K + k]), xv, acc[r]);
                }
            }
        }
#pragma unroll
        for (int r = 0; r < ROWS; ++r) acc[r] = warp_sum(acc[r]);
        if (KSPLIT > 1) {
            if (lane == 0) {
#pragma unroll
                for (int r = 0; r < ROWS; ++r) red[warp * ROWS + r] = acc[r];
            }
            asm volatile("bar.sync %0, %1;" ::"r"(1 + rg), "r"(KSPLIT * 32) : "memory");
            if (ks == 0 && lane < ROWS) {
                float s = 0.f;
#pragma unroll
                for (int j = 0; j < KSPLIT; ++j) s += red[(rg * KSPLIT + j) * ROWS + lane];
                const int row = r0 + lane;
                if (row < row_end) {
                    if (bias) s += to_f32<T>(bias[row]);
                    y[row] = from_f32<T>(s);
                }
            }
            asm volatile("bar.sync %0, %1;" ::"r"(1 + rg), "r"(KSPLIT * 32) : "memory");
        } else if (lane == 0) {
#pragma unroll
            for (int r = 0; r < ROWS; ++r) {
                const int row = r0 + r;
                if (row < row_end) {
                    float s = acc[r];
                    if (bias) s += to_f32<T>(bias[row]);
                    y[row] = from_f32<T>(s);
                }
            }
        }
    }
}

struct GemvPlan { int ksplit; int grid; };

// Pick the K split and grid: enough warps in flight to cover HBM latency even when N is small.
GemvPlan plan_gemv(const rcu_device* dev, int N, int K, int rows_per_warp, int ctas_per_sm) {
    GemvPlan p;
    const long long max_ctas = (long long)dev->sm_count * ctas_per_sm;
    // row groups needed if every warp took rows_per_warp rows and the full K
    const long long groups = (N + rows_per_warp - 1) / rows_per_warp;
    const long long warps_wanted = max_ctas * kWarps;
    int ksplit = 1;
    while (ksplit < 8 && groups * ksplit * 2 <= warps_wanted && (K / (ksplit * 2)) >= 1024) ksplit *= 2;
    p.ksplit = ksplit;
    const long long ctas_needed = (groups * ksplit + kWarps - 1) / kWarps;
    p.grid = (int)(ctas_needed < max_ctas ? (ctas_needed < 1 ? 1 : ctas_needed) : max_ctas);
    return p;
}

template <class ScaleT, class ActT>
rcu_status launch_q8(rcu_device* dev, const int8_t* qs, const void* scales, const void* x, const void* bias, void* y,
                     int N, int K) {
    constexpr int ROWS = 4, UNROLL = 2;
    const int ctas_per_sm = 3;
    GemvPlan p = plan_gemv(dev, N, K, ROWS, ctas_per_sm);
    const size_t smem = (size_t)K * sizeof(ActT) + kWarps * ROWS * sizeof(float);
    if (smem > (size_t)dev->smem_optin) return rcu_fail(dev, RCU_ERR_UNSUPPORTED, "gemv: K=%d does not fit the activation stage", K);
#define RCU_GEMV_Q8_CASE(KS)                                                                               \
    case KS: {                                                                                             \
        auto kern = gemv_q8_kernel<ScaleT, ActT, ROWS, KS, UNROLL>;                                        \
        if (smem > 48 * 1024) RCU_CUDA(dev, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        kern<<<p.grid, kThreads, smem, dev->stream>>>(qs, (const ScaleT*)scales, (const ActT*)x, (const ActT*)bias, \
                                                      (ActT*)y, N, K);                                     \
        break;                                                                                             \
    }
    switch (p.ksplit) {
        RCU_GEMV_Q8_CASE(1)
        RCU_GEMV_Q8_CASE(2)
        RCU_GEMV_Q8_CASE(4)
        RCU_GEMV_Q8_CASE(8)
    }
#undef RCU_GEMV_Q8_CASE
    RCU_LAUNCH_CHECK(dev);
    return RCU_OK;
}

template <class T>
rcu_status launch_float(rcu_device* dev, const void* Wm, const void* x, const void* bias, void* y, int N, int K) {
    constexpr int ROWS = 4, UNROLL = 2;
    GemvPlan p = plan_gemv(dev, N, K, ROWS, 3);
    const size_t smem = (((size_t)K * sizeof(T) + 15) / 16) * 16 + kWarps * ROWS * sizeof(float);
    if (smem > (size_t)dev->smem_optin) return rcu_fail(dev, RCU_ERR_UNSUPPORTED, "gemv: K=%d does not fit the activation stage", K);
#define RCU_GEMV_F_CASE(KS)                                                                                \
    case KS: {                                                                                             \
        auto kern = gemv_float_kernel<T, ROWS, KS, UNROLL>;                                                \
        if (smem > 48 * 1024) RCU_CUDA(dev, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        kern<<<p.grid, kThreads, smem, dev->stream>>>((const T*)Wm, (const T*)x, (const T*)bias, (T*)y, N, K); \
        break;                                                                                             \
    }
    switch (p.ksplit) {
        RCU_GEMV_F_CASE(1)
        RCU_GEMV_F_CASE(2)
        RCU_GEMV_F_CASE(4)
        RCU_GEMV_F_CASE(8)
    }
#undef RCU_GEMV_F_CASE
    RCU_LAUNCH_CHECK(dev);
    return RCU_OK;
}

}  // namespace

// Called by rcu_matmul once it has established: lhs = W[N,K] (stack 1, not transposed), rhs is a
// vector of K elements, dst holds N elements of the rhs dtype.
rcu_status rcu_gemv_dispatch(rcu_device* dev, int lhs_dt, const void* w, int act_dt, const void* x, const void* bias,
                             void* y, uint64_t N, uint64_t K) {
    if (N > 0x7fffffffull || K > 0x7fffffffull) return rcu_fail(dev, RCU_ERR_UNSUPPORTED, "gemv: dimension exceeds 2^31");
    DevGuard g(dev->ordinal);
    if (dt_is_q8(lhs_dt)) {
        if (K % 32 != 0) return rcu_fail(dev, RCU_ERR_INVALID_ARG, "gemv: Q8_0 rows must hold whole 32-element blocks (K=%llu)", (unsigned long long)K);
        const int8_t* qs = (const int8_t*)w;
        const void* sc = (const char*)w + align256(N * K);
        if (lhs_dt == RCU_Q8_0F && act_dt == RCU_F32) return launch_q8<float, float>(dev, qs, sc, x, bias, y, (int)N, (int)K);
        if (lhs_dt == RCU_Q8_0F && act_dt == RCU_F16) return launch_q8<float, __half>(dev, qs, sc, x, bias, y, (int)N, (int)K);
        if (lhs_dt == RCU_Q8_0H && act_dt == RCU_F16) return launch_q8<__half, __half>(dev, qs, sc, x, bias, y, (int)N, (int)K);
        return rcu_fail(dev, RCU_ERR_UNSUPPORTED, "gemv: dtype pair (%d,%d) has no kernel", lhs_dt, act_dt);
    }
    if (lhs_dt == RCU_F32 && act_dt == RCU_F32) return launch_float<float>(dev, w, x, bias, y, (int)N, (int)K);
    if (lhs_dt == RCU_F16 && act_dt == RCU_F16) return launch_float<__half>(dev, w, x, bias, y, (int)N, (int)K);
    return rcu_fail(dev, RCU_ERR_UNSUPPORTED, "gemv: dtype pair (%d,%d) has no kernel", lhs_dt, act_dt);
}
