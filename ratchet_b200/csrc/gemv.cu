// Decode GEMV entry: y[N] = W[N,K] . x[K] (+ bias) for Q8_0 weights (kernel template in gemv_q8.cuh)
// and for plain f16 / f32 weights (kernel below).
//
// Takes the place of ratchet-core's subgroup_gemv / workgroup_gemv WGSL kernels
// (ops/matmul/subgroup_gemv.rs:89-309, ops/matmul/workgroup_gemv.rs:221-371) for the case
// Matmul::select_kernel (ops/matmul/mod.rs:716-748) routes to them: rhs is a vector and lhs is not
// transposed.
#include "ring.cuh"

namespace {

using gemvq8::kThreads;
using gemvq8::kWarps;

// Plain f16 / f32 weights: same work layout, 16 bytes (8 halves / 4 floats) per lane per step.
template <class T, int ROWS, int KSPLIT, int UNROLL>
__global__ void __launch_bounds__(kThreads)
gemv_float_kernel(const T* __restrict__ Wm, const T* __restrict__ x, const T* __restrict__ bias, T* __restrict__ y,
                  int N, int K) {
    rcu_kernel_entry();
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

GemvPlan plan_gemv(const rcu_device* dev, int N, int K, int rows_per_warp, int ctas_per_sm) {
    const gemvq8::Plan p = gemvq8::plan(dev, N, 4 / rows_per_warp == 0 ? 1 : 1, K, ctas_per_sm);
    return GemvPlan{p.ksplit, p.grid};
}

template <class ScaleT, class ActT>
rcu_status launch_q8(rcu_device* dev, const int8_t* qs, const void* scales, const void* x, const void* bias, void* y, int N, int K) {
    gemvq8::PlainPrologue<ActT> pro{(const ActT*)x};
    gemvq8::PlainEpilogue<ActT> epi{(const ActT*)bias, (ActT*)y};
    if constexpr (sizeof(ActT) == 2) {
        // f16 activations, rows of whole 256-element runs: the weight stream goes through the shared-memory rings
        // (long streams only: a launch that streams a few MB ends before a ring of 200 KB per SM has paid for its start)
        if (K >= 2048 && (size_t)N * K >= ((size_t)96 << 20)) {
            ringq8::PlainPlanes<ringq8::VecSource> rpro{{(const __half*)x}};
            const rcu_status st = ringq8::launch<ScaleT>(dev, qs, scales, rpro, epi, N, K, dev->const_weights);
            if (st != RCU_ERR_UNSUPPORTED) return st;
        }
    }
    const int ctas = 3;
    // short streams (tens of MB) gain from the pre-loaded, double-buffered variant; long ones from occupancy
    const bool pipe = (size_t)N * K < (size_t)128 << 20;
    // Programmatic dependent launch only on the caller's word (rcu_set_constant_weights): the kernels read weights
    // before they wait for their predecessor, and through this entry point the predecessor may have produced them.
    const bool overlap = dev->const_weights;
    // f16 activations: dp4a on 16-bit fixed-point planes with 16-element scales (the conversions of an f16
    // fma path saturate the XU pipe: 4.4 TB/s against 6.6); f32 activations: exact int8 -> f32 and FFMA.
    constexpr int MODE = sizeof(ActT) == 2 ? 2 : 1;
    return gemvq8::launch<ScaleT, ActT, MODE>(dev, qs, scales, pro, epi, N, K, overlap, ctas, pipe);
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
        rcu_launch(dev, kern, p.grid, kThreads, smem, (const T*)Wm, (const T*)x, (const T*)bias, (T*)y, N, K); \
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
