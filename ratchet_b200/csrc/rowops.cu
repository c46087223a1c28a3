// Row-wise reductions: LayerNorm / RMSNorm / GroupNorm, Softmax and the standalone row reduce.
//
// Stand in for ratchet-core's layer_norm / rms_norm / group_norm WGSL kernels
// (ops/norm/mod.rs:112-245), softmax (ops/softmax.rs:55-180) and the reduce step both contain.
// Formulas follow the CPU device (the parity target): LayerNorm uses var = E[x^2] - E[x]^2 and
// y = (x - mu) * (1/sqrt(var + eps)) * gamma (+ beta) (cpu/norm.rs:91-147); RMSNorm
// y = x * (1/sqrt(mean(x^2) + eps)) * gamma (cpu/norm.rs:185-213).  Softmax subtracts the row
// maximum (the CPU device does not, cpu/softmax.rs:21-42; the results agree to f32 rounding and
// the maximum keeps large logits finite).
//
// Each row is read from HBM once, kept in registers, reduced with warp shuffles (plus one
// shared-memory hop across the warps of a CTA for long rows) and written once.
#include <type_traits>

#include "common.cuh"

namespace {

constexpr int kCtaThreads = 256;

struct SumOp { __device__ static float id() { return 0.f; } __device__ static float f(float a, float b) { return a + b; } };
struct MaxOp { __device__ static float id() { return -INFINITY; } __device__ static float f(float a, float b) { return fmaxf(a, b); } };

template <class Op> __device__ __forceinline__ float warp_reduce(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = Op::f(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// reduce across the CTA; every thread gets the result. `scratch` holds 32 floats.
template <class Op> __device__ __forceinline__ float cta_reduce(float v, float* scratch) {
    v = warp_reduce<Op>(v);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();  // scratch may still be read from a previous reduction
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float r = lane < (blockDim.x >> 5) ? scratch[lane] : Op::id();
    return warp_reduce<Op>(r);
}

// Reduce two values across each group of G consecutive threads (G = 32: shuffles only; G > 32: one
// shared-memory hop across the group's warps).  Every thread of the CTA must call it.
template <class Op, int G> __device__ __forceinline__ void group_reduce2(float& a, float& b, float (*scratch)[32]) {
    a = warp_reduce<Op>(a);
    b = warp_reduce<Op>(b);
    if (G > 32) {
        constexpr int WPG = G / 32;
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        __syncthreads();
        if (lane == 0) { scratch[0][warp] = a; scratch[1][warp] = b; }
        __syncthreads();
        const int first = (warp / WPG) * WPG;
        a = lane < WPG ? scratch[0][first + lane] : Op::id();
        b = lane < WPG ? scratch[1][first + lane] : Op::id();
        a = warp_reduce<Op>(a);
        b = warp_reduce<Op>(b);
    }
}

enum { MODE_LN = 0, MODE_RMS = 1, MODE_SOFTMAX = 2 };

template <class T, int V> struct alignas(sizeof(T) * V) RowVec { T v[V]; };

__device__ __forceinline__ float exp2f_fast(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Per-vector arithmetic.  The generic version computes in f32 and rounds to T after every operation.
// The f16 version does the same steps with native half2 instructions: an f16 add or multiply of two
// f16 values is the f32 operation rounded once to f16 (the f32 result is exact, or far from an f16
// rounding boundary), so the results are identical and the f32<->f16 conversions disappear.
template <class T, int V> struct RowMath {
    typedef RowVec<T, V> VT;
    __device__ static __forceinline__ void stats(const VT& x, float& s, float& s2) {
#pragma unroll
        for (int e = 0; e < V; ++e) { const float v = to_f32<T>(x.v[e]); s += v; s2 += rnd<T>(v * v); }
    }
    __device__ static __forceinline__ VT layer_norm(const VT& x, float mu, float rstd, const VT& g, const VT* b) {
        VT o;
#pragma unroll
        for (int e = 0; e < V; ++e) {
            float y = rnd<T>(rnd<T>(to_f32<T>(x.v[e]) - mu) * rstd);
            y = rnd<T>(y * to_f32<T>(g.v[e]));
            if (b) y = rnd<T>(y + to_f32<T>(b->v[e]));
            o.v[e] = from_f32<T>(y);
        }
        return o;
    }
    __device__ static __forceinline__ VT rms_norm(const VT& x, float rstd, const VT& g) {
        VT o;
#pragma unroll
        for (int e = 0; e < V; ++e) o.v[e] = from_f32<T>(rnd<T>(rnd<T>(to_f32<T>(x.v[e]) * rstd) * to_f32<T>(g.v[e])));
        return o;
    }
    __device__ static __forceinline__ void maxv(const VT& x, float& mx) {
#pragma unroll
        for (int e = 0; e < V; ++e) mx = fmaxf(mx, to_f32<T>(x.v[e]));
    }
    // x <- fp(exp(x - mx)) in place; the terms are added to `sum`
    __device__ static __forceinline__ void exp_inplace(VT& x, float mx, float& sum) {
#pragma unroll
        for (int e = 0; e < V; ++e) {
            const float d = to_f32<T>(x.v[e]) - mx;
            const float p = rnd<T>(sizeof(T) == 2 ? __expf(d) : expf(d));
            x.v[e] = from_f32<T>(p);
            sum += p;
        }
    }
    // 16-bit types multiply by the reciprocal (one unit in the last place of f32 away from the quotient,
    // which almost never changes the rounded 16-bit result); f32 divides
    __device__ static __forceinline__ VT normalise(const VT& p, float sum, float inv) {
        VT o;
#pragma unroll
        for (int e = 0; e < V; ++e) {
            const float v = to_f32<T>(p.v[e]);
            o.v[e] = from_f32<T>(sizeof(T) == 2 ? v * inv : v / sum);
        }
        return o;
    }
};

template <int V> struct RowMath<__half, V> {
    static_assert(V % 2 == 0 || V == 1, "f16 vectors hold pairs");
    typedef RowVec<__half, V> VT;
    __device__ static __forceinline__ void stats(const VT& x, float& s, float& s2) {
        if (V == 1) {
            const float v = __half2float(x.v[0]);
            s += v;
            s2 += rnd<__half>(v * v);
        } else {
#pragma unroll
            for (int e = 0; e < V / 2; ++e) {
                const __half2 h = reinterpret_cast<const __half2*>(x.v)[e];
                const float2 f = __half22float2(h), q = __half22float2(__hmul2_rn(h, h));
                s += f.x; s += f.y;
                s2 += q.x; s2 += q.y;
            }
        }
    }
    __device__ static __forceinline__ VT layer_norm(const VT& x, float mu, float rstd, const VT& g, const VT* b) {
        VT o;
        if (V == 1) {
            __half y = __hmul_rn(__hmul_rn(__hsub_rn(x.v[0], __float2half_rn(mu)), __float2half_rn(rstd)), g.v[0]);
            if (b) y = __hadd_rn(y, b->v[0]);
            o.v[0] = y;
        } else {
            const __half2 mu2 = __float2half2_rn(mu), r2 = __float2half2_rn(rstd);   // both already f16 values
#pragma unroll
            for (int e = 0; e < V / 2; ++e) {
                __half2 y = __hmul2_rn(__hmul2_rn(__hsub2_rn(reinterpret_cast<const __half2*>(x.v)[e], mu2), r2),
                                       reinterpret_cast<const __half2*>(g.v)[e]);
                if (b) y = __hadd2_rn(y, reinterpret_cast<const __half2*>(b->v)[e]);
                reinterpret_cast<__half2*>(o.v)[e] = y;
            }
        }
        return o;
    }
    __device__ static __forceinline__ VT rms_norm(const VT& x, float rstd, const VT& g) {
        VT o;
        if (V == 1) {
            o.v[0] = __hmul_rn(__hmul_rn(x.v[0], __float2half_rn(rstd)), g.v[0]);
        } else {
            const __half2 r2 = __float2half2_rn(rstd);
#pragma unroll
            for (int e = 0; e < V / 2; ++e)
                reinterpret_cast<__half2*>(o.v)[e] =
                    __hmul2_rn(__hmul2_rn(reinterpret_cast<const __half2*>(x.v)[e], r2), reinterpret_cast<const __half2*>(g.v)[e]);
        }
        return o;
    }
    // softmax steps on pairs: one conversion instruction per pair in each direction, the maximum in
    // native half2, exp in f32 (hardware exp2), the sum of the unrounded terms in f32
    __device__ static __forceinline__ void maxv(const VT& x, float& mx) {
        if (V == 1) {
            mx = fmaxf(mx, __half2float(x.v[0]));
        } else {
            __half2 m = reinterpret_cast<const __half2*>(x.v)[0];
#pragma unroll
            for (int e = 1; e < V / 2; ++e) m = __hmax2(m, reinterpret_cast<const __half2*>(x.v)[e]);
            const float2 f = __half22float2(m);
            mx = fmaxf(mx, fmaxf(f.x, f.y));
        }
    }
    __device__ static __forceinline__ void exp_inplace(VT& x, float mx, float& sum) {
        const float kLog2e = 1.4426950408889634f;
        const float bias = -mx * kLog2e;
        if (V == 1) {
            const float p = exp2f_fast(fmaf(__half2float(x.v[0]), kLog2e, bias));
            x.v[0] = __float2half_rn(p);
            sum += p;
        } else {
#pragma unroll
            for (int e = 0; e < V / 2; ++e) {
                const float2 f = __half22float2(reinterpret_cast<const __half2*>(x.v)[e]);
                const float p0 = exp2f_fast(fmaf(f.x, kLog2e, bias)), p1 = exp2f_fast(fmaf(f.y, kLog2e, bias));
                reinterpret_cast<__half2*>(x.v)[e] = __floats2half2_rn(p0, p1);
                sum += p0;
                sum += p1;
            }
        }
    }
    __device__ static __forceinline__ VT normalise(const VT& p, float, float inv) {
        VT o;
        if (V == 1) {
            o.v[0] = __float2half_rn(__half2float(p.v[0]) * inv);
        } else {
#pragma unroll
            for (int e = 0; e < V / 2; ++e) {
                const float2 f = __half22float2(reinterpret_cast<const __half2*>(p.v)[e]);
                reinterpret_cast<__half2*>(o.v)[e] = __floats2half2_rn(f.x * inv, f.y * inv);
            }
        }
        return o;
    }
};

// One row per group of G threads (a CTA holds max(256, G) / G rows).  Thread t of the group owns
// vectors t, t + G, ... (up to kPer of them, V elements each; N % V == 0).  Rows of up to 512
// vectors belong to one warp (G = 32, up to 16 vectors per lane): no block-wide barrier, so the warps
// of a CTA stream independently.  The row is read from
// HBM once with all of a thread's loads in flight together, kept in registers in its own type, and
// written once.  16-bit types round to their own precision after every operation, as the CPU device
// does.
template <class T, int MODE, int G, int V, int kPer>
__global__ void __launch_bounds__(G > kCtaThreads ? G : kCtaThreads)
row_kernel(const T* __restrict__ x, const T* __restrict__ gamma, const T* __restrict__ beta, T* __restrict__ out,
           size_t rows, int N, float eps) {
    rcu_kernel_entry();
    typedef RowVec<T, V> VT;
    typedef RowMath<T, V> Math;
    constexpr int CTA = G > kCtaThreads ? G : kCtaThreads;
    constexpr int GROUPS = CTA / G;
    __shared__ float scratch[2][32];
    const int g = threadIdx.x / G, t = threadIdx.x % G;
    const int nvec = N / V;
    for (size_t base = (size_t)blockIdx.x * GROUPS; base < rows; base += (size_t)gridDim.x * GROUPS) {
        const size_t row = base + g;
        const bool valid = row < rows;           // the loop bound is uniform across the CTA (barriers inside)
        const VT* xr = reinterpret_cast<const VT*>(x + row * (size_t)N);
        VT* orow = reinterpret_cast<VT*>(out + row * (size_t)N);
        VT raw[kPer];
#pragma unroll
        for (int i = 0; i < kPer; ++i) {
            const int j = t + i * G;
            if (valid && j < nvec) raw[i] = xr[j];
        }
        if (MODE == MODE_SOFTMAX) {
            float mx = -INFINITY, dummy = -INFINITY;
#pragma unroll
            for (int i = 0; i < kPer; ++i) {
                const int j = t + i * G;
                if (valid && j < nvec) Math::maxv(raw[i], mx);
            }
            group_reduce2<MaxOp, G>(mx, dummy, scratch);
            float sum = 0.f, zero = 0.f;
#pragma unroll
            for (int i = 0; i < kPer; ++i) {
                const int j = t + i * G;
                if (valid && j < nvec) Math::exp_inplace(raw[i], mx, sum);
            }
            group_reduce2<SumOp, G>(sum, zero, scratch);
            sum = rnd<T>(sum);
            const float inv = 1.0f / sum;
#pragma unroll
            for (int i = 0; i < kPer; ++i) {
                const int j = t + i * G;
                if (valid && j < nvec) orow[j] = Math::normalise(raw[i], sum, inv);
            }
        } else {
            float s = 0.f, s2 = 0.f;
#pragma unroll
            for (int i = 0; i < kPer; ++i) {
                const int j = t + i * G;
                if (valid && j < nvec) Math::stats(raw[i], s, s2);
            }
            const float nf = rnd<T>((float)N);
            const float e_ = rnd<T>(eps);
            group_reduce2<SumOp, G>(s, s2, scratch);
            float mu = 0.f, rstd;
            if (MODE == MODE_LN) {
                mu = rnd<T>(rnd<T>(s) / nf);
                const float ex2 = rnd<T>(rnd<T>(s2) / nf);
                const float var = rnd<T>(ex2 - rnd<T>(mu * mu));
                rstd = rnd<T>(1.0f / rnd<T>(sqrtf(rnd<T>(var + e_))));
            } else {
                const float ms = rnd<T>(rnd<T>(s2) / nf);
                rstd = rnd<T>(1.0f / rnd<T>(sqrtf(rnd<T>(ms + e_))));
            }
#pragma unroll
            for (int i = 0; i < kPer; ++i) {
                const int j = t + i * G;
                if (valid && j < nvec) {
                    const VT gm = reinterpret_cast<const VT*>(gamma)[j];
                    if (MODE == MODE_LN) {
                        VT bt;
                        if (beta) bt = reinterpret_cast<const VT*>(beta)[j];
                        orow[j] = Math::layer_norm(raw[i], mu, rstd, gm, beta ? &bt : nullptr);
                    } else {
                        orow[j] = Math::rms_norm(raw[i], rstd, gm);
                    }
                }
            }
        }
    }
}

// Rows too long for the register-resident kernels: three passes over a row that stays in L2.
template <class T, int MODE>
__global__ void __launch_bounds__(kCtaThreads)
row_kernel_long(const T* __restrict__ x, const T* __restrict__ gamma, const T* __restrict__ beta, T* __restrict__ out,
                size_t rows, int N, float eps) {
    rcu_kernel_entry();
    __shared__ float scratch[32];
    for (size_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const T* xr = x + row * (size_t)N;
        T* orow = out + row * (size_t)N;
        float s = 0.f, s2 = 0.f, mx = -INFINITY;
        for (int j = threadIdx.x; j < N; j += blockDim.x) {
            const float v = to_f32<T>(xr[j]);
            mx = fmaxf(mx, v); s += v; s2 += rnd<T>(v * v);
        }
        if (MODE == MODE_SOFTMAX) {
            mx = cta_reduce<MaxOp>(mx, scratch);
            float sum = 0.f;
            for (int j = threadIdx.x; j < N; j += blockDim.x) sum += rnd<T>(expf(to_f32<T>(xr[j]) - mx));
            sum = rnd<T>(cta_reduce<SumOp>(sum, scratch));
            for (int j = threadIdx.x; j < N; j += blockDim.x) orow[j] = from_f32<T>(rnd<T>(expf(to_f32<T>(xr[j]) - mx)) / sum);
        } else {
            const float nf = rnd<T>((float)N), e = rnd<T>(eps);
            s = cta_reduce<SumOp>(s, scratch);
            s2 = cta_reduce<SumOp>(s2, scratch);
            const float mu = MODE == MODE_LN ? rnd<T>(rnd<T>(s) / nf) : 0.f;
            const float ex2 = rnd<T>(rnd<T>(s2) / nf);
            const float var = MODE == MODE_LN ? rnd<T>(ex2 - rnd<T>(mu * mu)) : ex2;
            const float rstd = rnd<T>(1.0f / rnd<T>(sqrtf(rnd<T>(var + e))));
            for (int j = threadIdx.x; j < N; j += blockDim.x) {
                float y = rnd<T>(rnd<T>(to_f32<T>(xr[j]) - mu) * rstd);
                y = rnd<T>(y * to_f32<T>(gamma[j]));
                if (MODE == MODE_LN && beta) y = rnd<T>(y + to_f32<T>(beta[j]));
                orow[j] = from_f32<T>(y);
            }
        }
    }
}

constexpr int kMaxRowVecs = 1024 * 8;   // longest row (in vectors) the register-resident kernel takes

template <class T, int MODE, int V>
rcu_status launch_rows_v(rcu_device* dev, const T* xp, const T* gp, const T* bp, T* op, size_t rows, int N, float eps) {
    const int nvec = N / V;
    const size_t cap = (size_t)dev->sm_count * 8;
#define RCU_ROW(G, PER)                                                                                    \
    {                                                                                                      \
        constexpr int cta = G > kCtaThreads ? G : kCtaThreads;                                             \
        const size_t groups = cta / G;                                                                     \
        const int grid = (int)std::min<size_t>((rows + groups - 1) / groups, cap);                         \
        rcu_launch(dev, row_kernel<T, MODE, G, V, PER>, grid, cta, 0, xp, gp, bp, op, rows, N, eps);       \
    }
    if (nvec <= 32 * 4) RCU_ROW(32, 4)
    else if (nvec <= 32 * 8) RCU_ROW(32, 8)
    else if (nvec <= 32 * 16) RCU_ROW(32, 16)
    else if (nvec <= 128 * 8) RCU_ROW(128, 8)
    else if (nvec <= 256 * 8) RCU_ROW(256, 8)
    else if (nvec <= 1024 * 4) RCU_ROW(1024, 4)
    else RCU_ROW(1024, 8)
#undef RCU_ROW
    RCU_LAUNCH_CHECK(dev);
    return RCU_OK;
}

template <class T, int MODE>
rcu_status launch_rows(rcu_device* dev, const void* x, const void* gamma, const void* beta, void* out, size_t rows, int N, float eps) {
    const T* xp = (const T*)x; const T* gp = (const T*)gamma; const T* bp = (const T*)beta; T* op = (T*)out;
    constexpr int VFULL = 16 / sizeof(T), VHALF = 8 / sizeof(T);
    const uintptr_t ptr_bits = reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out) |
                               reinterpret_cast<uintptr_t>(gamma) | reinterpret_cast<uintptr_t>(beta);
    auto fits = [&](int v) { return N % v == 0 && (ptr_bits & ((uintptr_t)v * sizeof(T) - 1)) == 0 && N / v <= kMaxRowVecs; };
    constexpr bool kVector = !std::is_same<T, __nv_bfloat16>::value;   // bf16 activations are rare: scalar path only
    if (kVector && fits(VFULL)) return launch_rows_v<T, MODE, kVector ? VFULL : 1>(dev, xp, gp, bp, op, rows, N, eps);
    if (kVector && fits(VHALF)) return launch_rows_v<T, MODE, kVector ? VHALF : 1>(dev, xp, gp, bp, op, rows, N, eps);
    if (fits(1)) return launch_rows_v<T, MODE, 1>(dev, xp, gp, bp, op, rows, N, eps);
    const int grid = (int)std::min<size_t>(rows, (size_t)dev->sm_count * 8);
    rcu_launch(dev, row_kernel_long<T, MODE>, grid, kCtaThreads, 0, xp, gp, bp, op, rows, N, eps);
    RCU_LAUNCH_CHECK(dev);
    return RCU_OK;
}

template <int MODE>
rcu_status dispatch_rows(rcu_device* dev, int dt, const void* x, const void* gamma, const void* beta, void* out, size_t rows, int N, float eps) {
    switch (dt) {
        case RCU_F32: return launch_rows<float, MODE>(dev, x, gamma, beta, out, rows, N, eps);
        case RCU_F16: return launch_rows<__half, MODE>(dev, x, gamma, beta, out, rows, N, eps);
        case RCU_BF16: return launch_rows<__nv_bfloat16, MODE>(dev, x, gamma, beta, out, rows, N, eps);
    }
    return rcu_fail(dev, RCU_ERR_UNSUPPORTED, "row op: dtype %d", dt);
}

// GroupNorm (ops/norm/groupnorm.rs): x [B,C,L]; statistics over each group of C/groups channels
// times L positions; y = (x - mu) * rsqrt(var + eps) * gamma[c] + beta[c].
template <class T>
__global__ void __launch_bounds__(kCtaThreads)
group_norm_kernel(const T* __restrict__ x, const T* __restrict__ gamma, const T* __restrict__ beta, T* __restrict__ out,
                  int C, int L, int groups, float eps) {
    rcu_kernel_entry();
    __shared__ float scratch[32];
    const int cpg = C / groups;
    const size_t base = (size_t)blockIdx.x * cpg * L;   // blockIdx.x = b * groups + g
    const int g = blockIdx.x % groups;
    const size_t n = (size_t)cpg * L;
    float s = 0.f, s2 = 0.f;
    for (size_t i = threadIdx.x; i < n; i += blockDim.x) { const float v = to_f32<T>(x[base + i]); s += v; s2 += v * v; }
    s = cta_reduce<SumOp>(s, scratch);
    s2 = cta_reduce<SumOp>(s2, scratch);
    const float mu = s / (float)n;
    const float var = s2 / (float)n - mu * mu;
    const float rstd = rsqrtf(var + eps);
    for (size_t i = threadIdx.x; i < n; i += blockDim.x) {
        const int c = g * cpg + (int)(i / L);
        float y = (to_f32<T>(x[base + i]) - mu) * rstd * to_f32<T>(gamma[c]);
        if (beta) y += to_f32<T>(beta[c]);
        out[base + i] = from_f32<T>(y);
    }
}

// Warp per row; V elements per load (N % V == 0), four loads in flight per lane.
template <class T, int KIND, int V>
__global__ void __launch_bounds__(256) reduce_rows_kernel(const T* __restrict__ x, T* __restrict__ out, size_t rows, int N) {
    rcu_kernel_entry();
    typedef RowVec<T, V> VT;
    const int lane = threadIdx.x & 31;
    const size_t wpc = blockDim.x >> 5;
    const int nvec = N / V;
    for (size_t row = (size_t)blockIdx.x * wpc + (threadIdx.x >> 5); row < rows; row += (size_t)gridDim.x * wpc) {
        const VT* xr = reinterpret_cast<const VT*>(x + row * (size_t)N);
        float acc = KIND == RCU_REDUCE_MAX ? -INFINITY : 0.f;
        for (int j0 = 0; j0 < nvec; j0 += 128) {
            VT raw[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int j = j0 + u * 32 + lane;
                if (j < nvec) raw[u] = xr[j];
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int j = j0 + u * 32 + lane;
                if (j < nvec) {
#pragma unroll
                    for (int e = 0; e < V; ++e) {
                        const float v = to_f32<T>(raw[u].v[e]);
                        acc = KIND == RCU_REDUCE_MAX ? fmaxf(acc, v) : acc + v;
                    }
                }
            }
        }
        acc = KIND == RCU_REDUCE_MAX ? warp_reduce<MaxOp>(acc) : warp_reduce<SumOp>(acc);
        if (KIND == RCU_REDUCE_MEAN) acc = rnd<T>(acc) / rnd<T>((float)N);   // cpu/norm.rs:72-89
        if (lane == 0) out[row] = from_f32<T>(acc);
    }
}

}  // namespace

extern "C" {

rcu_status rcu_norm(rcu_device* dev, int kind, const rcu_tensor* x, const rcu_tensor* scale, const rcu_tensor* bias, float eps,
                    uint32_t groups, rcu_tensor* dst) {
    if (!dev) return RCU_ERR_INVALID_ARG;
    RCU_REQUIRE(dev, t_valid(x) && t_valid(scale) && t_valid(dst), "norm: invalid tensor descriptor");
    RCU_REQUIRE(dev, x->dt == scale->dt, "norm: DTypeMismatch expected %d, actual %d (scale)", x->dt, scale->dt);  // cpu/norm.rs:35-41
    RCU_REQUIRE(dev, !bias || bias->dt == x->dt, "norm: DTypeMismatch (bias)");
    RCU_REQUIRE(dev, dst->dt == x->dt && t_numel(dst) == t_numel(x), "norm: dst must match x");
    DevGuard g(dev->ordinal);
    const uint64_t N = x->shape[x->rank - 1];
    if (kind == RCU_GROUP_NORM) {
        RCU_REQUIRE(dev, x->rank == 3 && groups > 0 && x->shape[1] % groups == 0, "group_norm: x must be [B,C,L] with C %% groups == 0");
        RCU_REQUIRE(dev, t_numel(scale) == x->shape[1] && (!bias || t_numel(bias) == x->shape[1]), "group_norm: scale/bias must have C elements");
        const int grid = (int)(x->shape[0] * groups);
        const void* bp = bias ? bias->data : nullptr;
        switch (x->dt) {
            case RCU_F32: rcu_launch(dev, group_norm_kernel<float>, grid, kCtaThreads, 0, (const float*)x->data, (const float*)scale->data, (const float*)bp, (float*)dst->data, (int)x->shape[1], (int)x->shape[2], (int)groups, eps); break;
            case RCU_F16: rcu_launch(dev, group_norm_kernel<__half>, grid, kCtaThreads, 0, (const __half*)x->data, (const __half*)scale->data, (const __half*)bp, (__half*)dst->data, (int)x->shape[1], (int)x->shape[2], (int)groups, eps); break;
            default: return rcu_fail(dev, RCU_ERR_UNSUPPORTED, "group_norm: dtype %d", x->dt);
        }
        RCU_LAUNCH_CHECK(dev);
        return RCU_OK;
    }
    RCU_REQUIRE(dev, kind == RCU_LAYER_NORM || kind == RCU_RMS_NORM, "norm: unknown kind %d", kind);
    RCU_REQUIRE(dev, t_numel(scale) == N && (!bias || t_numel(bias) == N), "norm: scale/bias must have %llu elements", (unsigned long long)N);
    RCU_REQUIRE(dev, N <= 0x7fffffffull && N > 0, "norm: bad row length");
    const size_t rows = t_numel(x) / N;
    const void* bp = (bias && kind == RCU_LAYER_NORM) ? bias->data : nullptr;
    if (kind == RCU_LAYER_NORM) return dispatch_rows<MODE_LN>(dev, x->dt, x->data, scale->data, bp, dst->data, rows, (int)N, eps);
    return dispatch_rows<MODE_RMS>(dev, x->dt, x->data, scale->data, nullptr, dst->data, rows, (int)N, eps);
}

rcu_status rcu_softmax(rcu_device* dev, const rcu_tensor* x, uint32_t dim, rcu_tensor* dst) {
    if (!dev) return RCU_ERR_INVALID_ARG;
    RCU_REQUIRE(dev, t_valid(x) && t_valid(dst), "softmax: invalid tensor descriptor");
    RCU_REQUIRE(dev, dim == x->rank - 1, "softmax: only the last dimension is supported (dim=%u, rank=%u)", dim, x->rank);
    RCU_REQUIRE(dev, dst->dt == x->dt && t_numel(dst) == t_numel(x), "softmax: dst must match x");
    DevGuard g(dev->ordinal);
    const uint64_t N = x->shape[dim];
    RCU_REQUIRE(dev, N <= 0x7fffffffull && N > 0, "softmax: bad row length");
    return dispatch_rows<MODE_SOFTMAX>(dev, x->dt, x->data, nullptr, nullptr, dst->data, t_numel(x) / N, (int)N, 0.f);
}

rcu_status rcu_reduce(rcu_device* dev, int kind, const rcu_tensor* x, rcu_tensor* dst) {
    if (!dev) return RCU_ERR_INVALID_ARG;
    RCU_REQUIRE(dev, t_valid(x) && t_valid(dst), "reduce: invalid tensor descriptor");
    const uint64_t N = x->shape[x->rank - 1];
    const size_t rows = t_numel(x) / N;
    RCU_REQUIRE(dev, dst->dt == x->dt && t_numel(dst) == rows, "reduce: dst must hold one element per row");
    RCU_REQUIRE(dev, kind >= RCU_REDUCE_SUM && kind <= RCU_REDUCE_MEAN, "reduce: unknown kind %d", kind);
    DevGuard g(dev->ordinal);
    const int grid = (int)std::min<size_t>((rows + 7) / 8, (size_t)dev->sm_count * 8);
    const bool vec = N % 8 == 0 && (reinterpret_cast<uintptr_t>(x->data) & 15) == 0;   // 16-byte loads for 2- and 4-byte types
#define RCU_RED(T, K)                                                                                                        \
    if (vec) rcu_launch(dev, reduce_rows_kernel<T, K, 16 / sizeof(T)>, grid, 256, 0, (const T*)x->data, (T*)dst->data, rows, (int)N); \
    else rcu_launch(dev, reduce_rows_kernel<T, K, 1>, grid, 256, 0, (const T*)x->data, (T*)dst->data, rows, (int)N)
#define RCU_RED_T(T)                                       \
    switch (kind) {                                        \
        case RCU_REDUCE_SUM: RCU_RED(T, RCU_REDUCE_SUM); break; \
        case RCU_REDUCE_MAX: RCU_RED(T, RCU_REDUCE_MAX); break; \
        default: RCU_RED(T, RCU_REDUCE_MEAN); break;       \
    }
    switch (x->dt) {
        case RCU_F32: RCU_RED_T(float) break;
        case RCU_F16: RCU_RED_T(__half) break;
        case RCU_BF16: RCU_RED_T(__nv_bfloat16) break;
        default: return rcu_fail(dev, RCU_ERR_UNSUPPORTED, "reduce: dtype %d", x->dt);
    }
#undef RCU_RED_T
#undef RCU_RED
    RCU_LAUNCH_CHECK(dev);
    return RCU_OK;
}

}  // extern "C"
