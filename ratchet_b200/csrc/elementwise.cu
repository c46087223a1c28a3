// Binary / Unary / Cast elementwise kernels.
//
// Stand in for ratchet-core's add/sub/mul/div (ops/binary.rs:71-113), the 14 unary functions
// (ops/unary.rs:91-227) and cast (ops/cast.rs:56-99).  Arithmetic follows the CPU device, which is
// the parity target: cpu/binary.rs:78-119, cpu/unary.rs:46-66 (gelu without the tanh clamp; silu
// and sigmoid as x/(1+exp(-x)), 1/(1+exp(-x))), cpu/mod.rs:127-156 (f32<->i32/u32 casts are bit
// reinterpretations).  16-bit types compute every operation in f32 and round to nearest even after
// each one, which is what the `half` crate does on the CPU.
//
// All kernels are HBM-bound: 128-bit loads and stores, grid-stride over 16-byte vectors, grid sized
// as a multiple of the SM count.  The Binary kernel folds the broadcast the reference materialises
// beforehand (tensor.rs:252-278) into its index arithmetic (stride 0 on broadcast dimensions).
#include "common.cuh"

namespace {

template <class T, int V> struct alignas(sizeof(T) * V) Vec { T v[V]; };

template <class T> __device__ __forceinline__ float binary_apply(int op, float x, float y) {
    switch (op) {
        case RCU_ADD: return x + y;
        case RCU_SUB: return x - y;
        case RCU_MUL: return x * y;
        default: return x / y;
    }
}

__device__ __forceinline__ float exp2f_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// exp and division for the 16-bit types: the hardware approximations (2^-21 relative) round to the
// same 16-bit value as the exact functions in all but a few cases per thousand, and those differ by
// one unit in the last place; f32 keeps the accurate functions.
template <class T> __device__ __forceinline__ float ew_exp(float x) { return sizeof(T) == 2 ? __expf(x) : expf(x); }
template <class T> __device__ __forceinline__ float ew_div(float x, float y) { return sizeof(T) == 2 ? __fdividef(x, y) : x / y; }
template <class T> __device__ __forceinline__ float ew_tanh(float a) {
    if (sizeof(T) != 2) return tanhf(a);
    // 1 - 2 / (1 + e^(2a)): absolute error ~3e-7, saturates to +-1, propagates NaN
    const float e = exp2f_approx(a * 2.8853900817779268f);
    return 1.0f - __fdividef(2.0f, 1.0f + e);
}

template <class T, int OP> __device__ __forceinline__ float unary_apply(float x) {
    switch (OP) {
        case RCU_GELU: {
            const float c05 = rnd<T>(0.5f), c1 = 1.0f, ck = rnd<T>(0.7978846f), cc = rnd<T>(0.044715f);
            const float inner = rnd<T>(c1 + rnd<T>(rnd<T>(cc * x) * x));
            const float arg = rnd<T>(rnd<T>(ck * x) * inner);
            return rnd<T>(rnd<T>(c05 * x) * rnd<T>(c1 + rnd<T>(ew_tanh<T>(arg))));
        }
        case RCU_TANH: return tanhf(x);
        case RCU_EXP: return expf(x);
        case RCU_LOG: return logf(x);
        case RCU_SIN: return sinf(x);
        case RCU_COS: return cosf(x);
        case RCU_ABS: return fabsf(x);
        case RCU_SQRT: return sqrtf(x);
        case RCU_RELU: return fmaxf(x, 0.f);
        case RCU_FLOOR: return floorf(x);
        case RCU_CEIL: return ceilf(x);
        case RCU_NEG: return -x;
        case RCU_SILU: return ew_div<T>(x, rnd<T>(1.0f + rnd<T>(ew_exp<T>(-x))));
        default: return ew_div<T>(1.0f, rnd<T>(1.0f + rnd<T>(ew_exp<T>(-x))));  // sigmoid
    }
}

// GELU on f16 pairs with native half2 arithmetic.  An f16 add or multiply of two f16 values is the
// f32 operation rounded once to f16 (the f32 result is exact or far from an f16 midpoint), so each
// step equals the "compute in f32, round to f16" step of the scalar formula above.
__device__ __forceinline__ __half2 gelu_h2(__half2 x) {
    const __half2 c05 = __float2half2_rn(0.5f), c1 = __float2half2_rn(1.0f), ck = __float2half2_rn(0.7978846f),
                  cc = __float2half2_rn(0.044715f);
    const __half2 inner = __hadd2_rn(c1, __hmul2_rn(__hmul2_rn(cc, x), x));
    const float2 arg = __half22float2(__hmul2_rn(__hmul2_rn(ck, x), inner));
    const __half2 t = __floats2half2_rn(ew_tanh<__half>(arg.x), ew_tanh<__half>(arg.y));
    return __hmul2_rn(__hmul2_rn(c05, x), __hadd2_rn(c1, t));
}

// ---------------------------------------------------------------------------------- same-shape binary
// Two 16-byte vectors per operand are in flight per thread before the first is used.
template <class T, int V>
__global__ void __launch_bounds__(256) binary_same_kernel(int op, const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out, size_t n) {
    rcu_kernel_entry();
    typedef Vec<T, V> VT;
    const size_t nvec = n / V;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (; i + stride < nvec; i += 2 * stride) {
        const VT a0 = reinterpret_cast<const VT*>(a)[i], b0 = reinterpret_cast<const VT*>(b)[i];
        const VT a1 = reinterpret_cast<const VT*>(a)[i + stride], b1 = reinterpret_cast<const VT*>(b)[i + stride];
        VT o0, o1;
#pragma unroll
        for (int j = 0; j < V; ++j) {
            o0.v[j] = from_f32<T>(binary_apply<T>(op, to_f32<T>(a0.v[j]), to_f32<T>(b0.v[j])));
            o1.v[j] = from_f32<T>(binary_apply<T>(op, to_f32<T>(a1.v[j]), to_f32<T>(b1.v[j])));
        }
        reinterpret_cast<VT*>(out)[i] = o0;
        reinterpret_cast<VT*>(out)[i + stride] = o1;
    }
    if (i < nvec) {
        const VT va = reinterpret_cast<const VT*>(a)[i], vb = reinterpret_cast<const VT*>(b)[i];
        VT vo;
#pragma unroll
        for (int j = 0; j < V; ++j) vo.v[j] = from_f32<T>(binary_apply<T>(op, to_f32<T>(va.v[j]), to_f32<T>(vb.v[j])));
        reinterpret_cast<VT*>(out)[i] = vo;
    }
    if (blockIdx.x == 0) {
        const size_t t = nvec * V + threadIdx.x;
        if (threadIdx.x < (unsigned)V && t < n) out[t] = from_f32<T>(binary_apply<T>(op, to_f32<T>(a[t]), to_f32<T>(b[t])));
    }
}

// ---------------------------------------------------------------------------------- broadcasting binary
struct Bcast4 {
    uint32_t d[4];      // dst shape (4-D promoted)
    uint32_t sa[4];     // element strides of a (0 on broadcast dims)
    uint32_t sb[4];
};

// Each thread produces V consecutive elements of the innermost axis (d[3] % V == 0).  An operand
// whose innermost stride is 1 is read as one vector, one whose innermost stride is 0 is read once
// and repeated.  I is the index type: 32-bit division whenever the vector count allows it.
template <class T, int V, class I>
__global__ void __launch_bounds__(256) binary_bcast_kernel(int op, const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out, size_t nvec, Bcast4 p) {
    rcu_kernel_entry();
    typedef Vec<T, V> VT;
    const I row_units = (I)(p.d[3] / V);
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < nvec; idx += stride) {
        I r = (I)idx;
        const uint32_t i3 = (uint32_t)(r % row_units) * V; r /= row_units;
        const uint32_t i2 = (uint32_t)(r % p.d[2]); r /= p.d[2];
        const uint32_t i1 = (uint32_t)(r % p.d[1]); r /= p.d[1];
        const uint32_t i0 = (uint32_t)r;
        const size_t oa = (size_t)i0 * p.sa[0] + (size_t)i1 * p.sa[1] + (size_t)i2 * p.sa[2] + (size_t)i3 * p.sa[3];
        const size_t ob = (size_t)i0 * p.sb[0] + (size_t)i1 * p.sb[1] + (size_t)i2 * p.sb[2] + (size_t)i3 * p.sb[3];
        VT va, vb, vo;
        if (p.sa[3]) va = *reinterpret_cast<const VT*>(a + oa);
        else {
            const T s = a[oa];
#pragma unroll
            for (int j = 0; j < V; ++j) va.v[j] = s;
        }
        if (p.sb[3]) vb = *reinterpret_cast<const VT*>(b + ob);
        else {
            const T s = b[ob];
#pragma unroll
            for (int j = 0; j < V; ++j) vb.v[j] = s;
        }
#pragma unroll
        for (int j = 0; j < V; ++j) vo.v[j] = from_f32<T>(binary_apply<T>(op, to_f32<T>(va.v[j]), to_f32<T>(vb.v[j])));
        reinterpret_cast<VT*>(out)[idx] = vo;
    }
}

// ---------------------------------------------------------------------------------- unary / cast
template <class T, int V, int OP> __device__ __forceinline__ Vec<T, V> unary_vec(const Vec<T, V>& vx) {
    Vec<T, V> vo;
#pragma unroll
    for (int j = 0; j < V; ++j) vo.v[j] = from_f32<T>(unary_apply<T, OP>(to_f32<T>(vx.v[j])));
    return vo;
}
template <> __device__ __forceinline__ Vec<__half, 8> unary_vec<__half, 8, RCU_GELU>(const Vec<__half, 8>& vx) {
    Vec<__half, 8> vo;
#pragma unroll
    for (int j = 0; j < 4; ++j)
        reinterpret_cast<__half2*>(vo.v)[j] = gelu_h2(reinterpret_cast<const __half2*>(vx.v)[j]);
    return vo;
}

template <class T, int V, int OP>
__global__ void __launch_bounds__(256) unary_kernel(const T* __restrict__ x, T* __restrict__ out, size_t n) {
    rcu_kernel_entry();
    typedef Vec<T, V> VT;
    const size_t nvec = n / V;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (; i + stride < nvec; i += 2 * stride) {
        const VT x0 = reinterpret_cast<const VT*>(x)[i];
        const VT x1 = reinterpret_cast<const VT*>(x)[i + stride];
        reinterpret_cast<VT*>(out)[i] = unary_vec<T, V, OP>(x0);
        reinterpret_cast<VT*>(out)[i + stride] = unary_vec<T, V, OP>(x1);
    }
    if (i < nvec) reinterpret_cast<VT*>(out)[i] = unary_vec<T, V, OP>(reinterpret_cast<const VT*>(x)[i]);
    if (blockIdx.x == 0) {
        const size_t t = nvec * V + threadIdx.x;
        if (threadIdx.x < (unsigned)V && t < n) out[t] = from_f32<T>(unary_apply<T, OP>(to_f32<T>(x[t])));
    }
}

template <class S, class D, int V>
__global__ void __launch_bounds__(256) cast_kernel(const S* __restrict__ x, D* __restrict__ out, size_t n) {
    rcu_kernel_entry();
    const size_t nvec = n / V;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (; i + stride < nvec; i += 2 * stride) {
        const Vec<S, V> x0 = reinterpret_cast<const Vec<S, V>*>(x)[i];
        const Vec<S, V> x1 = reinterpret_cast<const Vec<S, V>*>(x)[i + stride];
        Vec<D, V> o0, o1;
#pragma unroll
        for (int j = 0; j < V; ++j) { o0.v[j] = from_f32<D>(to_f32<S>(x0.v[j])); o1.v[j] = from_f32<D>(to_f32<S>(x1.v[j])); }
        reinterpret_cast<Vec<D, V>*>(out)[i] = o0;
        reinterpret_cast<Vec<D, V>*>(out)[i + stride] = o1;
    }
    if (i < nvec) {
        const Vec<S, V> vx = reinterpret_cast<const Vec<S, V>*>(x)[i];
        Vec<D, V> vo;
#pragma unroll
        for (int j = 0; j < V; ++j) vo.v[j] = from_f32<D>(to_f32<S>(vx.v[j]));
        reinterpret_cast<Vec<D, V>*>(out)[i] = vo;
    }
    if (blockIdx.x == 0) {
        const size_t t = nvec * V + threadIdx.x;
        if (threadIdx.x < (unsigned)V && t < n) out[t] = from_f32<D>(to_f32<S>(x[t]));
    }
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

inline int ew_grid(const rcu_device* dev, size_t work) {
    // up to 8 CTAs of 256 threads per SM, always a multiple of the SM count once the work is large
    const size_t blocks = (work + 255) / 256;
    const size_t cap = (size_t)dev->sm_count * 8;
    return (int)(blocks < 1 ? 1 : (blocks < cap ? blocks : cap));
}

template <class T>
rcu_status launch_binary_same(rcu_device* dev, int op, const void* a, const void* b, void* out, size_t n) {
    constexpr int V = 16 / sizeof(T);
    if (aligned16(a) && aligned16(b) && aligned16(out)) {
        rcu_launch(dev, binary_same_kernel<T, V>, ew_grid(dev, n / V / 2 + 1), 256, 0, op, (const T*)a, (const T*)b, (T*)out, n);
    } else {
        rcu_launch(dev, binary_same_kernel<T, 1>, ew_grid(dev, n / 2 + 1), 256, 0, op, (const T*)a, (const T*)b, (T*)out, n);
    }
    RCU_LAUNCH_CHECK(dev);
    return RCU_OK;
}

template <class T, int OP>
rcu_status launch_unary_op(rcu_device* dev, const void* x, void* out, size_t n) {
    constexpr int V = 16 / sizeof(T);
    if (aligned16(x) && aligned16(out)) {
        rcu_launch(dev, unary_kernel<T, V, OP>, ew_grid(dev, n / V / 2 + 1), 256, 0, (const T*)x, (T*)out, n);
    } else {
        rcu_launch(dev, unary_kernel<T, 1, OP>, ew_grid(dev, n / 2 + 1), 256, 0, (const T*)x, (T*)out, n);
    }
    RCU_LAUNCH_CHECK(dev);
    return RCU_OK;
}

template <class T>
rcu_status launch_unary(rcu_device* dev, int op, const void* x, void* out, size_t n) {
    switch (op) {
#define RCU_UNARY_CASE(OP) case OP: return launch_unary_op<T, OP>(dev, x, out, n)
        RCU_UNARY_CASE(RCU_GELU); RCU_UNARY_CASE(RCU_TANH); RCU_UNARY_CASE(RCU_EXP); RCU_UNARY_CASE(RCU_LOG);
        RCU_UNARY_CASE(RCU_SIN); RCU_UNARY_CASE(RCU_COS); RCU_UNARY_CASE(RCU_ABS); RCU_UNARY_CASE(RCU_SQRT);
        RCU_UNARY_CASE(RCU_RELU); RCU_UNARY_CASE(RCU_FLOOR); RCU_UNARY_CASE(RCU_CEIL); RCU_UNARY_CASE(RCU_NEG);
        RCU_UNARY_CASE(RCU_SILU);
#undef RCU_UNARY_CASE
        default: return launch_unary_op<T, RCU_SIGMOID>(dev, x, out, n);
    }
}

template <class S, class D>
rcu_status launch_cast(rcu_device* dev, const void* x, void* out, size_t n) {
    constexpr int V = 4;  // 16-byte vectors on the 4-byte side, 8-byte on the 2-byte side
    const bool ok = (reinterpret_cast<uintptr_t>(x) % (sizeof(S) * V) == 0) && (reinterpret_cast<uintptr_t>(out) % (sizeof(D) * V) == 0);
    if (ok) rcu_launch(dev, cast_kernel<S, D, V>, ew_grid(dev, n / V / 2 + 1), 256, 0, (const S*)x, (D*)out, n);
    else rcu_launch(dev, cast_kernel<S, D, 1>, ew_grid(dev, n / 2 + 1), 256, 0, (const S*)x, (D*)out, n);
    RCU_LAUNCH_CHECK(dev);
    return RCU_OK;
}

// Widest vector (in elements) the broadcast kernel can use: it must divide the innermost extent, every
// pointer must be aligned to it, and an operand read as vectors must have vector-aligned outer strides.
template <class T>
void launch_binary_bcast(rcu_device* dev, int op, const void* a, const void* b, void* out, size_t n, const Bcast4& p) {
    auto fits = [&](int v) {
        const uintptr_t mask = (uintptr_t)v * sizeof(T) - 1;
        if (p.d[3] % v) return false;
        if (reinterpret_cast<uintptr_t>(out) & mask) return false;
        const void* ptr[2] = {a, b};
        const uint32_t* st[2] = {p.sa, p.sb};
        for (int k = 0; k < 2; ++k) {
            if (!st[k][3]) continue;   // read as a scalar and repeated
            if (reinterpret_cast<uintptr_t>(ptr[k]) & mask) return false;
            for (int i = 0; i < 3; ++i)
                if (st[k][i] % v) return false;
        }
        return true;
    };
    constexpr int VMAX = 16 / sizeof(T);
    int v = VMAX;
    while (v > 1 && !fits(v)) v >>= 1;
    const size_t nvec = n / v;
    const bool narrow = nvec <= 0xffffffffull;
    const int grid = ew_grid(dev, nvec);
#define RCU_BCAST(VV)                                                                                                         \
    if (narrow) rcu_launch(dev, binary_bcast_kernel<T, VV, uint32_t>, grid, 256, 0, op, (const T*)a, (const T*)b, (T*)out, nvec, p); \
    else rcu_launch(dev, binary_bcast_kernel<T, VV, uint64_t>, grid, 256, 0, op, (const T*)a, (const T*)b, (T*)out, nvec, p)
    if (v == VMAX) { RCU_BCAST(VMAX); }
    else if (v >= 2 && VMAX >= 4 && v == VMAX / 2) { RCU_BCAST((VMAX >= 4 ? VMAX / 2 : 1)); }
    else if (v >= 2) { RCU_BCAST(2); }
    else { RCU_BCAST(1); }
#undef RCU_BCAST
}

// numpy-style broadcast of `src` to the 4-D promoted `dst` shape: stride 0 where src has size 1.
bool bcast_strides(const rcu_tensor* src, const uint64_t d4[4], uint32_t out[4]) {
    uint64_t s4[4];
    t_promote4(src, s4);
    uint64_t acc = 1;
    for (int i = 3; i >= 0; --i) {
        if (s4[i] == d4[i]) out[i] = (uint32_t)acc;
        else if (s4[i] == 1) out[i] = 0;
        else return false;
        if (s4[i] == 1) out[i] = 0;
        acc *= s4[i];
    }
    return true;
}

}  // namespace

extern "C" {

rcu_status rcu_binary(rcu_device* dev, int op, const rcu_tensor* a, const rcu_tensor* b, rcu_tensor* dst) {
    if (!dev) return RCU_ERR_INVALID_ARG;
    RCU_REQUIRE(dev, t_valid(a) && t_valid(b) && t_valid(dst), "binary: invalid tensor descriptor");
    RCU_REQUIRE(dev, op >= RCU_ADD && op <= RCU_DIV, "binary: unknown op %d", op);
    RCU_REQUIRE(dev, a->dt == b->dt && a->dt == dst->dt, "binary: dtype mismatch (%d, %d -> %d)", a->dt, b->dt, dst->dt);
    if (!dt_is_float(a->dt)) return rcu_fail(dev, RCU_ERR_UNSUPPORTED, "binary: dtype %d", a->dt);
    DevGuard g(dev->ordinal);
    const size_t n = t_numel(dst);
    if (n == 0) return RCU_OK;
    if (t_same_shape(a, b) && t_numel(a) == n) {
        switch (a->dt) {
            case RCU_F32: return launch_binary_same<float>(dev, op, a->data, b->data, dst->data, n);
            case RCU_F16: return launch_binary_same<__half>(dev, op, a->data, b->data, dst->data, n);
            default: return launch_binary_same<__nv_bfloat16>(dev, op, a->data, b->data, dst->data, n);
        }
    }
    // broadcasting: dst shape must be the numpy broadcast of a and b (Shape::multi_broadcast, shape.rs:118-136)
    Bcast4 p;
    uint64_t d4[4];
    t_promote4(dst, d4);
    for (int i = 0; i < 4; ++i) {
        RCU_REQUIRE(dev, d4[i] <= 0xffffffffull, "binary: dimension too large");
        p.d[i] = (uint32_t)d4[i];
    }
    if (!bcast_strides(a, d4, p.sa) || !bcast_strides(b, d4, p.sb))
        return rcu_fail(dev, RCU_ERR_INVALID_ARG, "binary: operands do not broadcast to dst's shape");
    RCU_REQUIRE(dev, dst->data != a->data || t_numel(a) == n, "binary: in-place needs a to have dst's shape");
    switch (a->dt) {
        case RCU_F32: launch_binary_bcast<float>(dev, op, a->data, b->data, dst->data, n, p); break;
        case RCU_F16: launch_binary_bcast<__half>(dev, op, a->data, b->data, dst->data, n, p); break;
        default: launch_binary_bcast<__nv_bfloat16>(dev, op, a->data, b->data, dst->data, n, p); break;
    }
    RCU_LAUNCH_CHECK(dev);
    return RCU_OK;
}

rcu_status rcu_unary(rcu_device* dev, int op, const rcu_tensor* x, rcu_tensor* dst) {
    if (!dev) return RCU_ERR_INVALID_ARG;
    RCU_REQUIRE(dev, t_valid(x) && t_valid(dst), "unary: invalid tensor descriptor");
    RCU_REQUIRE(dev, op >= RCU_GELU && op <= RCU_SIGMOID, "unary: unknown op %d", op);
    RCU_REQUIRE(dev, x->dt == dst->dt && t_numel(x) == t_numel(dst), "unary: x and dst must match");
    DevGuard g(dev->ordinal);
    const size_t n = t_numel(x);
    if (n == 0) return RCU_OK;
    switch (x->dt) {
        case RCU_F32: return launch_unary<float>(dev, op, x->data, dst->data, n);
        case RCU_F16: return launch_unary<__half>(dev, op, x->data, dst->data, n);
        case RCU_BF16: return launch_unary<__nv_bfloat16>(dev, op, x->data, dst->data, n);
    }
    return rcu_fail(dev, RCU_ERR_UNSUPPORTED, "unary: dtype %d", x->dt);
}

rcu_status rcu_cast(rcu_device* dev, const rcu_tensor* x, rcu_tensor* dst) {
    if (!dev) return RCU_ERR_INVALID_ARG;
    RCU_REQUIRE(dev, t_valid(x) && t_valid(dst), "cast: invalid tensor descriptor");
    RCU_REQUIRE(dev, t_numel(x) == t_numel(dst), "cast: element counts differ");
    DevGuard g(dev->ordinal);
    const size_t n = t_numel(x);
    if (n == 0) return RCU_OK;
    const int s = x->dt, d = dst->dt;
    if (s == d) {
        if (x->data != dst->data) RCU_CUDA(dev, cudaMemcpyAsync(dst->data, x->data, n * dt_esize(s), cudaMemcpyDeviceToDevice, dev->stream));
        return RCU_OK;
    }
    if (s == RCU_F32 && d == RCU_F16) return launch_cast<float, __half>(dev, x->data, dst->data, n);
    if (s == RCU_F32 && d == RCU_BF16) return launch_cast<float, __nv_bfloat16>(dev, x->data, dst->data, n);
    if (s == RCU_F16 && d == RCU_F32) return launch_cast<__half, float>(dev, x->data, dst->data, n);
    if (s == RCU_BF16 && d == RCU_F32) return launch_cast<__nv_bfloat16, float>(dev, x->data, dst->data, n);
    const bool reinterpret = (s == RCU_F32 && (d == RCU_I32 || d == RCU_U32)) || ((s == RCU_I32 || s == RCU_U32) && d == RCU_F32);
    if (reinterpret) {  // bytemuck::try_cast_slice (cpu/mod.rs:116-125)
        if (x->data != dst->data) RCU_CUDA(dev, cudaMemcpyAsync(dst->data, x->data, n * 4, cudaMemcpyDeviceToDevice, dev->stream));
        return RCU_OK;
    }
    return rcu_fail(dev, RCU_ERR_UNSUPPORTED, "Cannot cast %d -> %d", s, d);
}

}  // extern "C"
