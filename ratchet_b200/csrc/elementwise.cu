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

template <class T> __device__ __forceinline__ float unary_apply(int op, float x) {
    switch (op) {
        case RCU_GELU: {
            const float c05 = rnd<T>(0.5f), c1 = 1.0f, ck = rnd<T>(0.7978846f), cc = rnd<T>(0.044715f);
            const float inner = rnd<T>(c1 + rnd<T>(rnd<T>(cc * x) * x));
            const float arg = rnd<T>(rnd<T>(ck * x) * inner);
            return rnd<T>(rnd<T>(c05 * x) * rnd<T>(c1 + rnd<T>(tanhf(arg))));
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
        case RCU_SILU: return x / rnd<T>(1.0f + rnd<T>(expf(-x)));
        default: return 1.0f / rnd<T>(1.0f + rnd<T>(expf(-x)));  // sigmoid
    }
}

// ---------------------------------------------------------------------------------- same-shape binary
template <class T, int V>
__global__ void __launch_bounds__(256) binary_same_kernel(int op, const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out, size_t n) {
    const size_t nvec = n / V;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
        const Vec<T, V> va = reinterpret_cast<const Vec<T, V>*>(a)[i];
        const Vec<T, V> vb = reinterpret_cast<const Vec<T, V>*>(b)[i];
        Vec<T, V> vo;
#pragma unroll
        for (int j = 0; j < V; ++j) vo.v[j] = from_f32<T>(binary_apply<T>(op, to_f32<T>(va.v[j]), to_f32<T>(vb.v[j])));
        reinterpret_cast<Vec<T, V>*>(out)[i] = vo;
    }
    if (blockIdx.x == 0) {
        const size_t i = nvec * V + threadIdx.x;
        if (threadIdx.x < (unsigned)V && i < n) out[i] = from_f32<T>(binary_apply<T>(op, to_f32<T>(a[i]), to_f32<T>(b[i])));
    }
}

// ---------------------------------------------------------------------------------- broadcasting binary
struct Bcast4 {
    uint32_t d[4];      // dst shape (4-D promoted)
    uint32_t sa[4];     // element strides of a (0 on broadcast dims)
    uint32_t sb[4];
};

template <class T>
__global__ void __launch_bounds__(256) binary_bcast_kernel(int op, const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out, size_t n, Bcast4 p) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        size_t r = i;
        const uint32_t i3 = (uint32_t)(r % p.d[3]); r /= p.d[3];
        const uint32_t i2 = (uint32_t)(r % p.d[2]); r /= p.d[2];
        const uint32_t i1 = (uint32_t)(r % p.d[1]); r /= p.d[1];
        const uint32_t i0 = (uint32_t)r;
        const size_t oa = (size_t)i0 * p.sa[0] + (size_t)i1 * p.sa[1] + (size_t)i2 * p.sa[2] + (size_t)i3 * p.sa[3];
        const size_t ob = (size_t)i0 * p.sb[0] + (size_t)i1 * p.sb[1] + (size_t)i2 * p.sb[2] + (size_t)i3 * p.sb[3];
        out[i] = from_f32<T>(binary_apply<T>(op, to_f32<T>(a[oa]), to_f32<T>(b[ob])));
    }
}

// ---------------------------------------------------------------------------------- unary / cast
template <class T, int V>
__global__ void __launch_bounds__(256) unary_kernel(int op, const T* __restrict__ x, T* __restrict__ out, size_t n) {
    const size_t nvec = n / V;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
        const Vec<T, V> vx = reinterpret_cast<const Vec<T, V>*>(x)[i];
        Vec<T, V> vo;
#pragma unroll
        for (int j = 0; j < V; ++j) vo.v[j] = from_f32<T>(unary_apply<T>(op, to_f32<T>(vx.v[j])));
        reinterpret_cast<Vec<T, V>*>(out)[i] = vo;
    }
    if (blockIdx.x == 0) {
        const size_t i = nvec * V + threadIdx.x;
        if (threadIdx.x < (unsigned)V && i < n) out[i] = from_f32<T>(unary_apply<T>(op, to_f32<T>(x[i])));
    }
}

template <class S, class D, int V>
__global__ void __launch_bounds__(256) cast_kernel(const S* __restrict__ x, D* __restrict__ out, size_t n) {
    const size_t nvec = n / V;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
        const Vec<S, V> vx = reinterpret_cast<const Vec<S, V>*>(x)[i];
        Vec<D, V> vo;
#pragma unroll
        for (int j = 0; j < V; ++j) vo.v[j] = from_f32<D>(to_f32<S>(vx.v[j]));
        reinterpret_cast<Vec<D, V>*>(out)[i] = vo;
    }
    if (blockIdx.x == 0) {
        const size_t i = nvec * V + threadIdx.x;
        if (threadIdx.x < (unsigned)V && i < n) out[i] = from_f32<D>(to_f32<S>(x[i]));
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
        binary_same_kernel<T, V><<<ew_grid(dev, n / V + 1), 256, 0, dev->stream>>>(op, (const T*)a, (const T*)b, (T*)out, n);
    } else {
        binary_same_kernel<T, 1><<<ew_grid(dev, n), 256, 0, dev->stream>>>(op, (const T*)a, (const T*)b, (T*)out, n);
    }
    RCU_LAUNCH_CHECK(dev);
    return RCU_OK;
}

template <class T>
rcu_status launch_unary(rcu_device* dev, int op, const void* x, void* out, size_t n) {
    constexpr int V = 16 / sizeof(T);
    if (aligned16(x) && aligned16(out)) {
        unary_kernel<T, V><<<ew_grid(dev, n / V + 1), 256, 0, dev->stream>>>(op, (const T*)x, (T*)out, n);
    } else {
        unary_kernel<T, 1><<<ew_grid(dev, n), 256, 0, dev->stream>>>(op, (const T*)x, (T*)out, n);
    }
    RCU_LAUNCH_CHECK(dev);
    return RCU_OK;
}

template <class S, class D>
rcu_status launch_cast(rcu_device* dev, const void* x, void* out, size_t n) {
    constexpr int V = 4;  // 16-byte vectors on the 4-byte side, 8-byte on the 2-byte side
    const bool ok = (reinterpret_cast<uintptr_t>(x) % (sizeof(S) * V) == 0) && (reinterpret_cast<uintptr_t>(out) % (sizeof(D) * V) == 0);
    if (ok) cast_kernel<S, D, V><<<ew_grid(dev, n / V + 1), 256, 0, dev->stream>>>((const S*)x, (D*)out, n);
    else cast_kernel<S, D, 1><<<ew_grid(dev, n), 256, 0, dev->stream>>>((const S*)x, (D*)out, n);
    RCU_LAUNCH_CHECK(dev);
    return RCU_OK;
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
        case RCU_F32: binary_bcast_kernel<float><<<ew_grid(dev, n), 256, 0, dev->stream>>>(op, (const float*)a->data, (const float*)b->data, (float*)dst->data, n, p); break;
        case RCU_F16: binary_bcast_kernel<__half><<<ew_grid(dev, n), 256, 0, dev->stream>>>(op, (const __half*)a->data, (const __half*)b->data, (__half*)dst->data, n, p); break;
        default: binary_bcast_kernel<__nv_bfloat16><<<ew_grid(dev, n), 256, 0, dev->stream>>>(op, (const __nv_bfloat16*)a->data, (const __nv_bfloat16*)b->data, (__nv_bfloat16*)dst->data, n, p); break;
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
