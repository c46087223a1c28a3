// Rotary position embedding on [B,H,S,D], rotating the first `dim` features in half-split pairs
// (i, i + dim/2); features >= dim pass through.
//
// Stands in for ratchet-core's `rope` WGSL kernel (ops/rope.rs:112-164).  Arithmetic follows the
// CPU device (cpu/rope.rs:23-143): inv_f[i] = exp(-i * ln(base) / (dim/2)), theta = (s + offset) *
// inv_f[i] in f32, out1 = x1*cos - x2*sin, out2 = x1*sin + x2*cos.  ln(base) is taken on the host
// with the C library; exp / sin / cos are evaluated in double precision from the f32 arguments and
// rounded to f32, which reproduces a correctly rounded f32 libm (the angle reaches thousands of
// radians at long offsets, where a 1-ulp difference in inv_f alone would move sin/cos by 1e-4).
#include <cmath>

#include "common.cuh"

namespace {

template <class T>
__global__ void __launch_bounds__(128)
rope_kernel(const T* __restrict__ x, T* __restrict__ out, int BH, int S, int D, int dim, float ln_base, int offset) {
    const int half = dim >> 1;
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;   // over S * half
    if (idx < S * half) {
        const int s = idx / half, i = idx - s * half;
        const float neg_i = -(float)i;
        const float e = neg_i * ln_base / (float)half;       // f32 ops, left to right (cpu/rope.rs:38-41)
        const float inv = (float)exp((double)e);
        const float th = (float)(s + offset) * inv;
        double sd, cd;
        sincos((double)th, &sd, &cd);
        const float sn = (float)sd, cs = (float)cd;
        for (int bh = blockIdx.y; bh < BH; bh += gridDim.y) {
            const size_t o = ((size_t)bh * S + s) * D;
            const float x1 = to_f32<T>(x[o + i]), x2 = to_f32<T>(x[o + half + i]);
            // each product is rounded on its own, as on the CPU (no fma contraction)
            out[o + i] = from_f32<T>(__fsub_rn(rnd<T>(__fmul_rn(x1, cs)), rnd<T>(__fmul_rn(x2, sn))));
            out[o + half + i] = from_f32<T>(__fadd_rn(rnd<T>(__fmul_rn(x1, sn)), rnd<T>(__fmul_rn(x2, cs))));
        }
    }
    // pass-through tail (only needed when out != x)
    if (dim < D && out != x) {
        const int tail = D - dim;
        if (idx < S * tail) {
            const int s = idx / tail, i = dim + (idx - s * tail);
            for (int bh = blockIdx.y; bh < BH; bh += gridDim.y) {
                const size_t o = ((size_t)bh * S + s) * D + i;
                out[o] = x[o];
            }
        }
    }
}

}  // namespace

extern "C" rcu_status rcu_rope(rcu_device* dev, const rcu_tensor* x, uint32_t dim, float base, uint32_t offset, rcu_tensor* dst) {
    if (!dev) return RCU_ERR_INVALID_ARG;
    RCU_REQUIRE(dev, t_valid(x) && t_valid(dst), "rope: invalid tensor descriptor");
    RCU_REQUIRE(dev, x->rank == 4, "rope: input must be [B,H,S,D]");           // ops/rope.rs check_shapes
    RCU_REQUIRE(dev, dst->dt == x->dt && t_numel(dst) == t_numel(x), "rope: dst must match x");
    const uint64_t B = x->shape[0], H = x->shape[1], S = x->shape[2], D = x->shape[3];
    RCU_REQUIRE(dev, dim >= 2 && dim % 2 == 0 && dim <= D, "rope: dim must be even and <= head dim");
    RCU_REQUIRE(dev, S * D <= 0x7fffffffull && B * H <= 0x7fffffffull, "rope: tensor too large");
    DevGuard g(dev->ordinal);
    const int half = (int)dim / 2;
    const int per_row = std::max(half, (int)(D - dim));
    const int work = (int)S * per_row;
    dim3 grid((work + 127) / 128, (unsigned)std::min<uint64_t>(B * H, 64));
    const float ln_base = logf(base);
    switch (x->dt) {
        case RCU_F32: rope_kernel<float><<<grid, 128, 0, dev->stream>>>((const float*)x->data, (float*)dst->data, (int)(B * H), (int)S, (int)D, (int)dim, ln_base, (int)offset); break;
        case RCU_F16: rope_kernel<__half><<<grid, 128, 0, dev->stream>>>((const __half*)x->data, (__half*)dst->data, (int)(B * H), (int)S, (int)D, (int)dim, ln_base, (int)offset); break;
        default: return rcu_fail(dev, RCU_ERR_UNSUPPORTED, "rope: dtype %d", x->dt);
    }
    RCU_LAUNCH_CHECK(dev);
    return RCU_OK;
}
