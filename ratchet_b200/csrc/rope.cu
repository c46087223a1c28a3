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

template <class T, int V> struct alignas(sizeof(T) * V) RopeVec { T v[V]; };

// Thread = V consecutive rotation pairs of one sequence position: the V angles are evaluated once
// and applied to that position in every (batch, head) slice this thread visits, one vector load per
// half and one vector store per half each time.  (dim/2) % V == 0 and D % V == 0.
template <class T, int V>
__global__ void __launch_bounds__(128)
rope_kernel(const T* x, T* out, int BH, int S, int D, int dim, float ln_base, int offset) {
    rcu_kernel_entry();
    typedef RopeVec<T, V> VT;
    const int half = dim >> 1;
    const int hv = half / V;
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;   // over S * hv
    if (idx < S * hv) {
        const int s = idx / hv, i0 = (idx - s * hv) * V;
        float sn[V], cs[V];
#pragma unroll
        for (int e = 0; e < V; ++e) {
            const float neg_i = -(float)(i0 + e);
            const float ex = neg_i * ln_base / (float)half;   // f32 ops, left to right (cpu/rope.rs:38-41)
            const float inv = (float)exp((double)ex);
            const float th = (float)(s + offset) * inv;
            double sd, cd;
            sincos((double)th, &sd, &cd);
            sn[e] = (float)sd;
            cs[e] = (float)cd;
        }
#pragma unroll 2
        for (int bh = blockIdx.y; bh < BH; bh += gridDim.y) {
            const size_t o = ((size_t)bh * S + s) * D + i0;
            const VT a = *reinterpret_cast<const VT*>(x + o);
            const VT b = *reinterpret_cast<const VT*>(x + o + half);
            VT ra, rb;
#pragma unroll
            for (int e = 0; e < V; ++e) {
                const float x1 = to_f32<T>(a.v[e]), x2 = to_f32<T>(b.v[e]);
                // each product is rounded on its own, as on the CPU (no fma contraction)
                ra.v[e] = from_f32<T>(__fsub_rn(rnd<T>(__fmul_rn(x1, cs[e])), rnd<T>(__fmul_rn(x2, sn[e]))));
                rb.v[e] = from_f32<T>(__fadd_rn(rnd<T>(__fmul_rn(x1, sn[e])), rnd<T>(__fmul_rn(x2, cs[e]))));
            }
            *reinterpret_cast<VT*>(out + o) = ra;
            *reinterpret_cast<VT*>(out + o + half) = rb;
        }
    }
    // pass-through tail (only needed when out != x)
    if (dim < D && out != x) {
        const int tv = (D - dim) / V;
        if (idx < S * tv) {
            const int s = idx / tv, i = dim + (idx - s * tv) * V;
            for (int bh = blockIdx.y; bh < BH; bh += gridDim.y) {
                const size_t o = ((size_t)bh * S + s) * D + i;
                *reinterpret_cast<VT*>(out + o) = *reinterpret_cast<const VT*>(x + o);
            }
        }
    }
}

template <class T>
void launch_rope(rcu_device* dev, const void* x, void* out, int BH, int S, int D, int dim, float ln_base, int offset) {
    constexpr int VF = 16 / sizeof(T);
    const int half = dim / 2;
    const bool vec = half % VF == 0 && D % VF == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
    const int v = vec ? VF : 1;
    const int per_row = std::max(half, D - dim) / v;
    const int work = S * per_row;
    const int gx = (work + 127) / 128;
    // enough (batch, head) slices per thread to amortise the angle evaluation, enough CTAs to fill the GPU
    const int want = (dev->sm_count * 16 + gx - 1) / gx;
    dim3 grid(gx, (unsigned)std::max(1, std::min(BH, want)));
    if (vec) rcu_launch(dev, rope_kernel<T, VF>, grid, 128, 0, (const T*)x, (T*)out, BH, S, D, dim, ln_base, offset);
    else rcu_launch(dev, rope_kernel<T, 1>, grid, 128, 0, (const T*)x, (T*)out, BH, S, D, dim, ln_base, offset);
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
    const float ln_base = logf(base);
    switch (x->dt) {
        case RCU_F32: launch_rope<float>(dev, x->data, dst->data, (int)(B * H), (int)S, (int)D, (int)dim, ln_base, (int)offset); break;
        case RCU_F16: launch_rope<__half>(dev, x->data, dst->data, (int)(B * H), (int)S, (int)D, (int)dim, ln_base, (int)offset); break;
        default: return rcu_fail(dev, RCU_ERR_UNSUPPORTED, "rope: dtype %d", x->dt);
    }
    RCU_LAUNCH_CHECK(dev);
    return RCU_OK;
}
