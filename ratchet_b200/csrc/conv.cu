// conv1d with kernel size 3 (the only size the reference supports, ops/conv.rs:139-144).
//
// Stands in for ratchet-core's `conv1d_3x3` WGSL kernel (ops/conv.rs:40-123): x [B,Cin,Lin],
// w [Cout,Cin,3], bias [Cout] -> y [B,Cout,Lout], Lout = (Lin + 2*pad - 3)/stride + 1.  As in the
// shader, the three taps are accumulated in three separate fma chains over the input channels and
// summed with the bias at the end.
//
// A CTA computes a 64 (Cout) x 64 (Lout) output tile; input channels are consumed 8 at a time
// through shared memory (input window and filter slab), each thread owning a 4 x 4 register tile.
//
// f32 problems large enough for the tensor cores take another route: the input is unfolded into
// col[Lout, 3*Cin] (col[l, 3*ci + t] = x[ci, l*stride + t - pad], zero outside the input) and the product
// y[Cout, Lout] = w[Cout, 3*Cin] . col^T runs on the split-TF32 tcgen05 GEMM with the bias added per row.
#include "common.cuh"

rcu_status rcu_gemm_tc_f32_dispatch(rcu_device* dev, const void* w, const void* x, const void* bias, void* y, uint64_t M, uint64_t N,
                                    uint64_t K, uint64_t batches, const void* bias_rows);
bool rcu_gemm_tc_f32_eligible(int lhs_dt, int act_dt, uint64_t M, uint64_t N, uint64_t K);

namespace {

constexpr int TCO = 64, TLO = 64, TCI = 8;

template <class T, int STRIDE>
__global__ void __launch_bounds__(256)
conv1d_k3_kernel(const T* __restrict__ x, const T* __restrict__ w, const T* __restrict__ bias, T* __restrict__ y,
                 int Cin, int Lin, int Cout, int Lout, int pad) {
    rcu_kernel_entry();
    constexpr int WIN = (TLO - 1) * STRIDE + 3;           // input positions needed by the tile
    __shared__ float xs[TCI][WIN + 1];
    __shared__ float ws[TCI][3][TCO + 1];
    const int b = blockIdx.z;
    const int co0 = blockIdx.y * TCO, lo0 = blockIdx.x * TLO;
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;                // tx -> 4 output positions, ty -> 4 channels
    const int in0 = lo0 * STRIDE - pad;
    float a0[4][4], a1[4][4], a2[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) a0[i][j] = a1[i][j] = a2[i][j] = 0.f;

    for (int ci0 = 0; ci0 < Cin; ci0 += TCI) {
        for (int e = tid; e < TCI * WIN; e += 256) {
            const int c = e / WIN, p = e - c * WIN;
            const int ci = ci0 + c, pos = in0 + p;
            xs[c][p] = (ci < Cin && pos >= 0 && pos < Lin) ? to_f32<T>(x[((size_t)b * Cin + ci) * Lin + pos]) : 0.f;
        }
        for (int e = tid; e < TCO * TCI * 3; e += 256) {
            // weights are [Cout][Cin][3]: walk (co, c, t) with (c, t) fastest so reads are contiguous
            const int co = e / (TCI * 3), rem = e - co * (TCI * 3);
            const int c = rem / 3, t = rem - c * 3;
            const int gco = co0 + co, ci = ci0 + c;
            ws[c][t][co] = (gco < Cout && ci < Cin) ? to_f32<T>(w[((size_t)gco * Cin + ci) * 3 + t]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int c = 0; c < TCI; ++c) {
            float w0[4], w1[4], w2[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) { w0[i] = ws[c][0][ty * 4 + i]; w1[i] = ws[c][1][ty * 4 + i]; w2[i] = ws[c][2][ty * 4 + i]; }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int p = (tx * 4 + j) * STRIDE;
                const float x0 = xs[c][p], x1 = xs[c][p + 1], x2 = xs[c][p + 2];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    a0[i][j] = fmaf(x0, w0[i], a0[i][j]);
                    a1[i][j] = fmaf(x1, w1[i], a1[i][j]);
                    a2[i][j] = fmaf(x2, w2[i], a2[i][j]);
                }
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int co = co0 + ty * 4 + i;
        if (co >= Cout) continue;
        const float bv = bias ? to_f32<T>(bias[co]) : 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int lo = lo0 + tx * 4 + j;
            if (lo < Lout) y[((size_t)b * Cout + co) * Lout + lo] = from_f32<T>(a0[i][j] + a1[i][j] + a2[i][j] + bv);
        }
    }
}

// Unfold one batch of x [Cin, Lin] into col [Lout, 3*Cin].  A CTA takes 32 output positions x 32 input
// channels: the input window goes through shared memory so that both the reads (along the length) and
// the writes (96 consecutive floats per output position) are coalesced.
template <int STRIDE>
__global__ void __launch_bounds__(256)
unfold_k3_kernel(const float* __restrict__ x, float* __restrict__ col, int Cin, int Lin, int Lout, int pad) {
    rcu_kernel_entry();
    constexpr int WIN = 31 * STRIDE + 3;
    __shared__ float win[32][WIN + 1];
    const int l0 = blockIdx.x * 32, ci0 = blockIdx.y * 32;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int p0 = l0 * STRIDE - pad;
    for (int r = warp; r < 32; r += 8) {
        const int ci = ci0 + r;
        for (int p = lane; p < WIN; p += 32) {
            const int pos = p0 + p;
            win[r][p] = (ci < Cin && pos >= 0 && pos < Lin) ? x[(size_t)ci * Lin + pos] : 0.f;
        }
    }
    __syncthreads();
    const int K = 3 * Cin;
    const int width = min(32, Cin - ci0) * 3;
    for (int idx = threadIdx.x; idx < 32 * 96; idx += 256) {
        const int l = idx / 96, t = idx - l * 96;
        if (l0 + l < Lout && t < width) col[(size_t)(l0 + l) * K + ci0 * 3 + t] = win[t / 3][l * STRIDE + t % 3];
    }
}

}  // namespace

extern "C" rcu_status rcu_conv1d(rcu_device* dev, const rcu_tensor* x, const rcu_tensor* w, const rcu_tensor* bias,
                                 uint32_t stride, uint32_t padding, rcu_tensor* dst) {
    if (!dev) return RCU_ERR_INVALID_ARG;
    RCU_REQUIRE(dev, t_valid(x) && t_valid(w) && t_valid(dst), "conv1d: invalid tensor descriptor");
    RCU_REQUIRE(dev, x->rank == 3 && w->rank == 3, "conv1d: input and weight must be rank 3");   // ops/conv.rs:129-131
    RCU_REQUIRE(dev, w->shape[2] == 3, "conv1d: only kernel size 3 is supported");
    RCU_REQUIRE(dev, x->dt == w->dt && dst->dt == x->dt && (!bias || bias->dt == x->dt), "conv1d: dtype mismatch");
    RCU_REQUIRE(dev, stride == 1 || stride == 2, "conv1d: stride must be 1 or 2");
    const uint64_t B = x->shape[0], Cin = x->shape[1], Lin = x->shape[2], Cout = w->shape[0];
    RCU_REQUIRE(dev, w->shape[1] == Cin, "conv1d: weight expects %llu input channels, x has %llu", (unsigned long long)w->shape[1], (unsigned long long)Cin);
    RCU_REQUIRE(dev, Lin + 2 * padding >= 3, "conv1d: input shorter than the kernel");
    const uint64_t Lout = (Lin + 2 * padding - 3) / stride + 1;
    RCU_REQUIRE(dev, dst->rank == 3 && dst->shape[0] == B && dst->shape[1] == Cout && dst->shape[2] == Lout, "conv1d: dst must be [%llu,%llu,%llu]", (unsigned long long)B, (unsigned long long)Cout, (unsigned long long)Lout);
    RCU_REQUIRE(dev, !bias || t_numel(bias) == Cout, "conv1d: bias must have Cout elements");
    DevGuard g(dev->ordinal);
    dim3 grid((unsigned)((Lout + TLO - 1) / TLO), (unsigned)((Cout + TCO - 1) / TCO), (unsigned)B);
    RCU_REQUIRE(dev, grid.y <= 65535 && grid.z <= 65535, "conv1d: too many channels / batches");
    const void* bp = bias ? bias->data : nullptr;
    if (rcu_gemm_tc_f32_eligible(w->dt, x->dt, Cout, Lout, 3 * Cin) && Cin <= 65535ull * 32 && Lin <= 0x3fffffffull) {
        void* col = nullptr;
        rcu_status st = rcu_alloc(dev, Lout * 3 * Cin * 4, &col);
        if (st != RCU_OK) return st;
        const dim3 ugrid((unsigned)((Lout + 31) / 32), (unsigned)((Cin + 31) / 32));
        for (uint64_t b = 0; b < B && st == RCU_OK; ++b) {
            const float* xb = (const float*)x->data + b * Cin * Lin;
            if (stride == 1) rcu_launch(dev, unfold_k3_kernel<1>, ugrid, 256, 0, xb, (float*)col, (int)Cin, (int)Lin, (int)Lout, (int)padding);
            else rcu_launch(dev, unfold_k3_kernel<2>, ugrid, 256, 0, xb, (float*)col, (int)Cin, (int)Lin, (int)Lout, (int)padding);
            st = rcu_gemm_tc_f32_dispatch(dev, col, w->data, nullptr, (float*)dst->data + b * Cout * Lout, Cout, Lout, 3 * Cin, 1, bp);
        }
        rcu_free(dev, col);       // the pool reuses blocks in stream order
        if (st != RCU_ERR_UNSUPPORTED) {
            if (st == RCU_OK) RCU_LAUNCH_CHECK(dev);
            return st;
        }
    }
#define RCU_CONV(T, S) rcu_launch(dev, conv1d_k3_kernel<T, S>, grid, 256, 0, (const T*)x->data, (const T*)w->data, (const T*)bp, (T*)dst->data, (int)Cin, (int)Lin, (int)Cout, (int)Lout, (int)padding)
    if (x->dt == RCU_F32) { if (stride == 1) RCU_CONV(float, 1); else RCU_CONV(float, 2); }
    else if (x->dt == RCU_F16) { if (stride == 1) RCU_CONV(__half, 1); else RCU_CONV(__half, 2); }
    else return rcu_fail(dev, RCU_ERR_UNSUPPORTED, "conv1d: dtype %d", x->dt);
#undef RCU_CONV
    RCU_LAUNCH_CHECK(dev);
    return RCU_OK;
}
