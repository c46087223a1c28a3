// Q4_K GEMV: y[N] = W[N, K] . x[K] (+ bias) for Q4_KF / Q4_KH weights in ratchet's segment layout
// ([qs numel/2][scales 12 B per 256][dmin][d], dtype/blocks.rs:124-148) and an f32 / f16 vector.
//
// The reference has no kernel for this pair (`(gemv, q4)` is `todo!()`, ops/matmul/mod.rs:746); its
// meaning is fixed by QMatMul's block decode (ops/matmul/quantized.rs:158-266): per 32-weight
// sub-block j of a 256-weight block, weight = q * (d * sc_j) - dmin * m_j, sub-blocks 2c / 2c+1 in the
// low / high nibbles of the c-th 32-byte chunk.  A row's dot product is therefore
//   sum_j [ (d sc_j) * sum_i q_ji x_ji  -  (dmin m_j) * sum_i x_ji ],
// so the kernel needs integer dot products of 4-bit codes with the activations, and the activations'
// sums per 16 elements.
//
// HBM-bound at 0.5625 bytes per weight, which leaves about one and a half instruction slots per weight at
// full bandwidth.  The activations are staged once per CTA as fixed point (x = s * X with s = max|x| /
// (2^(8P-1) - 1); P = 2 byte planes for f16 activations, 3 for f32: 2^-15 / 2^-23 of the vector's scale),
// the top plane signed and the others unsigned, and every four codes meet each plane in one dp4a.  The
// twelve packed 6-bit scale / min bytes of a block are unpacked eight at a time with word-wide masks.
// d * sc and dmin * m are kept in f32 (the dequantiser rounds them to the scale type: a 2^-11 relative
// difference per sub-block in the f16 layout, far inside the bar); the sums are f32.
//
// Work split: persistent CTAs, teams of KSPLIT warps own whole groups of four rows.  A lane takes one
// 32-byte chunk (sub-blocks 2c and 2c+1 whole) of one block in two of the four rows; a half-warp covers
// four blocks (1024 weights) of its two rows per step, and three register slots of loads stay in flight.
#include "common.cuh"

namespace {

constexpr int kThreadsQ4 = 256;
constexpr int kWarpsQ4 = kThreadsQ4 / 32;
constexpr int kRowsQ4 = 4;      // rows per group
constexpr int kLaneRows = 2;    // of which a lane handles two

__device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c) {   // unsigned bytes of a x signed bytes of b
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ int dp4a_uu(uint32_t a, uint32_t b, int c) {   // unsigned x unsigned
    uint32_t d;
    asm("dp4a.u32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"((uint32_t)c));
    return (int)d;
}

// 16-byte slot of activation vector c16 inside a byte plane.  The 16 lanes of a half-warp read the vectors
// (block b, chunk c, part t) = 16 b + 4 c + t for four b and four c at once; folding bits 3-5 of the index
// into its low three bits spreads them over all eight 16-byte bank groups (two per group, the minimum).
__device__ __forceinline__ int plane_slot(int c16) { return (c16 & ~7) | ((c16 ^ (c16 >> 3)) & 7); }

// 32 bytes in one streaming load (each lane's chunk is read exactly once)
__device__ __forceinline__ void ld_stream_256(const void* p, uint32_t (&v)[8]) {
    asm volatile("ld.global.cs.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                 : "l"(p));
}

// One pipeline slot.  Everything is kept as loaded (conversions happen where the values are used, so that
// filling a slot never waits for its own loads).
template <class FP> struct SlotQ4 {
    uint32_t w[kLaneRows][8];       // the 32-byte chunk of each row
    uint32_t sc[kLaneRows][3];      // the block's 12 packed scale bytes
    FP d[kLaneRows], dmin[kLaneRows];
};

template <class FP, class ActT, int KSPLIT>
__global__ void __launch_bounds__(kThreadsQ4, 2)
gemv_q4k_kernel(const uint8_t* __restrict__ qs, const uint8_t* __restrict__ scales, const FP* __restrict__ dmin,
                const FP* __restrict__ d, const ActT* __restrict__ x, const ActT* __restrict__ bias, ActT* __restrict__ y,
                int N, int K) {
    rcu_kernel_entry();
    constexpr int P = sizeof(ActT) == 4 ? 3 : 2;                   // byte planes of the fixed-point activations
    constexpr float kXmax = P == 3 ? 8388607.f : 32767.f;
    extern __shared__ __align__(16) unsigned char smem_q4[];
    unsigned char* plane = smem_q4;                                // plane p at p * K: p = 0 is the signed top byte
    float* xsum = reinterpret_cast<float*>(smem_q4 + (size_t)P * K);   // s * sum of X over each 32 elements
    float* red = xsum + K / 32;                                    // [kWarpsQ4][kRowsQ4]
    float* misc = red + kWarpsQ4 * kRowsQ4;                        // [kWarpsQ4] warp maxima

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    constexpr int RG = kWarpsQ4 / KSPLIT;
    const int rg = warp / KSPLIT, ks = warp % KSPLIT;
    const long long gw = (long long)blockIdx.x * RG + rg, W = (long long)gridDim.x * RG;
    const long long n_groups_all = (N + kRowsQ4 - 1) / kRowsQ4;
    const int g_begin = (int)((gw * n_groups_all) / W), g_end = (int)(((gw + 1) * n_groups_all) / W);
    const int kblocks = K >> 8;                       // 256-weight blocks per row
    const int nchunks = (kblocks + 3) >> 2;           // a half-warp covers four blocks per step
    const int ncs = (nchunks - ks + KSPLIT - 1) / KSPLIT;          // steps of this warp per row group
    const int n_items = (g_end - g_begin) * ncs;
    const int cidx = lane & 3;                        // 32-byte chunk of the block: sub-blocks 2 cidx (low nibbles), 2 cidx + 1 (high)
    const int bl = (lane >> 2) & 3;                   // block within the step
    const int rsel = (lane >> 4) * kLaneRows;         // first of this lane's two rows within the group

    auto load_item = [&](int it, SlotQ4<FP>& s) {
        const int r0 = (g_begin + it / ncs) * kRowsQ4 + rsel;
        const int kb = (ks + (it % ncs) * KSPLIT) * 4 + bl;
        const bool live = kb < kblocks;
#pragma unroll
        for (int r = 0; r < kLaneRows; ++r) {
            const size_t B = (size_t)min(r0 + r, N - 1) * kblocks + kb;    // rows past N repeat the last one; dropped at the store
            if (live) {
                ld_stream_256(qs + B * 128 + cidx * 32, s.w[r]);
                const uint32_t* pk = reinterpret_cast<const uint32_t*>(scales + B * 12);
                s.sc[r][0] = __ldg(pk); s.sc[r][1] = __ldg(pk + 1); s.sc[r][2] = __ldg(pk + 2);
                s.d[r] = d[B];
                s.dmin[r] = dmin[B];
            } else {
#pragma unroll
                for (int q = 0; q < 8; ++q) s.w[r][q] = 0;
                s.sc[r][0] = s.sc[r][1] = s.sc[r][2] = 0;
                s.d[r] = s.dmin[r] = from_f32<FP>(0.f);
            }
        }
    };

    SlotQ4<FP> s0, s1, s2;
    if (n_items > 0) load_item(0, s0);
    if (n_items > 1) load_item(1, s1);
    if (n_items > 2) load_item(2, s2);

    // ---- stage x: scale, fixed-point byte planes, sums per 32 elements
    // 16 elements per thread and trip, as 16-byte vector loads (x comes from the kernel before: read at L2)
    auto load16 = [&](int i16, float (&v)[16]) {
        if constexpr (sizeof(ActT) == 4) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float4 f = __ldcg(reinterpret_cast<const float4*>(x) + i16 * 4 + q);
                v[4 * q] = f.x; v[4 * q + 1] = f.y; v[4 * q + 2] = f.z; v[4 * q + 3] = f.w;
            }
        } else {
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                const uint4 u = __ldcg(reinterpret_cast<const uint4*>(x) + i16 * 2 + q);
                const uint32_t hw[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&hw[e]));
                    v[8 * q + 2 * e] = f.x; v[8 * q + 2 * e + 1] = f.y;
                }
            }
        }
    };
    float amax = 0.f;
    for (int i16 = tid; i16 < K / 16; i16 += kThreadsQ4) {
        float v[16];
        load16(i16, v);
#pragma unroll
        for (int e = 0; e < 16; ++e) amax = fmaxf(amax, fabsf(v[e]));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if (lane == 0) misc[warp] = amax;
    __syncthreads();
    amax = misc[0];
#pragma unroll
    for (int w = 1; w < kWarpsQ4; ++w) amax = fmaxf(amax, misc[w]);
    const float sx = amax / kXmax;
    const float inv = amax > 0.f ? kXmax / amax : 0.f;
    for (int base = warp * 32; base < K / 16; base += kThreadsQ4) {       // warp-uniform trip count: the shuffle below needs every lane
        const int i16 = base + lane;
        const bool on = i16 < K / 16;
        uint32_t pw[P][4];
        int tot = 0;
        float v[16];
        if (on) load16(i16, v);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
#pragma unroll
            for (int p = 0; p < P; ++p) pw[p][q] = 0;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int X = on ? __float2int_rn(v[q * 4 + e] * inv) : 0;
                tot += X;
#pragma unroll
                for (int p = 0; p < P; ++p) pw[p][q] |= (uint32_t)((X >> (8 * (P - 1 - p))) & 0xFF) << (8 * e);
            }
        }
        // two neighbouring lanes hold the halves of a 32-element sum
        const int both = tot + __shfl_xor_sync(0xffffffffu, tot, 1);
        if (on) {
#pragma unroll
            for (int p = 0; p < P; ++p)
                reinterpret_cast<uint4*>(plane + (size_t)p * K)[plane_slot(i16)] = make_uint4(pw[p][0], pw[p][1], pw[p][2], pw[p][3]);
            if ((i16 & 1) == 0) xsum[i16 >> 1] = sx * (float)both;
        }
    }
    __syncthreads();

    float acc[kLaneRows];
#pragma unroll
    for (int r = 0; r < kLaneRows; ++r) acc[r] = 0.f;

    auto compute_item = [&](int it, const SlotQ4<FP>& s) {
        const int kb = (ks + (it % ncs) * KSPLIT) * 4 + bl;
        if (kb < kblocks) {
            const int e_lo = kb * 256 + cidx * 64, e_hi = e_lo + 32;
            const int slot_base = (kb * 16 + cidx * 4) & ~7, slot_lo = (cidx & 1) * 4, slot_x = (kb * 2 + (cidx >> 1)) & 7;
            // integer dots of both rows' codes with the activation planes, one sub-block (nibble half) at a time
            int dot[kLaneRows][P][2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                uint32_t xa[P][8];                  // [plane][8 words of four elements]
#pragma unroll
                for (int p = 0; p < P; ++p) {
                    // vectors 16 kb + 4 cidx + 2 h + {0, 1}: plane_slot() with the shared terms taken out
                    const uint4* src = reinterpret_cast<const uint4*>(plane + (size_t)p * K) + slot_base;
                    const uint4 a = src[(slot_lo + 2 * h) ^ slot_x], b = src[(slot_lo + 2 * h + 1) ^ slot_x];
                    xa[p][0] = a.x; xa[p][1] = a.y; xa[p][2] = a.z; xa[p][3] = a.w;
                    xa[p][4] = b.x; xa[p][5] = b.y; xa[p][6] = b.z; xa[p][7] = b.w;
                }
#pragma unroll
                for (int r = 0; r < kLaneRows; ++r) {
                    const uint32_t* ws = s.w[r];
#pragma unroll
                    for (int p = 0; p < P; ++p) dot[r][p][h] = 0;
#pragma unroll
                    for (int q = 0; q < 8; ++q) {
                        const uint32_t c4 = (h ? ws[q] >> 4 : ws[q]) & 0x0F0F0F0Fu;
                        dot[r][0][h] = dp4a_us(c4, xa[0][q], dot[r][0][h]);
#pragma unroll
                        for (int p = 1; p < P; ++p) dot[r][p][h] = dp4a_uu(c4, xa[p][q], dot[r][p][h]);
                    }
                }
            }
            const float xs_lo = xsum[e_lo >> 5], xs_hi = xsum[e_hi >> 5];
#pragma unroll
            for (int r = 0; r < kLaneRows; ++r) {
                // the block's eight 6-bit scales and mins, four per word (quantized.rs:158-204): sub-blocks 0-3
                // sit in the low six bits of bytes 0-3 / 4-7; sub-blocks 4-7 take four bits from bytes 8-11
                // and two from the top of bytes 0-3 (scales) or 4-7 (mins)
                const uint32_t w0 = s.sc[r][0], w1 = s.sc[r][1], w2 = s.sc[r][2];
                const uint32_t sc4 = cidx < 2 ? (w0 & 0x3F3F3F3Fu) : ((w2 & 0x0F0F0F0Fu) | ((w0 >> 2) & 0x30303030u));
                const uint32_t mn4 = cidx < 2 ? (w1 & 0x3F3F3F3Fu) : (((w2 >> 4) & 0x0F0F0F0Fu) | ((w1 >> 2) & 0x30303030u));
                const int sh = (cidx & 1) * 16;       // sub-blocks 2 cidx, 2 cidx + 1 within their group of four
                const float df = to_f32<FP>(s.d[r]), mf = to_f32<FP>(s.dmin[r]);
                const float del0 = (float)((sc4 >> sh) & 0xFFu) * df, del1 = (float)((sc4 >> (sh + 8)) & 0xFFu) * df;
                const float mn0 = (float)((mn4 >> sh) & 0xFFu) * mf, mn1 = (float)((mn4 >> (sh + 8)) & 0xFFu) * mf;
                float v0, v1;
                if (P == 2) {
                    v0 = (float)(dot[r][0][0] * 256 + dot[r][1][0]);
                    v1 = (float)(dot[r][0][1] * 256 + dot[r][1][1]);
                } else {
                    v0 = fmaf((float)dot[r][0][0], 65536.f, (float)(dot[r][1][0] * 256 + dot[r][P - 1][0]));
                    v1 = fmaf((float)dot[r][0][1], 65536.f, (float)(dot[r][1][1] * 256 + dot[r][P - 1][1]));
                }
                float a = acc[r];
                a = fmaf(del0 * sx, v0, a);
                a = fmaf(del1 * sx, v1, a);
                a = fmaf(-mn0, xs_lo, a);
                a = fmaf(-mn1, xs_hi, a);
                acc[r] = a;
            }
        }
        if (it % ncs != ncs - 1) return;
        // last step of this row group: reduce over each half-warp (and the team's warps) and store
        const int r0 = (g_begin + it / ncs) * kRowsQ4;
#pragma unroll
        for (int r = 0; r < kLaneRows; ++r) {
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) acc[r] += __shfl_xor_sync(0xffffffffu, acc[r], o);
        }
        if (KSPLIT > 1) {
            if ((lane & 15) == 0) {
#pragma unroll
                for (int r = 0; r < kLaneRows; ++r) red[warp * kRowsQ4 + rsel + r] = acc[r];
            }
            asm volatile("bar.sync %0, %1;" ::"r"(1 + rg), "r"(KSPLIT * 32) : "memory");
            if (ks == 0 && lane < kRowsQ4 && r0 + lane < N) {
                float sum = 0.f;
#pragma unroll
                for (int q = 0; q < KSPLIT; ++q) sum += red[(rg * KSPLIT + q) * kRowsQ4 + lane];
                if (bias) sum += to_f32<ActT>(bias[r0 + lane]);
                y[r0 + lane] = from_f32<ActT>(sum);
            }
            asm volatile("bar.sync %0, %1;" ::"r"(1 + rg), "r"(KSPLIT * 32) : "memory");
        } else if ((lane & 15) == 0) {
#pragma unroll
            for (int r = 0; r < kLaneRows; ++r) {
                const int row = r0 + rsel + r;
                if (row < N) y[row] = from_f32<ActT>(acc[r] + (bias ? to_f32<ActT>(bias[row]) : 0.f));
            }
        }
#pragma unroll
        for (int r = 0; r < kLaneRows; ++r) acc[r] = 0.f;
    };

    for (int it = 0; it < n_items; it += 3) {
        compute_item(it, s0);
        if (it + 3 < n_items) load_item(it + 3, s0);
        if (it + 1 < n_items) {
            compute_item(it + 1, s1);
            if (it + 4 < n_items) load_item(it + 4, s1);
        }
        if (it + 2 < n_items) {
            compute_item(it + 2, s2);
            if (it + 5 < n_items) load_item(it + 5, s2);
        }
    }
}

template <class FP, class ActT>
rcu_status launch_q4k(rcu_device* dev, const void* w, const void* x, const void* bias, void* y, int N, int K) {
    uint64_t off[4];
    rcu_dtype_segments(sizeof(FP) == 4 ? RCU_Q4_KF : RCU_Q4_KH, (uint64_t)N * K, off);
    const uint8_t* base = (const uint8_t*)w;
    const size_t smem = (sizeof(ActT) == 4 ? 3 : 2) * (size_t)K + (size_t)(K / 32) * 4 + (kWarpsQ4 * kRowsQ4 + kWarpsQ4) * sizeof(float);
    if (smem > (size_t)dev->smem_optin) return rcu_fail(dev, RCU_ERR_UNSUPPORTED, "gemv_q4k: K=%d does not fit the activation stage", K);
    const long long max_ctas = (long long)dev->sm_count * 2;
    const long long groups = (N + kRowsQ4 - 1) / kRowsQ4;
    const int nchunks = ((K >> 8) + 3) >> 2;
    // enough warps in flight when N is small: split a row group's steps over 2-8 warps; with only a few
    // groups per team the team that gets one more sets the kernel's time, so when that imbalance exceeds
    // 6 % take the split that minimises it
    int ksplit = 1;
    while (ksplit < 8 && groups * ksplit * 2 <= max_ctas * kWarpsQ4 && nchunks >= ksplit * 2) ksplit *= 2;
    auto imbalance = [&](int ks) {
        const long long teams = max_ctas * (kWarpsQ4 / ks);
        const double avg = (double)groups / (double)teams;
        return avg <= 0.0 ? 1.0 : (double)((groups + teams - 1) / teams) / avg;
    };
    if (groups * ksplit > max_ctas * kWarpsQ4 / 2 && imbalance(ksplit) > 1.06) {
        int best = ksplit;
        for (int ks = ksplit * 2; ks <= 8 && nchunks >= ks * 2; ks *= 2)
            if (imbalance(ks) < imbalance(best) - 0.01) best = ks;
        ksplit = best;
    }
    const long long ctas_needed = (groups * ksplit + kWarpsQ4 - 1) / kWarpsQ4;
    const int grid = (int)std::max<long long>(1, std::min(ctas_needed, max_ctas));
#define RCU_Q4K_CASE(KS)                                                                                                   \
    case KS: {                                                                                                             \
        auto kern = gemv_q4k_kernel<FP, ActT, KS>;                                                                         \
        if (smem > 48 * 1024) RCU_CUDA(dev, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        rcu_launch(dev, kern, grid, kThreadsQ4, smem, base, base + off[1], (const FP*)(base + off[2]), (const FP*)(base + off[3]), \
                                                      (const ActT*)x, (const ActT*)bias, (ActT*)y, N, K);                  \
        break;                                                                                                             \
    }
    switch (ksplit) {
        RCU_Q4K_CASE(1)
        RCU_Q4K_CASE(2)
        RCU_Q4K_CASE(4)
        RCU_Q4K_CASE(8)
    }
#undef RCU_Q4K_CASE
    RCU_LAUNCH_CHECK(dev);
    return RCU_OK;
}

}  // namespace

// lhs_dt is RCU_Q4_KF (with f32 x) or RCU_Q4_KH (with f16 x); K a multiple of 256.
rcu_status rcu_gemv_q4k_dispatch(rcu_device* dev, int lhs_dt, const void* w, int act_dt, const void* x, const void* bias, void* y,
                                 uint64_t N, uint64_t K) {
    if (K % 256 != 0) return rcu_fail(dev, RCU_ERR_INVALID_ARG, "gemv: Q4_K rows must hold whole 256-element blocks (K=%llu)", (unsigned long long)K);
    if (N > 0x7fffffffull || K > 0x7fffffffull) return rcu_fail(dev, RCU_ERR_UNSUPPORTED, "gemv: dimension exceeds 2^31");
    if ((reinterpret_cast<uintptr_t>(w) & 31) || (reinterpret_cast<uintptr_t>(x) & 15))
        return rcu_fail(dev, RCU_ERR_INVALID_ARG, "gemv: Q4_K weights must be 32-byte aligned and the vector 16-byte aligned");
    DevGuard g(dev->ordinal);
    if (lhs_dt == RCU_Q4_KF && act_dt == RCU_F32) return launch_q4k<float, float>(dev, w, x, bias, y, (int)N, (int)K);
    if (lhs_dt == RCU_Q4_KH && act_dt == RCU_F16) return launch_q4k<__half, __half>(dev, w, x, bias, y, (int)N, (int)K);
    return rcu_fail(dev, RCU_ERR_UNSUPPORTED, "gemv: dtype pair (%d,%d) has no kernel", lhs_dt, act_dt);
}
