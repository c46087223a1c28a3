// Prefill GEMM on the 5th-generation tensor cores (tcgen05), Linear convention:
//   out[M, N] = X[M, K] . W[N, K]^T (+ bias),  X and out f16, f32 accumulation in tensor memory.
//
// Takes the place of ratchet-core's `gemm` WGSL kernel (ops/matmul/gemm.rs:462-746: 32x32 SIMT tiles,
// f32 accumulate) and of its Q4_K stub (ops/matmul/quantized.rs:138-278) for the shapes a Linear
// produces at sequence length > 1 (ratchet-nn/src/linear.rs:17-24: lhs = W[N,K], trans_rhs,
// trans_dst).  Both operands are K-major, which is what UMMA shared-memory descriptors want.
//
// One CTA computes one 128 x BN output tile:
//   warp 0 (one lane)  TMA producer: 128 x 64 activation tile and BN x 64 weight tile per stage,
//                      128-byte swizzle, completion on the stage's `full` mbarrier;
//   warp 1             allocates tensor memory; one lane issues four tcgen05.mma (K = 16 each) per
//                      stage and commits them to the stage's `empty` mbarrier, and at the end to
//                      the accumulator barrier;
//   warps 2-5          epilogue: tcgen05.ld the f32 accumulators (lane = token row, column =
//                      output feature), add bias, round to f16, store rows.
// Quantised weights (Q8_0H, Q4_KH) are dequantised inside the kernel (up to 256 token rows): TMA
// brings the packed bytes of the weight tile into shared memory, further warps convert them to f16
// with the CPU dequantiser's arithmetic and write the swizzled tile the MMA reads.  Larger M
// dequantises once into pooled scratch and runs the f16 kernel.
//
// Every mbarrier wait is bounded; a wait that gives up sets RCU_DEVFLAG_TIMEOUT and an abort word in
// shared memory that ends all other waits of the CTA, and the CTA still frees its tensor memory.
#include <cuda.h>

#include <cstdlib>

#include "dequant.cuh"
#include "tc_common.cuh"

namespace {

using namespace rcu_dequant;
using namespace tc;

}  // namespace

namespace {

enum { WK_F16 = 0, WK_Q8 = 1, WK_Q4K = 2 };   // how the weight tile reaches shared memory

struct QuantArgs {
    const void* scales;     // Q8_0H: f16 block scales [N * K/32]; Q4_KH: 12-byte (scale, min) packs [N * K/256]
    const __half* d;        // Q4_KH super-block scale  [N * K/256]
    const __half* dmin;     // Q4_KH super-block min    [N * K/256]
};

// One CTA computes one 128 x BN output tile.  WK_F16: the weight tile arrives by TMA like the
// activation tile.  WK_Q8 / WK_Q4K: TMA brings the packed bytes of the tile (BN rows x 64 int8 or
// BN rows x 32 nibble bytes) into the tail of the stage's weight area; warps 6-9 read them into
// registers, convert to f16 and write the 128-byte-swizzled K-major tile the MMA reads, so the
// dequantised matrix never exists in global memory.
// converting warps per CTA: two per scheduler for the wide tile (one 32-weight task per thread per stage)
__host__ __device__ constexpr int conv_warps(int bn) { return bn >= 128 ? 8 : 4; }

// Two CTAs share an SM (half of its shared memory and at most half of its tensor memory each), so one
// CTA's pipeline fill and epilogue overlap the other's main loop.
template <int BN, int WK, int STAGES>
__global__ void __launch_bounds__(WK == WK_F16 ? kThreadsTc : kThreadsTc + conv_warps(BN) * 32, 2)
gemm_tc_kernel(const __grid_constant__ CUtensorMap xmap, const __grid_constant__ CUtensorMap wmap, const QuantArgs qa,
               const __half* __restrict__ bias, __half* __restrict__ out, int M, int N, int K, int* status, int splits, float* __restrict__ partial) {
    rcu_kernel_entry_wait_only();
    constexpr int A_BYTES = TM * TK * 2;          // 16 KiB
    constexpr int B_BYTES = BN * TK * 2;
    constexpr int STAGE = A_BYTES + B_BYTES;
    constexpr int RAW_ROW = WK == WK_Q8 ? 64 : 32;
    constexpr int RAW_BYTES = WK == WK_F16 ? 0 : BN * RAW_ROW;
    extern __shared__ unsigned char smem_dyn[];
    // 1024-byte alignment: the 128-byte swizzle pattern repeats every 8 rows = 1024 bytes
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE);
    uint64_t* empty = full + STAGES;
    uint64_t* raw_full = empty + STAGES;
    uint64_t* accum_bar = raw_full + STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum_bar + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.y * TM, n0 = blockIdx.x * BN;
    // blockIdx.z is an independent problem (batched f16 products), or - splits > 1 - a slice of K: the CTA then runs
    // k-steps [it_base, it_base + nk) and leaves f32 partial sums for sum_k_slices_kernel
    const int nk_all = (K + TK - 1) / TK;
    const int nk_per = splits > 1 ? (((nk_all + splits - 1) / splits + 3) & ~3) : nk_all;     // whole Q4_K super-blocks per slice
    const int sp = splits > 1 ? (int)blockIdx.z : 0;
    const int it_base = sp * nk_per;
    const int nk = max(0, min(nk_all - it_base, nk_per));
    const int bz = splits > 1 ? 0 : (int)blockIdx.z;
    out += (size_t)bz * M * N;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], WK == WK_F16 ? 1 : conv_warps(BN));   // TMA transaction, or one arrival per converting warp
            mbar_init(&empty[s], 1);
            mbar_init(&raw_full[s], 1);
        }
        mbar_init(accum_bar, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        // tensor memory: BN f32 columns x 128 lanes for the accumulator tile (power of two >= 32)
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "n"(BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            for (int it = 0; it < nk; ++it) {
                const int s = it % STAGES;
                if (it >= STAGES && !mbar_wait(&empty[s], ((it / STAGES) - 1) & 1, abort_flag, status)) break;
                unsigned char* st = smem + s * STAGE;
                if (WK == WK_F16) {
                    mbar_expect_tx(&full[s], STAGE);
                    tma_load_3d(st, &xmap, (it_base + it) * TK, m0, bz, &full[s]);             // activations: rows m0.., k it*64..
                    tma_load_3d(st + A_BYTES, &wmap, (it_base + it) * TK, n0, bz, &full[s]);   // weights: rows n0..
                } else {
                    mbar_expect_tx(&raw_full[s], A_BYTES + RAW_BYTES);
                    tma_load_3d(st, &xmap, (it_base + it) * TK, m0, 0, &raw_full[s]);
                    tma_load_2d(st + STAGE - RAW_BYTES, &wmap, (it_base + it) * RAW_ROW, n0, &raw_full[s]);   // packed bytes of 64 weights per row
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_f16(TM, BN);
            bool ok = true;
            for (int it = 0; it < nk && ok; ++it) {
                const int s = it % STAGES;
                ok = mbar_wait(&full[s], (it / STAGES) & 1, abort_flag, status);
                if (!ok) break;
                tc_fence_after();
                unsigned char* st = smem + s * STAGE;
                const uint64_t adesc = umma_desc_sw128(st);
                const uint64_t bdesc = umma_desc_sw128(st + A_BYTES);
#pragma unroll
                for (int k = 0; k < TK / 16; ++k) {
                    // advance 16 elements = 32 bytes inside the 128-byte swizzle row: +2 in 16-byte units
                    umma_f16(tmem_base, adesc + 2 * k, bdesc + 2 * k, idesc, (it > 0 || k > 0) ? 1u : 0u);
                }
                umma_commit(&empty[s]);      // the stage may be refilled once these MMAs have read it
            }
            umma_commit(accum_bar);          // accumulators complete (arrives even after an abort so the epilogue ends)
        }
    } else if (warp < 6) {
        // epilogue warps 2..5: tensor-memory lane quarter = warp index modulo 4
        const int q = warp & 3;
        const bool ok = mbar_wait(accum_bar, 0, abort_flag, status);
        tc_fence_after();
        const int row = m0 + q * 32 + lane;
        if (ok) {
#pragma unroll 1
            for (int c = 0; c < BN; c += 32) {
                float v[32];
                tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c, v);
                if (row < M && splits > 1) {         // a K slice: f32 partial sums, bias and rounding in the summing kernel (N % 8 == 0)
                    float* prow = partial + ((size_t)sp * M + row) * N + n0 + c;
#pragma unroll
                    for (int j = 0; j < 32; j += 4)
                        if (n0 + c + j + 4 <= N) *reinterpret_cast<float4*>(prow + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                } else if (row < M) {
                    __half* orow = out + (size_t)row * N + n0 + c;
                    if ((N & 7) == 0) {              // rows start on 16-byte boundaries
#pragma unroll
                        for (int j = 0; j < 32; j += 8) {
                            const int col = n0 + c + j;
                            if (col + 8 <= N) {
                                __align__(16) __half h[8];
#pragma unroll
                                for (int e = 0; e < 8; ++e) h[e] = __float2half_rn(v[j + e] + (bias ? __half2float(bias[col + e]) : 0.f));
                                *reinterpret_cast<uint4*>(orow + j) = *reinterpret_cast<const uint4*>(h);
                            } else {
                                for (int e = 0; e < 8 && col + e < N; ++e)
                                    orow[j + e] = __float2half_rn(v[j + e] + (bias ? __half2float(bias[col + e]) : 0.f));
                            }
                        }
                    } else {                         // N a multiple of 4 (checked by the host): 8-byte stores
#pragma unroll
                        for (int j = 0; j < 32; j += 4) {
                            const int col = n0 + c + j;
                            if (col + 4 <= N) {
                                __align__(8) __half h[4];
#pragma unroll
                                for (int e = 0; e < 4; ++e) h[e] = __float2half_rn(v[j + e] + (bias ? __half2float(bias[col + e]) : 0.f));
                                *reinterpret_cast<uint2*>(orow + j) = *reinterpret_cast<const uint2*>(h);
                            }
                        }
                    }
                }
            }
        }
    } else if (WK != WK_F16) {
        // converting warps 6...  Task = (tile row r, half h): 32 weights = one Q8_0 block or one Q4_K
        // sub-block = four 16-byte chunks of the row's 128-byte swizzled line.
        constexpr int CT = conv_warps(BN) * 32;      // converting threads
        constexpr int TPT = BN * 2 / CT;
        constexpr int PF = 4;                       // Q8_0: block scales are fetched this many stages ahead
        const int dt = threadIdx.x - kThreadsTc;
        // Scales come from global memory and are requested ahead of use, so their latency overlaps the
        // conversion of earlier stages: Q8_0 keeps a queue of PF block scales per task; Q4_K keeps the
        // current and the next super-block's packs (one super-block = four stages).
        __half q8_queue[PF][TPT];
        uint32_t pk_cur[TPT][3], pk_next[TPT][3];
        __half dd_cur[TPT][2], dd_next[TPT][2];
        auto q8_fetch = [&](int stage, int t) -> __half {
            const int task = dt + t * CT, r = task >> 1, h = task & 1;
            const int row = n0 + r, kk = stage * TK + h * 32;
            if (row < N && kk < K) return reinterpret_cast<const __half*>(qa.scales)[(size_t)row * (K >> 5) + (kk >> 5)];
            return __float2half_rn(0.f);
        };
        auto q4_fetch = [&](int sblock, int t, uint32_t* pk, __half* dd) {
            const int task = dt + t * CT, r = task >> 1;
            const int row = n0 + r;
            pk[0] = pk[1] = pk[2] = 0u;
            dd[0] = dd[1] = __float2half_rn(0.f);
            if (row < N && sblock * 256 < K) {
                const size_t sb = (size_t)row * (K >> 8) + sblock;
                const uint32_t* g = reinterpret_cast<const uint32_t*>(qa.scales) + sb * 3;
                pk[0] = __ldg(g); pk[1] = __ldg(g + 1); pk[2] = __ldg(g + 2);
                dd[0] = qa.d[sb];
                dd[1] = qa.dmin[sb];
            }
        };
#pragma unroll
        for (int t = 0; t < TPT; ++t) {
            if (WK == WK_Q8) {
#pragma unroll
                for (int p = 0; p < PF; ++p) q8_queue[p][t] = q8_fetch(it_base + p, t);
            } else {
                q4_fetch(it_base >> 2, t, pk_next[t], dd_next[t]);
            }
        }
        bool stop = false;
        for (int it0 = 0; it0 < nk && !stop; it0 += PF) {
#pragma unroll
        for (int u = 0; u < PF; ++u) {               // unrolled: queue slot u is a fixed register
            const int it = it0 + u;
            if (it >= nk || stop) break;
            const int s = it % STAGES;
            const int itg = it_base + it;                // k-step of the whole problem
            const int k0 = itg * TK;
            __half2 mul2[TPT], neg2[TPT];
            bool valid[TPT];
#pragma unroll
            for (int t = 0; t < TPT; ++t) {
                const int task = dt + t * CT, r = task >> 1, h = task & 1;
                const int row = n0 + r;
                valid[t] = row < N && k0 + h * 32 < K;
                neg2[t] = __float2half2_rn(0.f);
                if (WK == WK_Q8) {
                    mul2[t] = __half2half2(q8_queue[u][t]);
                    q8_queue[u][t] = q8_fetch(itg + PF, t);    // consumed PF stages from now
                } else {
                    if ((itg & 3) == 0) {
#pragma unroll
                        for (int i = 0; i < 3; ++i) pk_cur[t][i] = pk_next[t][i];
                        dd_cur[t][0] = dd_next[t][0];
                        dd_cur[t][1] = dd_next[t][1];
                        q4_fetch((itg >> 2) + 1, t, pk_next[t], dd_next[t]);
                    }
                    const uint32_t* w = pk_cur[t];
                    const int j = (itg & 3) * 2 + h;
                    uint32_t sc, mn;
                    if (j < 4) {                                   // quantized.rs:158-204
                        sc = pack_byte(w, j) & 63u;
                        mn = pack_byte(w, j + 4) & 63u;
                    } else {
                        sc = (pack_byte(w, j + 4) & 0xFu) | ((pack_byte(w, j - 4) >> 6) << 4);
                        mn = (pack_byte(w, j + 4) >> 4) | ((pack_byte(w, j) >> 6) << 4);
                    }
                    // delta = fp(scale * d), min = fp(m * dmin): small integers times f16, rounded once
                    mul2[t] = __half2half2(__hmul_rn(__uint2half_rn(sc), dd_cur[t][0]));
                    neg2[t] = __half2half2(__hneg(__hmul_rn(__uint2half_rn(mn), dd_cur[t][1])));
                }
            }
            const bool arrived = mbar_wait(&raw_full[s], (it / STAGES) & 1, abort_flag, status);
            unsigned char* bt = smem + s * STAGE + A_BYTES;
            const unsigned char* raw = smem + s * STAGE + STAGE - RAW_BYTES;
            uint4 qv[TPT][2];
#pragma unroll
            for (int t = 0; t < TPT; ++t) {
                const int task = dt + t * CT, r = task >> 1, h = task & 1;
                const uint4* src = reinterpret_cast<const uint4*>(raw + r * RAW_ROW + (WK == WK_Q8 ? h * 32 : 0));
                qv[t][0] = src[0];
                qv[t][1] = src[1];
            }
            // the packed bytes sit inside the area the f16 tile is written to: every task's bytes are in
            // registers before any thread stores (named barrier 1: the four converting warps).  The same
            // barrier tells all of them whether any wait gave up, so they leave the loop together.
            uint32_t gave_up;
            asm volatile(
                "{\n\t.reg .pred p, q;\n\t"
                "setp.eq.u32 q, %1, 0;\n\t"
                "barrier.cta.red.or.pred p, 1, %2, q;\n\t"
                "selp.u32 %0, 1, 0, p;\n\t}"
                : "=r"(gave_up)
                : "r"((uint32_t)arrived), "n"(CT)
                : "memory");
            if (gave_up) { stop = true; break; }
#pragma unroll
            for (int t = 0; t < TPT; ++t) {
                const int task = dt + t * CT, r = task >> 1, h = task & 1;
                const uint32_t w[8] = {qv[t][0].x, qv[t][0].y, qv[t][0].z, qv[t][0].w, qv[t][1].x, qv[t][1].y, qv[t][1].z, qv[t][1].w};
                unsigned char* line = bt + r * 128;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    uint4 o = make_uint4(0u, 0u, 0u, 0u);
                    if (valid[t]) {
                        if (WK == WK_Q8) o = dequant8_q8(w[2 * i], w[2 * i + 1], mul2[t]);
                        else o = dequant8_q4(w[2 * i] >> (4 * h), w[2 * i + 1] >> (4 * h), mul2[t], neg2[t]);
                    }
                    const int chunk = (4 * h + i) ^ (r & 7);           // 128-byte swizzle: 16-byte chunk index xor row-in-group
                    *reinterpret_cast<uint4*>(line + chunk * 16) = o;
                }
            }
            // generic-proxy stores -> visible to the tensor core's async-proxy reads, then one arrival per warp
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&full[s]);
        }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "n"(BN) : "memory");
    }
}

// out[m, n] = f16(sum over slices, in order, of partial[s, m, n] + bias[n]); eight outputs per thread
__global__ void __launch_bounds__(256) sum_k_slices_kernel(const float* __restrict__ partial, const __half* __restrict__ bias, __half* __restrict__ out,
                                                          size_t MN, int N, int splits) {
    rcu_kernel_entry();
    const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (i >= MN) return;
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
    for (int s = 0; s < splits; ++s) {
        const float4 a = *reinterpret_cast<const float4*>(partial + (size_t)s * MN + i), b = *reinterpret_cast<const float4*>(partial + (size_t)s * MN + i + 4);
        acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
        acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
    }
    __align__(16) __half h[8];
    const int col = (int)(i % (size_t)N);
#pragma unroll
    for (int e = 0; e < 8; ++e) h[e] = __float2half_rn(acc[e] + (bias ? __half2float(bias[col + e]) : 0.f));
    *reinterpret_cast<uint4*>(out + i) = *reinterpret_cast<const uint4*>(h);
}

template <int BN, int WK>
rcu_status launch_tc(rcu_device* dev, const CUtensorMap& xmap, const CUtensorMap& wmap, const QuantArgs& qa, const void* bias, void* out,
                     int M, int N, int K, int batch = 1) {
    constexpr int STAGE = TM * TK * 2 + BN * TK * 2;
    constexpr int STAGES = (100 * 1024) / STAGE;     // two CTAs per SM
    const size_t smem = (size_t)STAGES * STAGE + 1024 + 512;
    auto kern = gemm_tc_kernel<BN, WK, STAGES>;
    RCU_CUDA(dev, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid((N + BN - 1) / BN, (M + TM - 1) / TM, batch);
    const int threads = WK == WK_F16 ? kThreadsTc : kThreadsTc + conv_warps(BN) * 32;
    // Few tiles and a long K (a Linear at a few hundred token rows): every CTA's k loop is a chain of TMA -> convert -> MMA
    // hand-overs about half a microsecond per step long, so K is cut into slices that run side by side (two CTAs fit an SM).
    const int nk = (K + TK - 1) / TK;
    const long long tiles = (long long)grid.x * grid.y;
    int splits = 1;
    if (batch == 1 && N % 8 == 0 && tiles <= dev->sm_count && nk >= 16) {
        splits = (int)std::min<long long>(4, (2ll * dev->sm_count) / tiles);
        while (splits > 1 && (((nk + splits - 1) / splits + 3) & ~3) * (splits - 1) >= nk) --splits;     // every slice gets k-steps
    }
    if (splits > 1) {
        void* partial = nullptr;
        rcu_status st = rcu_alloc(dev, (uint64_t)splits * M * N * 4, &partial);
        if (st != RCU_OK) return st;
        grid.z = splits;
        rcu_launch(dev, kern, grid, threads, smem, xmap, wmap, qa, nullptr, (__half*)out, M, N, K, dev->d_status, splits, (float*)partial);
        dev->launches++;
        const size_t MN = (size_t)M * N;
        rcu_launch(dev, sum_k_slices_kernel, (unsigned)((MN / 8 + 255) / 256), 256, 0, (const float*)partial, (const __half*)bias, (__half*)out, MN, N, splits);
        rcu_free(dev, partial);      // the pool reuses blocks in stream order
        RCU_LAUNCH_CHECK(dev);
        return RCU_OK;
    }
    rcu_launch(dev, kern, grid, threads, smem, xmap, wmap, qa, (const __half*)bias, (__half*)out, M, N, K, dev->d_status, 1, nullptr);
    RCU_LAUNCH_CHECK(dev);
    return RCU_OK;
}

// [batch, rows, K] f16, rows `pitch` elements apart (a multiple of 8: tensor-map strides are 16-byte multiples), box =
// box_rows x 64 elements of one problem, 128-byte swizzle; reads beyond K or rows are filled with zeros
bool make_map_f16_sw128(CUtensorMap* map, const void* base, uint64_t rows, uint64_t K, uint32_t box_rows, uint64_t batch = 1, uint64_t pitch = 0) {
    gemvq8::EncodeTiledFn fn = gemvq8::encode_tiled_fn();
    if (!fn) return false;
    if (pitch == 0) pitch = K;
    cuuint64_t dims[3] = {K, rows, batch};
    cuuint64_t strides[2] = {pitch * 2, rows * pitch * 2};
    cuuint32_t box[3] = {(cuuint32_t)TK, box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

bool rcu_gemm_tc_eligible(int lhs_dt, int act_dt, uint64_t M, uint64_t N, uint64_t K) {
    if (act_dt != RCU_F16) return false;
    if (!(lhs_dt == RCU_F16 || lhs_dt == RCU_Q8_0H || lhs_dt == RCU_Q4_KH)) return false;
    // small problems stay on the SIMT kernel; K rows must be 16-byte multiples for the tensor maps
    if (M < 32 || N < 64 || K < 64 || K % 8 != 0 || N % 8 != 0) return false;
    if (M > 0x7fffffffull || N > 0x7fffffffull || K > 0x7fffffffull) return false;
    return true;
}

// gemm_tc2.cu: the CTA-pair kernel for f16 weights
bool rcu_gemm_tc2_eligible(rcu_device* dev, uint64_t M, uint64_t N, uint64_t K);
rcu_status rcu_gemm_tc2_launch(rcu_device* dev, const void* w, const void* x, const void* bias, void* y, uint64_t M, uint64_t N, uint64_t K);

rcu_status rcu_gemm_tc_dispatch(rcu_device* dev, int lhs_dt, const void* w, int act_dt, const void* x, const void* bias, void* y,
                                uint64_t M, uint64_t N, uint64_t K) {
    if (!rcu_gemm_tc_eligible(lhs_dt, act_dt, M, N, K)) return RCU_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(w)) & 15) return RCU_ERR_UNSUPPORTED;
    DevGuard g(dev->ordinal);
    if (lhs_dt == RCU_F16 && rcu_gemm_tc2_eligible(dev, M, N, K)) return rcu_gemm_tc2_launch(dev, w, x, bias, y, M, N, K);
    // Quantised weights.  The fused kernel converts a weight tile once per 128-row token tile, i.e.
    // M/128 times over the whole problem, and it is the one-CTA kernel.  Beyond kFusedMaxM token rows it
    // is cheaper to convert the matrix once into pooled f16 scratch (which stays in L2) and run the f16
    // kernels on it (M = 512, N = 8192, K = 3072, Q4_K: 34 us against 46 us fused).  RCU_GEMM_FUSED=0/1
    // forces either path.
    constexpr uint64_t kFusedMaxM = 256;
    if (lhs_dt != RCU_F16) {
        const char* force = getenv("RCU_GEMM_FUSED");
        const bool fused = force ? atoi(force) != 0 : M <= kFusedMaxM;
        if (!fused) {
            void* scratch = nullptr;
            rcu_status st = rcu_alloc(dev, N * K * 2, &scratch);
            if (st != RCU_OK) return st;
            rcu_tensor src{lhs_dt, 2, {N, K, 1, 1}, const_cast<void*>(w)};
            rcu_tensor dst{RCU_F16, 2, {N, K, 1, 1}, scratch};
            st = rcu_dequantize(dev, &src, &dst);
            if (st == RCU_OK) st = rcu_gemm_tc_dispatch(dev, RCU_F16, scratch, act_dt, x, bias, y, M, N, K);
            rcu_free(dev, scratch);   // the pool reuses blocks in stream order
            return st;
        }
    }
    // tile width: enough CTAs to cover the SMs when M is small
    const uint64_t tiles128 = ((M + TM - 1) / TM) * ((N + 127) / 128);
    int bn = tiles128 >= (uint64_t)dev->sm_count ? 128 : 64;
    // f16 weights and enough 128 x 256 tiles for two CTAs on every SM: the wide tile halves the shared-memory
    // reads per flop (a 128 x 128 x 16 MMA reads A and B at the full shared-memory rate)
    static const int force_bn = [] { const char* e = getenv("RCU_GEMM_BN"); return e ? atoi(e) : 0; }();
    if (lhs_dt == RCU_F16 && (force_bn == 256 || (force_bn == 0 && tiles128 / 2 >= 2ull * dev->sm_count))) bn = 256;
    CUtensorMap xmap, wmap;
    QuantArgs qa{nullptr, nullptr, nullptr};
    bool maps = make_map_f16_sw128(&xmap, x, M, K, TM);
    const int wk = lhs_dt == RCU_F16 ? WK_F16 : (lhs_dt == RCU_Q8_0H ? WK_Q8 : WK_Q4K);
    size_t off[4];
    if (wk == WK_F16) {
        maps = maps && make_map_f16_sw128(&wmap, w, N, K, (uint32_t)bn);
    } else {
        rcu_dtype_segments(lhs_dt, N * K, off);
        const char* base = (const char*)w;
        if (wk == WK_Q8) {
            // packed int8 [N, K]: 64 bytes of a row per stage
            maps = maps && gemvq8::make_map_2d(&wmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, base, N, K, 64, (uint32_t)bn);
            qa.scales = base + off[1];
        } else {
            // nibble bytes [N, K/2]: 32 bytes of a row per stage (sub-blocks 2c and 2c+1 of a super-block)
            maps = maps && gemvq8::make_map_2d(&wmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, base, N, K / 2, 32, (uint32_t)bn);
            qa.scales = base + off[1];
            qa.dmin = (const __half*)(base + off[2]);
            qa.d = (const __half*)(base + off[3]);
        }
    }
    rcu_status st = RCU_OK;
    if (!maps)
        st = rcu_fail(dev, RCU_ERR_CUDA, "gemm_tc: cuTensorMapEncodeTiled failed (M=%llu N=%llu K=%llu)", (unsigned long long)M,
                      (unsigned long long)N, (unsigned long long)K);
#define RCU_TC(BN_, WK_) launch_tc<BN_, WK_>(dev, xmap, wmap, qa, bias, y, (int)M, (int)N, (int)K)
    if (st == RCU_OK) {
        if (wk == WK_F16) st = bn == 256 ? RCU_TC(256, WK_F16) : bn == 128 ? RCU_TC(128, WK_F16) : RCU_TC(64, WK_F16);
        else if (wk == WK_Q8) st = bn == 128 ? RCU_TC(128, WK_Q8) : RCU_TC(64, WK_Q8);
        else st = bn == 128 ? RCU_TC(128, WK_Q4K) : RCU_TC(64, WK_Q4K);
    }
#undef RCU_TC
    return st;
}

// `batch` independent products out[b] = X[b] . W[b]^T with X [batch, M, pitch_x] and W [batch, N, pitch_w] f16, both K-major
// (K <= pitch, pitches multiples of 8), out [batch, M, N] f16 contiguous with N a multiple of 4.  The attention products
// of an f16 model (whisper/mha.rs:95-110: q.k^T over 6 heads, then weights.v) take this; blockIdx.z is the problem.
rcu_status rcu_gemm_tc_batched_f16(rcu_device* dev, const void* w, const void* x, void* y, uint64_t M, uint64_t N, uint64_t K, uint64_t batch,
                                   uint64_t pitch_w, uint64_t pitch_x) {
    if (M < 32 || N < 64 || K < 64 || N % 4 != 0 || pitch_w % 8 != 0 || pitch_x % 8 != 0 || batch == 0 || batch > 65535) return RCU_ERR_UNSUPPORTED;
    if (M > 0x7fffffffull || N > 0x7fffffffull || K > 0x7fffffffull) return RCU_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) & 15) return RCU_ERR_UNSUPPORTED;
    if (reinterpret_cast<uintptr_t>(y) & ((N % 8 == 0) ? 15 : 7)) return RCU_ERR_UNSUPPORTED;
    DevGuard g(dev->ordinal);
    const uint64_t tiles128 = ((M + TM - 1) / TM) * ((N + 127) / 128) * batch;
    const int bn = (tiles128 >= (uint64_t)dev->sm_count && N >= 128) ? 128 : 64;
    CUtensorMap xmap, wmap;
    if (!make_map_f16_sw128(&xmap, x, M, K, TM, batch, pitch_x) || !make_map_f16_sw128(&wmap, w, N, K, (uint32_t)bn, batch, pitch_w))
        return rcu_fail(dev, RCU_ERR_CUDA, "gemm_tc: cuTensorMapEncodeTiled failed (batched M=%llu N=%llu K=%llu)", (unsigned long long)M,
                        (unsigned long long)N, (unsigned long long)K);
    QuantArgs qa{nullptr, nullptr, nullptr};
    return bn == 128 ? launch_tc<128, WK_F16>(dev, xmap, wmap, qa, nullptr, y, (int)M, (int)N, (int)K, (int)batch)
                     : launch_tc<64, WK_F16>(dev, xmap, wmap, qa, nullptr, y, (int)M, (int)N, (int)K, (int)batch);
}
