// f32 Linear on the tensor cores with f32-level accuracy (split-TF32):
//   out[M, N] = X[M, K] . W[N, K]^T (+ bias), everything f32.
//
// ratchet runs f32 models (Phi-2 and Whisper checkpoints as shipped, ops/matmul/gemm.rs) and its CPU
// device, the parity target, accumulates f32 products (cpu/gemm.rs); the bar for f32 ops is 1e-4.  A
// TF32 tensor-core product keeps 10 mantissa bits per operand, which alone misses that bar, so each
// operand is split into two TF32 values, x = hi + lo with hi = x truncated to TF32 and lo = x - hi
// (exact in f32), and three products are accumulated in tensor memory:
//   hi_a hi_b + hi_a lo_b + lo_a hi_b      (lo_a lo_b, below 2^-22 of the result, is dropped).
// The tensor core adds into its f32 accumulator with truncation: every accumulating MMA loses up to
// one unit in the last place of the running sum, always toward zero, which over K/8 k-steps measures
// about 1.3e-8 * K of the result.  Two things keep that below the bar for the K of real layers (up to
// 10240): the two small products go to accumulators of their own (their sum is 2^-11 of the main one,
// and so are its truncation errors), and the main products rotate over several accumulators (all 512
// tensor-memory columns are used), which the epilogue adds up with ordinary rounded f32 additions.
//
// Structure as gemm_tc.cu: TMA brings 128 x 32 (activations) and BN x 32 (weights) f32 tiles,
// 128-byte swizzled, into a shared-memory ring; the raw tile serves as the hi operand (the tensor core
// reads only the upper 19 bits of a word) and eight converting warps write the lo part to a twin tile at
// the same swizzled offsets (so no swizzle arithmetic is needed); one thread issues twelve tcgen05.mma
// kind::tf32 (K = 8) per stage; four warps read the f32 accumulators from tensor memory, add the bias
// and store.  The kernel is bound by shared-memory bandwidth (TMA fill, lo pass, three operand reads per
// k-step), so the tile width is chosen by whole waves and short grids split K over blockIdx.z with an
// ordered sum of the slices.  blockIdx.z otherwise indexes independent problems (attention heads).
// Every wait is bounded.
#include <cstdlib>

#include "tc_common.cuh"

namespace {

using namespace tc;

// kind::tf32 reads the upper 19 bits of each 32-bit operand word (the parity tests hold only if it does):
// the raw f32 tile already is the hi operand x & 0xFFFFE000, so only the lo tile x - hi is written.
constexpr int TK32 = 32;                 // K per stage: 32 f32 = 128 bytes = one swizzle row
constexpr int kConvWarps = 8;
// accumulators: the hi x hi products rotate over `mains`, the small products over `corrs` (512 columns in all)
__host__ __device__ constexpr int main_accs(int bn) { return bn == 64 ? 6 : 3; }
__host__ __device__ constexpr int corr_accs(int bn) { return bn == 64 ? 2 : 1; }
constexpr int kThreadsF32 = kThreadsTc + kConvWarps * 32;

// 32-bit instruction descriptor, kind::tf32: TF32 A and B (both K-major), f32 D, M x N tile.
__host__ __device__ constexpr uint32_t umma_idesc_tf32(int m, int n) {
    return (1u << 4)                      // D format f32
           | (2u << 7) | (2u << 10)       // A, B format TF32
           | (0u << 15) | (0u << 16)      // A, B K-major
           | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// TMR = token rows of a tile, 128 or 64.  With 64 the accumulator rows sit in the first 16 lanes of each 32-lane
// quarter of tensor memory (row r in lane 32 (r / 16) + r % 16); a tile costs half the shared-memory traffic on the
// activation side, which is what small M (Phi-2's 64 rows) and grids that do not fill the SMs want.
template <int BN, int STAGES, int TMR>
__global__ void __launch_bounds__(kThreadsF32, 1)
gemm_tc_f32_kernel(const __grid_constant__ CUtensorMap xmap, const __grid_constant__ CUtensorMap wmap, const float* __restrict__ bias,
                   const float* __restrict__ bias_rows,
                   float* __restrict__ out, int M, int N, int K, int kb_per_split, int* status) {
    rcu_kernel_entry_wait_only();
    constexpr int A_BYTES = TMR * TK32 * 4;       // 16 or 8 KiB
    constexpr int B_BYTES = BN * TK32 * 4;
    constexpr int RAW = A_BYTES + B_BYTES;        // hi tiles (A then B); the lo tiles follow in the same order
    constexpr int STAGE = 2 * RAW;
    extern __shared__ unsigned char smem_dyn[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE);
    uint64_t* empty = full + STAGES;
    uint64_t* raw_full = empty + STAGES;
    uint64_t* accum_bar = raw_full + STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum_bar + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.y * TMR, n0 = blockIdx.x * BN;
    // blockIdx.z is either the problem of a batch (attention heads: third coordinate of both maps) or, when
    // kb_per_split > 0, the slice of K this CTA sums: slice z covers k-blocks [z * kb_per_split, ...) of the
    // one problem and writes its partial result to slab z of `out`.
    const int nk_all = (K + TK32 - 1) / TK32;
    const int kb0 = kb_per_split > 0 ? (int)blockIdx.z * kb_per_split : 0;
    const int nk = kb_per_split > 0 ? min(kb_per_split, nk_all - kb0) : nk_all;
    const int batch = kb_per_split > 0 ? 0 : (int)blockIdx.z;
    out += (size_t)blockIdx.z * M * N;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], kConvWarps);
            mbar_init(&empty[s], 1);
            mbar_init(&raw_full[s], 1);
        }
        mbar_init(accum_bar, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "n"(512) : "memory");
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
                if (it >= STAGES && !mbar_wait_spin(&empty[s], ((it / STAGES) - 1) & 1, abort_flag, status)) break;
                unsigned char* st = smem + s * STAGE;
                mbar_expect_tx(&raw_full[s], RAW);
                tma_load_3d(st, &xmap, (kb0 + it) * TK32, m0, batch, &raw_full[s]);
                tma_load_3d(st + A_BYTES, &wmap, (kb0 + it) * TK32, n0, batch, &raw_full[s]);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_tf32(TMR, BN);
            for (int it = 0; it < nk; ++it) {
                const int s = it % STAGES;
                if (!mbar_wait_spin(&full[s], (it / STAGES) & 1, abort_flag, status)) break;
                tc_fence_after();
                unsigned char* st = smem + s * STAGE;
                const uint64_t a_hi = umma_desc_sw128(st), b_hi = umma_desc_sw128(st + A_BYTES);
                const uint64_t a_lo = umma_desc_sw128(st + RAW), b_lo = umma_desc_sw128(st + RAW + A_BYTES);
#pragma unroll
                for (int k = 0; k < TK32 / 8; ++k) {
                    // 8 f32 = 32 bytes inside the 128-byte swizzle row: +2 in 16-byte units
                    const int kk = it * (TK32 / 8) + k;
                    constexpr int MAINS = main_accs(BN), CORRS = corr_accs(BN);
                    const uint32_t corr = tmem_base + (uint32_t)((MAINS + kk % CORRS) * BN);
                    umma_tf32(corr, a_lo + 2 * k, b_hi + 2 * k, idesc, kk >= CORRS ? 1u : 0u);
                    umma_tf32(tmem_base + (uint32_t)((kk % MAINS) * BN), a_hi + 2 * k, b_hi + 2 * k, idesc, kk >= MAINS ? 1u : 0u);
                    umma_tf32(corr, a_hi + 2 * k, b_lo + 2 * k, idesc, 1u);
                }
                umma_commit(&empty[s]);
            }
            umma_commit(accum_bar);
        }
    } else if (warp < 6) {
        const int q = warp & 3;
        const bool ok = mbar_wait(accum_bar, 0, abort_flag, status);
        tc_fence_after();
        const int row = TMR == 128 ? m0 + q * 32 + lane : (lane < 16 ? m0 + q * 16 + lane : M);   // 64-row tiles: 16 rows per quarter
        if (ok) {
#pragma unroll 1
            for (int c = 0; c < BN; c += 32) {
                // main accumulators that were used (fewer than kMainAcc k-steps leave some untouched), then the small products
                constexpr int MAINS = main_accs(BN), CORRS = corr_accs(BN);
                const int ksteps = nk * (TK32 / 8);
                float v[32], t[32];
                tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c, v);
                for (int a = 1; a < min(MAINS, ksteps); ++a) {
                    tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(a * BN + c), t);
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] += t[j];
                }
                for (int a = 0; a < min(CORRS, ksteps); ++a) {
                    tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)((MAINS + a) * BN + c), t);
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] += t[j];
                }
                if (row < M) {
                    float* orow = out + (size_t)row * N + n0 + c;
                    if (bias_rows) {                 // one value per output row (the transposed product of conv1d)
                        const float br = bias_rows[row];
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] += br;
                    }
#pragma unroll
                    for (int j = 0; j < 32; j += 4) {
                        const int col = n0 + c + j;
                        if (col + 4 <= N) {
                            float4 o = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                            if (bias) {
                                const float4 b = *reinterpret_cast<const float4*>(bias + col);
                                o.x += b.x; o.y += b.y; o.z += b.z; o.w += b.w;
                            }
                            *reinterpret_cast<float4*>(orow + j) = o;
                        } else {
                            for (int e = 0; e < 4 && col + e < N; ++e) orow[j + e] = v[j + e] + (bias ? bias[col + e] : 0.f);
                        }
                    }
                }
            }
        }
    } else {
        // converting warps: raw tile (= hi as the tensor core reads it) -> lo (twin tile, same offsets)
        constexpr int CT = kConvWarps * 32;
        constexpr int VECS = RAW / 16;
        const int dt = threadIdx.x - kThreadsTc;
        for (int it = 0; it < nk; ++it) {
            const int s = it % STAGES;
            // the lanes of a warp leave together (they meet again at __syncwarp below)
            const bool arrived = __all_sync(0xffffffffu, mbar_wait_spin(&raw_full[s], (it / STAGES) & 1, abort_flag, status));
            if (!arrived) break;
            uint4* hi = reinterpret_cast<uint4*>(smem + s * STAGE);
            uint4* lo = reinterpret_cast<uint4*>(smem + s * STAGE + RAW);
#pragma unroll 4
            for (int i = dt; i < VECS; i += CT) {
                const uint4 x = hi[i];
                uint4 l;
                l.x = __float_as_uint(__uint_as_float(x.x) - __uint_as_float(x.x & 0xFFFFE000u));
                l.y = __float_as_uint(__uint_as_float(x.y) - __uint_as_float(x.y & 0xFFFFE000u));
                l.z = __float_as_uint(__uint_as_float(x.z) - __uint_as_float(x.z & 0xFFFFE000u));
                l.w = __float_as_uint(__uint_as_float(x.w) - __uint_as_float(x.w & 0xFFFFE000u));
                lo[i] = l;
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&full[s]);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "n"(512) : "memory");
    }
}

// out = sum of the `splits` partial results (in slab order) + bias per column / per row
__global__ void __launch_bounds__(256)
sum_splits_kernel(const float4* __restrict__ part, int splits, size_t slab4, const float* __restrict__ bias,
                  const float* __restrict__ bias_rows, float4* __restrict__ out, int N4) {
    rcu_kernel_entry();
    for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < slab4; i += (size_t)gridDim.x * 256) {
        float4 a = part[i];
        for (int s = 1; s < splits; ++s) {
            const float4 b = part[(size_t)s * slab4 + i];
            a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
        }
        if (bias) {
            const float4 b = reinterpret_cast<const float4*>(bias)[i % N4];
            a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
        }
        if (bias_rows) {
            const float b = bias_rows[i / N4];
            a.x += b; a.y += b; a.z += b; a.w += b;
        }
        out[i] = a;
    }
}

template <int BN, int TMR>
rcu_status launch_f32(rcu_device* dev, const CUtensorMap& xmap, const CUtensorMap& wmap, const void* bias, const void* bias_rows, void* out,
                      int M, int N, int K, int batches, int kb_per_split) {
    constexpr int STAGE = 2 * (TMR * TK32 * 4 + BN * TK32 * 4);
    constexpr int STAGES = (192 * 1024) / STAGE > 8 ? 8 : (192 * 1024) / STAGE;
    const size_t smem = (size_t)STAGES * STAGE + 1024 + 512;
    auto kern = gemm_tc_f32_kernel<BN, STAGES, TMR>;
    RCU_CUDA(dev, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid((N + BN - 1) / BN, (M + TMR - 1) / TMR, batches);
    rcu_launch(dev, kern, grid, kThreadsF32, smem, xmap, wmap, (const float*)bias, (const float*)bias_rows, (float*)out, M, N, K, kb_per_split, dev->d_status);
    RCU_LAUNCH_CHECK(dev);
    return RCU_OK;
}

rcu_status launch_f32_any(rcu_device* dev, int bn, int tmr, const CUtensorMap& xmap, const CUtensorMap& wmap, const void* bias, const void* bias_rows,
                          void* out, int M, int N, int K, int batches, int kb_per_split) {
    if (tmr == 64)
        return bn == 128 ? launch_f32<128, 64>(dev, xmap, wmap, bias, bias_rows, out, M, N, K, batches, kb_per_split)
                         : launch_f32<64, 64>(dev, xmap, wmap, bias, bias_rows, out, M, N, K, batches, kb_per_split);
    return bn == 128 ? launch_f32<128, 128>(dev, xmap, wmap, bias, bias_rows, out, M, N, K, batches, kb_per_split)
                     : launch_f32<64, 128>(dev, xmap, wmap, bias, bias_rows, out, M, N, K, batches, kb_per_split);
}

// [batches, rows, K] f32 row-major, box = 1 x box_rows x 32 elements, 128-byte swizzle
bool make_map_f32_sw128(CUtensorMap* map, const void* base, uint64_t batches, uint64_t rows, uint64_t K, uint32_t box_rows) {
    gemvq8::EncodeTiledFn fn = gemvq8::encode_tiled_fn();
    if (!fn) return false;
    cuuint64_t dims[3] = {K, rows, batches};
    cuuint64_t strides[2] = {K * 4, rows * K * 4};
    cuuint32_t box[3] = {(cuuint32_t)TK32, box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

bool rcu_gemm_tc_f32_eligible(int lhs_dt, int act_dt, uint64_t M, uint64_t N, uint64_t K) {
    if (act_dt != RCU_F32 || lhs_dt != RCU_F32) return false;
    // small problems stay on the SIMT kernel; rows must be 16-byte multiples for the tensor maps
    if (M < 32 || N < 64 || K < 32 || K % 4 != 0 || N % 4 != 0) return false;
    if (M > 0x7fffffffull || N > 0x7fffffffull || K > 0x7fffffffull) return false;
    static const bool off = [] { const char* e = std::getenv("RCU_GEMM_F32_TC"); return e && std::atoi(e) == 0; }();
    return !off;
}

rcu_status rcu_gemm_tc_f32_dispatch(rcu_device* dev, const void* w, const void* x, const void* bias, void* y, uint64_t M, uint64_t N,
                                    uint64_t K, uint64_t batches, const void* bias_rows) {
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(bias)) & 15)
        return RCU_ERR_UNSUPPORTED;
    // tensor-map strides are multiples of 16 bytes; the grid's z extent is limited
    if (batches < 1 || batches > 65535 || (batches > 1 && ((M * K) % 4 != 0 || (N * K) % 4 != 0 || (M * N) % 4 != 0 || bias || bias_rows))) return RCU_ERR_UNSUPPORTED;
    DevGuard g(dev->ordinal);
    // Tile height: 64 token rows when M fits one such tile (half of a 128-row tile would be padding).  Cutting larger
    // M into 64-row tiles to put a CTA on every SM was measured and is slower (Whisper-tiny's 1500 x 384 x 384
    // Linear and the unfolded conv1d): the weight side of a tile costs the same and is then paid twice as often.
    const uint64_t sms = (uint64_t)dev->sm_count;
    const int tmr = M <= 64 ? 64 : 128;
    // Tile width and K slices together.  A CTA spends about 0.7 us per 32-wide k-block almost regardless of the tile's
    // width (twelve small MMAs issued by one thread, the lo pass, the barrier hops between them), so what counts is
    // how many k-blocks a CTA runs one after the other and how many rounds of CTAs the grid needs; the width adds a
    // little through shared-memory traffic.  Slices of K (blockIdx.z; every slice writes a partial result to pooled
    // scratch and one pass sums the slices in order: deterministic) are taken whenever they shorten that chain, with a
    // charge for the summing pass.
    const uint64_t mt = (M + tmr - 1) / tmr, nk = (K + TK32 - 1) / TK32;
    constexpr uint64_t kMinBlocksPerSplit = 24, kFixed = 600, kSumCharge = 4;
    int bn = 64;
    uint64_t splits = 1, best = ~0ull;
    for (int cand : {64, 128}) {
        const uint64_t tiles_c = mt * ((N + cand - 1) / cand);
        const uint64_t sp_max = (batches == 1 && M * N % 4 == 0) ? std::max<uint64_t>(1, std::min<uint64_t>(8, nk / kMinBlocksPerSplit)) : 1;
        for (uint64_t sp = 1; sp <= sp_max; ++sp) {
            const uint64_t kbps_c = (nk + sp - 1) / sp;
            const uint64_t rounds = (tiles_c * sp * batches + sms - 1) / sms;
            const uint64_t cost = (rounds * kbps_c + (sp > 1 ? kSumCharge : 0)) * (kFixed + (uint64_t)(tmr + cand));
            if (cost < best) { best = cost; bn = cand; splits = sp; }
        }
    }
    CUtensorMap xmap, wmap;
    if (!make_map_f32_sw128(&xmap, x, batches, M, K, (uint32_t)tmr) || !make_map_f32_sw128(&wmap, w, batches, N, K, (uint32_t)bn))
        return rcu_fail(dev, RCU_ERR_CUDA, "gemm_tc_f32: cuTensorMapEncodeTiled failed (M=%llu N=%llu K=%llu x%llu)", (unsigned long long)M,
                        (unsigned long long)N, (unsigned long long)K, (unsigned long long)batches);
    if (splits > 1 && M * N % 4 == 0) {
        const uint64_t kbps = (nk + splits - 1) / splits;
        splits = (nk + kbps - 1) / kbps;
        void* part = nullptr;
        rcu_status st = rcu_alloc(dev, splits * M * N * 4, &part);
        if (st != RCU_OK) return st;
        st = launch_f32_any(dev, bn, tmr, xmap, wmap, nullptr, nullptr, part, (int)M, (int)N, (int)K, (int)splits, (int)kbps);
        if (st == RCU_OK) {
            const size_t slab4 = (size_t)(M * N / 4);
            const int grid = (int)std::min<size_t>((slab4 + 255) / 256, (size_t)dev->sm_count * 8);
            rcu_launch(dev, sum_splits_kernel, grid, 256, 0, (const float4*)part, (int)splits, slab4, (const float*)bias, (const float*)bias_rows,
                                                             (float4*)y, (int)(N / 4));
            RCU_LAUNCH_CHECK(dev);
        }
        rcu_free(dev, part);      // the pool reuses blocks in stream order
        return st;
    }
    return launch_f32_any(dev, bn, tmr, xmap, wmap, bias, bias_rows, y, (int)M, (int)N, (int)K, (int)batches, 0);
}
