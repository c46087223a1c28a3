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
// Quantised weights (Q8_0H, Q4_KH) are dequantised to f16 first by rcu_dequantize (bit-exact with
// the CPU dequantiser) into pooled scratch and then take the same path.
//
// Every mbarrier wait is bounded; a wait that gives up sets RCU_DEVFLAG_TIMEOUT and an abort word in
// shared memory that ends all other waits of the CTA, and the CTA still frees its tensor memory.
#include <cuda.h>

#include "gemv_q8_bulk.cuh"   // mbarrier + tensor-map helpers

namespace {

using gemvq8::mbar_arrive;
using gemvq8::mbar_expect_tx;
using gemvq8::mbar_init;
using gemvq8::mbar_wait;
using gemvq8::smem_u32;
using gemvq8::tma_load_2d;

constexpr int TM = 128;          // tokens per tile (UMMA M)
constexpr int TK = 64;           // K per stage: 64 f16 = 128 bytes = one swizzle row
constexpr int kStages = 4;
constexpr int kThreadsTc = 192;  // 6 warps

// 64-bit shared-memory matrix descriptor, K-major operand, 128-byte swizzle:
// rows of 128 bytes, 8-row groups 1024 bytes apart (SBO), descriptor version 1 (sm_100).
__device__ __forceinline__ uint64_t umma_desc_sw128(const void* smem_ptr) {
    const uint32_t addr = smem_u32(smem_ptr);
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFF) >> 4);            // start address, 16-byte units
    d |= (uint64_t)0 << 16;                            // leading byte offset: unused for swizzled K-major
    d |= (uint64_t)(1024 >> 4) << 32;                  // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                            // descriptor version
    d |= (uint64_t)2 << 61;                            // SWIZZLE_128B
    return d;
}

// 32-bit instruction descriptor, kind::f16: f16 A and B (both K-major), f32 D, M x N tile.
__host__ __device__ constexpr uint32_t umma_idesc_f16(int m, int n) {
    return (1u << 4)                      // D format f32
           | (0u << 7) | (0u << 10)       // A, B format f16
           | (0u << 15) | (0u << 16)      // A, B K-major
           | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// arrive on `bar` once every tcgen05.mma issued so far by this thread has finished
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// 32 lanes x 32 consecutive f32 columns of tensor memory -> 32 registers per thread
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, float* v) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

}  // namespace

namespace {

template <int BN>
__global__ void __launch_bounds__(kThreadsTc, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap xmap, const __grid_constant__ CUtensorMap wmap, const __half* __restrict__ bias,
               __half* __restrict__ out, int M, int N, int K, int* status) {
    constexpr int A_BYTES = TM * TK * 2;          // 16 KiB
    constexpr int B_BYTES = BN * TK * 2;
    constexpr int STAGE = A_BYTES + B_BYTES;
    extern __shared__ unsigned char smem_dyn[];
    // 1024-byte alignment: the 128-byte swizzle pattern repeats every 8 rows = 1024 bytes
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + kStages * STAGE);
    uint64_t* empty = full + kStages;
    uint64_t* accum_bar = empty + kStages;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum_bar + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.y * TM, n0 = blockIdx.x * BN;
    const int nk = (K + TK - 1) / TK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
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
                const int s = it % kStages;
                if (it >= kStages && !mbar_wait(&empty[s], ((it / kStages) - 1) & 1, abort_flag, status)) break;
                mbar_expect_tx(&full[s], STAGE);
                unsigned char* st = smem + s * STAGE;
                tma_load_2d(st, &xmap, it * TK, m0, &full[s]);             // activations: rows m0.., k it*64..
                tma_load_2d(st + A_BYTES, &wmap, it * TK, n0, &full[s]);   // weights: rows n0..
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_f16(TM, BN);
            bool ok = true;
            for (int it = 0; it < nk && ok; ++it) {
                const int s = it % kStages;
                ok = mbar_wait(&full[s], (it / kStages) & 1, abort_flag, status);
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
    } else {
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
                if (row < M) {
                    __half* orow = out + (size_t)row * N + n0 + c;
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
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "n"(BN) : "memory");
    }
}

template <int BN>
rcu_status launch_tc(rcu_device* dev, const CUtensorMap& xmap, const CUtensorMap& wmap, const void* bias, void* out, int M, int N, int K) {
    const size_t smem = (size_t)kStages * (TM * TK * 2 + BN * TK * 2) + 1024 + 256;
    auto kern = gemm_tc_kernel<BN>;
    RCU_CUDA(dev, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid((N + BN - 1) / BN, (M + TM - 1) / TM);
    kern<<<grid, kThreadsTc, smem, dev->stream>>>(xmap, wmap, (const __half*)bias, (__half*)out, M, N, K, dev->d_status);
    RCU_LAUNCH_CHECK(dev);
    return RCU_OK;
}

// [rows, K] f16 row-major, box = box_rows x 64 elements, 128-byte swizzle
bool make_map_f16_sw128(CUtensorMap* map, const void* base, uint64_t rows, uint64_t K, uint32_t box_rows) {
    gemvq8::EncodeTiledFn fn = gemvq8::encode_tiled_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {K, rows};
    cuuint64_t strides[1] = {K * 2};
    cuuint32_t box[2] = {(cuuint32_t)TK, box_rows};
    cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
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

rcu_status rcu_gemm_tc_dispatch(rcu_device* dev, int lhs_dt, const void* w, int act_dt, const void* x, const void* bias, void* y,
                                uint64_t M, uint64_t N, uint64_t K) {
    if (!rcu_gemm_tc_eligible(lhs_dt, act_dt, M, N, K)) return RCU_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(w)) & 15) return RCU_ERR_UNSUPPORTED;
    DevGuard g(dev->ordinal);
    const void* wf16 = w;
    void* scratch = nullptr;
    if (lhs_dt != RCU_F16) {
        // dequantise to f16 (bit-exact with quant.rs / quantized.rs arithmetic) into pooled scratch
        rcu_status st = rcu_alloc(dev, N * K * 2, &scratch);
        if (st != RCU_OK) return st;
        rcu_tensor src{lhs_dt, 2, {N, K, 1, 1}, const_cast<void*>(w)};
        rcu_tensor dst{RCU_F16, 2, {N, K, 1, 1}, scratch};
        st = rcu_dequantize(dev, &src, &dst);
        if (st != RCU_OK) { rcu_free(dev, scratch); return st; }
        wf16 = scratch;
    }
    // tile width: enough CTAs to cover the SMs when M is small
    const uint64_t tiles128 = ((M + TM - 1) / TM) * ((N + 127) / 128);
    const int bn = tiles128 >= (uint64_t)dev->sm_count ? 128 : 64;
    CUtensorMap xmap, wmap;
    rcu_status st = RCU_OK;
    if (!make_map_f16_sw128(&xmap, x, M, K, TM) || !make_map_f16_sw128(&wmap, wf16, N, K, (uint32_t)bn))
        st = rcu_fail(dev, RCU_ERR_CUDA, "gemm_tc: cuTensorMapEncodeTiled failed (M=%llu N=%llu K=%llu)", (unsigned long long)M,
                      (unsigned long long)N, (unsigned long long)K);
    if (st == RCU_OK) st = bn == 128 ? launch_tc<128>(dev, xmap, wmap, bias, y, (int)M, (int)N, (int)K)
                                     : launch_tc<64>(dev, xmap, wmap, bias, y, (int)M, (int)N, (int)K);
    // the pool reuses blocks in stream order, so the scratch can go back right after the launch
    if (scratch) rcu_free(dev, scratch);
    return st;
}
