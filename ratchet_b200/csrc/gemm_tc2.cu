// Prefill GEMM on CTA pairs (tcgen05 cta_group::2), Linear convention:
//   out[M, N] = X[M, K] . W[N, K]^T (+ bias),  X, W and out f16, f32 accumulation in tensor memory.
//
// Same contract as gemm_tc_kernel (ops/matmul/gemm.rs:462-746 is what it stands in for); used for
// f16 weights when the problem has at least a few 256 x 256 tiles.  A 128 x 256 x 16 MMA of one CTA
// reads 12 KiB of operands from shared memory in the 128 cycles it takes, and TMA writes the same
// amount: together more than the 128 bytes per cycle an SM's shared memory moves, which is what held
// the one-CTA kernel near two thirds of the tensor rate.  Here two CTAs of a cluster compute one
// 256 x 256 tile: each holds 128 token rows of X and 128 of the tile's 256 weight rows, the pair's
// tensor cores exchange the weight halves, and every CTA reads and writes 8 KiB per MMA.
//
//   warp 0 (one lane)  TMA producer: its CTA's 128 x 64 X tile and 128 x 64 W tile per stage, completion
//                      counted on the LEADER CTA's `full` barrier (the leader expects both CTAs' bytes);
//   warp 1 (one lane, leader CTA only)  issues four tcgen05.mma.cta_group::2 per stage and commits them
//                      to the stage's `empty` barrier of both CTAs, and at the end of a tile to both CTAs'
//                      `acc_full` barrier;
//   warps 2-5          epilogue of the CTA's own 128 rows: tcgen05.ld, bias, f16, 16-byte stores; then
//                      one arrival per warp on the leader's `acc_empty` barrier.
// The kernel is persistent: a pair walks over tiles pair, pair + n_pairs, ...; the accumulator is
// double-buffered (2 x 256 of the 512 tensor-memory columns), so the epilogue of tile i overlaps the
// MMAs of tile i + 1.  Tiles that share a weight tile run on neighbouring pairs at the same time (the
// activations, M x K, stay in L2).
//
// Every wait is bounded (mbar_wait); a wait that gives up raises RCU_DEVFLAG_TIMEOUT and ends the
// CTA's other waits through a flag in shared memory.  Both CTAs meet at a cluster barrier before tensor
// memory is freed, so neither touches the other's shared memory after it has exited.
#include <cuda.h>

#include "tc_common.cuh"

namespace {

using namespace tc;

constexpr int kStages2 = 6;
constexpr int kTileN2 = 256;                       // weight rows per pair tile (128 per CTA)
constexpr int kStageBytes2 = 2 * TM * TK * 2;      // 128 x 64 f16 of X + 128 x 64 f16 of W = 32 KiB
constexpr int kAccCols = 256;                      // f32 accumulator columns per buffer

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// address of `local` (a shared-memory address of this CTA) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// TMA tile load whose completion is counted on a barrier that may live in the peer CTA
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, int x, int y, uint32_t bar_cluster_addr) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
            smem_u32(dst)),
        "l"(map), "r"(x), "r"(y), "r"(bar_cluster_addr)
        : "memory");
}
__device__ __forceinline__ void umma2_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// arrive on the barrier at this shared-memory offset in both CTAs of the pair once every MMA issued so far is done
__device__ __forceinline__ void umma2_commit_both(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(smem_u32(bar)),
                 "h"((uint16_t)3)
                 : "memory");
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreadsTc, 1)
gemm_tc2_kernel(const __grid_constant__ CUtensorMap xmap, const __grid_constant__ CUtensorMap wmap, const __half* __restrict__ bias,
                __half* __restrict__ out, int M, int N, int K, int tiles_m, int n_tiles, int* status) {
    extern __shared__ unsigned char smem_dyn[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + kStages2 * kStageBytes2);   // leader's are the ones in use
    uint64_t* empty = full + kStages2;
    uint64_t* acc_full = empty + kStages2;        // [2]
    uint64_t* acc_empty = acc_full + 2;           // [2], leader's in use
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();                 // 0 = leader
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const int nk = (K + TK - 1) / TK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages2; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 8);           // four epilogue warps in each CTA
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "n"(2 * kAccCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    cluster_sync_all();            // barriers of both CTAs initialised before anyone signals them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            int it = 0;
            bool ok = true;
            for (int t = pair; t < n_tiles && ok; t += n_pairs) {
                const int m0 = (t % tiles_m) * 2 * TM + (int)rank * TM;
                const int n0 = (t / tiles_m) * kTileN2 + (int)rank * (kTileN2 / 2);
                for (int k = 0; k < nk; ++k, ++it) {
                    const int s = it % kStages2;
                    if (it >= kStages2 && !mbar_wait(&empty[s], ((it / kStages2) - 1) & 1, abort_flag, status)) { ok = false; break; }
                    unsigned char* st = smem + s * kStageBytes2;
                    if (rank == 0) mbar_expect_tx(&full[s], 2 * kStageBytes2);      // both CTAs' bytes
                    const uint32_t bar = map_to_cta(smem_u32(&full[s]), 0);
                    tma_load_2d_pair(st, &xmap, k * TK, m0, bar);
                    tma_load_2d_pair(st + TM * TK * 2, &wmap, k * TK, n0, bar);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc = umma_idesc_f16(2 * TM, kTileN2);
            int it = 0, i = 0;
            bool ok = true;
            for (int t = pair; t < n_tiles && ok; t += n_pairs, ++i) {
                const int b = i & 1;
                if (i >= 2) {
                    ok = mbar_wait(&acc_empty[b], ((i >> 1) - 1) & 1, abort_flag, status);
                    if (!ok) break;
                    tc_fence_after();
                }
                const uint32_t acc = tmem_base + (uint32_t)(b * kAccCols);
                for (int k = 0; k < nk; ++k, ++it) {
                    const int s = it % kStages2;
                    ok = mbar_wait(&full[s], (it / kStages2) & 1, abort_flag, status);
                    if (!ok) break;
                    tc_fence_after();
                    unsigned char* st = smem + s * kStageBytes2;
                    const uint64_t adesc = umma_desc_sw128(st);
                    const uint64_t bdesc = umma_desc_sw128(st + TM * TK * 2);
#pragma unroll
                    for (int kk = 0; kk < TK / 16; ++kk) umma2_f16(acc, adesc + 2 * kk, bdesc + 2 * kk, idesc, (k > 0 || kk > 0) ? 1u : 0u);
                    umma2_commit_both(&empty[s]);
                }
                umma2_commit_both(&acc_full[b]);      // also after an abort, so that the epilogues end
            }
        }
    } else {
        // epilogue warps 2..5: tensor-memory lane quarter = warp index modulo 4
        const int q = warp & 3;
        const uint32_t acc_empty_leader0 = map_to_cta(smem_u32(&acc_empty[0]), 0);
        int i = 0;
        bool ok = true;
        for (int t = pair; t < n_tiles && ok; t += n_pairs, ++i) {
            const int b = i & 1;
            ok = mbar_wait(&acc_full[b], (i >> 1) & 1, abort_flag, status);
            if (!ok) break;
            tc_fence_after();
            const int row = (t % tiles_m) * 2 * TM + (int)rank * TM + q * 32 + lane;
            const int n0 = (t / tiles_m) * kTileN2;
#pragma unroll 1
            for (int c = 0; c < kTileN2; c += 32) {
                float v[32];
                tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(b * kAccCols + c), v);
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
            // this warp has read its part of the buffer: tell the leader's MMA thread
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(acc_empty_leader0 + (uint32_t)(b * 8));
        }
    }
    tc_fence_before();
    cluster_sync_all();            // the peer may still be signalling barriers in this CTA's shared memory
    tc_fence_after();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "n"(2 * kAccCols) : "memory");
    }
}

bool make_map_f16_sw128_rows(CUtensorMap* map, const void* base, uint64_t rows, uint64_t K, uint32_t box_rows) {
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

// f16 x f16 problems with at least `min_tiles` 256 x 256 tiles take the CTA-pair kernel
bool rcu_gemm_tc2_eligible(rcu_device* dev, uint64_t M, uint64_t N, uint64_t K) {
    static const int mode = [] { const char* e = getenv("RCU_GEMM_PAIR"); return e ? atoi(e) : 1; }();
    if (mode == 0) return false;
    if (M < 256 || N < 256 || K < 64 || K % 8 != 0 || N % 8 != 0) return false;
    const uint64_t tiles = ((M + 255) / 256) * ((N + 255) / 256);
    return tiles >= (uint64_t)dev->sm_count / 4;
}

rcu_status rcu_gemm_tc2_launch(rcu_device* dev, const void* w, const void* x, const void* bias, void* y, uint64_t M, uint64_t N, uint64_t K) {
    CUtensorMap xmap, wmap;
    if (!make_map_f16_sw128_rows(&xmap, x, M, K, TM) || !make_map_f16_sw128_rows(&wmap, w, N, K, kTileN2 / 2))
        return rcu_fail(dev, RCU_ERR_CUDA, "gemm_tc2: cuTensorMapEncodeTiled failed (M=%llu N=%llu K=%llu)", (unsigned long long)M,
                        (unsigned long long)N, (unsigned long long)K);
    const int tiles_m = (int)((M + 255) / 256), tiles_n = (int)((N + 255) / 256);
    const int n_tiles = tiles_m * tiles_n;
    const int n_pairs = std::min(n_tiles, dev->sm_count / 2);
    const size_t smem = (size_t)kStages2 * kStageBytes2 + 1024 + 256;
    RCU_CUDA(dev, cudaFuncSetAttribute(gemm_tc2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    gemm_tc2_kernel<<<2 * n_pairs, kThreadsTc, smem, dev->stream>>>(xmap, wmap, (const __half*)bias, (__half*)y, (int)M, (int)N, (int)K, tiles_m,
                                                                  n_tiles, dev->d_status);
    RCU_LAUNCH_CHECK(dev);
    return RCU_OK;
}
