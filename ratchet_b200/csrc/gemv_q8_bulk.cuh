// Q8_0 GEMV with the weights staged through shared memory by TMA tile copies.
//
// Same contract as gemv_q8_kernel (gemv_q8.cuh): y = W[N,K] . x with ratchet Q8_0 segments, a
// Prologue that stages x and an Epilogue that stores units — but the bytes in flight no longer live
// in registers.  A producer warp issues `cp.async.bulk.tensor.2d` copies (boxes of 4 weight rows x
// 1 KiB, and the matching 4 x 32 block scales) into a ring of shared-memory stages of 16 rows, each
// stage guarded by a pair of mbarriers (full: transaction bytes counted by the copy engine; empty:
// one arrival per consumer warp).  Eight consumer warps own two weight rows each and read their
// 16-byte chunks back with conflict-free LDS.128.
//
// Inner product: the staged f16 activations are re-expressed once per CTA as 16-bit fixed point per
// 32-element block, x = s_b * (256 * hi + lo) with `hi` a signed and `lo` an unsigned byte plane, so
// the product with the int8 weights is two dp4a instructions per four weights with exact integer
// sums and no int8 -> float conversion.  Rounding x to 16 bits relative to its block maximum
// (2^-16) is 32 times finer than the activations' own f16 precision (2^-11).
//
// Why a ring in shared memory: HBM needs ~35 KB in flight per SM.  Held in registers that costs
// occupancy; held in shared memory it costs one CTA per SM and ~90 KB, the loads no longer depend
// on how fast the consumers issue, and there is room for the NEXT kernel's CTA to become resident
// under programmatic dependent launch and fill its own ring with weights while this kernel drains —
// a decode step is a chain of short GEMVs, so each one's ramp-up hides behind its predecessor's tail.
// Why tile copies: the copy engine spends roughly the same ~40 ns on a bulk copy whatever its size,
// so per-row 1 KiB copies (plus 128-byte scale copies) cap an SM near 16 GB/s; 4 KiB boxes do not.
//
// Requirements (checked by the launcher, which otherwise uses the register kernel): K % 1024 == 0,
// K <= 16384, 16-byte aligned base pointers.  Every wait on an mbarrier is bounded; a wait that gives
// up raises RCU_DEVFLAG_TIMEOUT in the device status word, tells the rest of the CTA through shared
// memory, and the CTA's warps return.
#pragma once
#include <cuda.h>

#include "gemv_q8.cuh"

namespace gemvq8 {

constexpr int kBulkConsumerWarps = 8;
constexpr int kBulkThreads = (kBulkConsumerWarps + 1) * 32;   // + one producer warp
constexpr int kBulkRowsPerWarp = 2;
constexpr int kBulkStageRows = kBulkConsumerWarps * kBulkRowsPerWarp;   // 16
constexpr int kBulkBoxRows = 4;
constexpr int kBulkBoxes = kBulkStageRows / kBulkBoxRows;      // 4 boxes per stage
constexpr int kBulkKC = 1024;                                  // bytes of one row per stage
constexpr int kBulkStages = 6;
constexpr unsigned kBulkSpinLimit = 1u << 22;                  // polls of try_wait (each may block in hardware)

template <class ScaleT> constexpr int bulk_stage_bytes() {
    return kBulkStageRows * kBulkKC + kBulkStageRows * (kBulkKC / 32) * (int)sizeof(ScaleT);
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Non-blocking probe of the phase (try_wait may suspend the thread for a hardware-chosen time slice
// before it answers; a pipeline whose stages hand over through several barriers pays that on every hop).
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// bounded busy wait for latency-critical hand-overs; same contract as mbar_wait
__device__ __forceinline__ bool mbar_wait_spin(uint64_t* bar, unsigned parity, volatile int* abort_flag, int* status) {
    unsigned long long t0 = 0;
    for (unsigned i = 0;; ++i) {
        if (mbar_test_wait(bar, parity)) return true;
        if ((i & 255u) == 255u) {
            if (*abort_flag) return false;
            unsigned long long t;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
            if (t0 == 0) t0 = t;
            else if (t - t0 > 1000000000ull) break;
        }
    }
    *abort_flag = 1;
    atomicOr(status, RCU_DEVFLAG_TIMEOUT);
    return false;
}
// bounded wait; returns false if it gave up (or another thread of the CTA already did)
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, unsigned parity, volatile int* abort_flag, int* status) {
    unsigned long long t0 = 0;
    for (unsigned i = 0; i < kBulkSpinLimit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if ((i & 1023u) == 1023u) {     // also bound the wait in wall time: one second
            unsigned long long t;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
            if (t0 == 0) t0 = t;
            else if (t - t0 > 1000000000ull) break;
        }
    }
    *abort_flag = 1;
    atomicOr(status, RCU_DEVFLAG_TIMEOUT);
    return false;
}
// dp4a_ss / dp4a_su (signed x signed, signed x unsigned byte dot products) come from gemv_q8.cuh
// 2-D tile: global (tensor map, element coordinates x = innermost, y = row) -> shared, completion in
// bytes on `bar`.  x * element size must be a multiple of 16 bytes (here x = kc * 256 u32 / kc * 32 scales).
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                     smem_u32(dst)),
                 "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
                 : "memory");
}
// 3-D tile (x = innermost, y = row, z = batch) -> shared, completion on `bar`
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, int x, int y, int z, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(
                     smem_u32(dst)),
                 "l"(map), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar))
                 : "memory");
}

template <class ScaleT, class Prologue, class Epilogue>
__global__ void __launch_bounds__(kBulkThreads, 1)
gemv_q8_bulk_kernel(const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap smap, Prologue pro, Epilogue epi,
                    int n_units, int unit_stride, int K, int* status) {
    constexpr int UNIT = Epilogue::UNIT;                 // 1: a warp owns two units; 2: a warp owns one (gate, up) pair
    constexpr int UG = kBulkStageRows / UNIT;            // units per stage group (16 or 8)
    constexpr int STAGE = bulk_stage_bytes<ScaleT>();
    constexpr int SCB = (kBulkKC / 32) * (int)sizeof(ScaleT);   // scale bytes per row per stage
    constexpr unsigned BOX_BYTES = kBulkBoxRows * (kBulkKC + SCB);
    extern __shared__ __align__(128) unsigned char smem_raw[];
    unsigned char* stages = smem_raw;
    __half* xs = reinterpret_cast<__half*>(smem_raw + kBulkStages * STAGE);
    float* red = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(xs) + (size_t)K * sizeof(__half));   // kWarps floats
    uint64_t* full = reinterpret_cast<uint64_t*>(red + 16);
    uint64_t* empty = full + kBulkStages;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(empty + kBulkStages);
    float* xsc = reinterpret_cast<float*>(const_cast<int*>(abort_flag) + 4);   // [K/32] block scales of x

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // units are dealt in quads (one tile box = 4 rows) so no CTA loads rows that belong to another
    const int n_quads = (n_units + kBulkBoxRows - 1) / kBulkBoxRows;
    const int u_begin = (int)(((long long)blockIdx.x * n_quads) / gridDim.x) * kBulkBoxRows;
    const int u_end = min(n_units, (int)(((long long)(blockIdx.x + 1) * n_quads) / gridDim.x) * kBulkBoxRows);
    const int n_groups = u_end > u_begin ? (u_end - u_begin + UG - 1) / UG : 0;
    const int nkc = K / kBulkKC;
    const int n_iters = n_groups * nkc;

    if (tid == 0) {
        for (int s = 0; s < kBulkStages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], kBulkConsumerWarps);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    pdl_launch_dependents();

    if (warp == kBulkConsumerWarps) {
        // ------------------------------------------------------------------ producer warp
        // Weights never depend on the previous kernel: start filling the ring at once.
        for (int it = 0; it < n_iters; ++it) {
            const int s = it % kBulkStages;
            const int g = it / nkc, kc = it - g * nkc;
            if (it >= kBulkStages) {
                if (!mbar_wait(&empty[s], ((it / kBulkStages) - 1) & 1, abort_flag, status)) break;
            }
            // box b of the stage: UNIT 1 -> units u0 + 4b .. +3 (rows = units);
            // UNIT 2 -> b = 0,1: gate rows of units u0 + 4b .. +3; b = 2,3: their up rows (+ unit_stride)
            const int u0 = u_begin + g * UG;
            const int b = lane;
            const int bu = UNIT == 1 ? u0 + kBulkBoxRows * b : u0 + kBulkBoxRows * (b & 1);
            const bool valid = b < kBulkBoxes && bu < u_end;
            const unsigned nvalid = __popc(__ballot_sync(0xffffffffu, valid));
            if (lane == 0) mbar_expect_tx(&full[s], nvalid * BOX_BYTES);
            __syncwarp();
            if (valid) {
                const int row = UNIT == 1 ? bu : bu + (b >> 1) * unit_stride;
                unsigned char* st = stages + (size_t)s * STAGE;
                tma_load_2d(st + b * kBulkBoxRows * kBulkKC, &wmap, kc * (kBulkKC / 4), row, &full[s]);
                tma_load_2d(st + kBulkStageRows * kBulkKC + b * kBulkBoxRows * SCB, &smap, kc * (kBulkKC / 32), row, &full[s]);
            }
        }
        // Every issued stage is waited for by the consumer warps before they leave, and the CTA's
        // shared memory stays allocated until all of its warps have exited.
        return;
    }

    // ---------------------------------------------------------------------- consumer warps
    pdl_wait();
    // stage x with the 256 consumer threads (named barrier 1: the producer warp does not take part)
    static_assert(kBulkConsumerWarps * 32 == kThreads, "prologues stage with kThreads threads");
    pro.stage(xs, K, red);
    asm volatile("bar.sync 1, %0;" ::"n"(kBulkConsumerWarps * 32) : "memory");
    // f16 staging -> byte planes in place: hi at bytes [0,K), lo at [K,2K) of the same buffer
    int8_t* xhi = reinterpret_cast<int8_t*>(xs);
    uint8_t* xlo = reinterpret_cast<uint8_t*>(xs) + K;
    {
        constexpr int NB = 2;                                // blocks per thread: K <= 256 * 32 * NB
        uint4 raw[NB][4];
#pragma unroll
        for (int b = 0; b < NB; ++b) {
            const int blk = tid + b * kThreads;
            if (blk * 32 < K) {
#pragma unroll
                for (int v = 0; v < 4; ++v) raw[b][v] = *reinterpret_cast<const uint4*>(xs + blk * 32 + v * 8);
            }
        }
        asm volatile("bar.sync 1, %0;" ::"n"(kBulkConsumerWarps * 32) : "memory");   // all reads done before planes overwrite
#pragma unroll
        for (int b = 0; b < NB; ++b) {
            const int blk = tid + b * kThreads;
            if (blk * 32 < K) {
                const __half2* h = reinterpret_cast<const __half2*>(&raw[b][0]);
                float mx = 0.f;
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float2 f = __half22float2(h[i]);
                    mx = fmaxf(mx, fmaxf(fabsf(f.x), fabsf(f.y)));
                }
                const bool finite = mx > 0.f && mx < INFINITY;
                const float inv = finite ? 32767.f / mx : 0.f;
                xsc[blk] = finite ? mx / 32767.f : 0.f;
                uint32_t hi[8], lo[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    uint32_t hw = 0, lw = 0;
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const float2 f = __half22float2(h[2 * i + e]);
                        const int a = __float2int_rn(f.x * inv), c = __float2int_rn(f.y * inv);
                        hw |= (uint32_t)((a >> 8) & 0xFF) << (16 * e) | (uint32_t)((c >> 8) & 0xFF) << (16 * e + 8);
                        lw |= (uint32_t)(a & 0xFF) << (16 * e) | (uint32_t)(c & 0xFF) << (16 * e + 8);
                    }
                    hi[i] = hw;
                    lo[i] = lw;
                }
                uint4* ph = reinterpret_cast<uint4*>(xhi + blk * 32);
                uint4* pl = reinterpret_cast<uint4*>(xlo + blk * 32);
                ph[0] = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                ph[1] = make_uint4(hi[4], hi[5], hi[6], hi[7]);
                pl[0] = make_uint4(lo[0], lo[1], lo[2], lo[3]);
                pl[1] = make_uint4(lo[4], lo[5], lo[6], lo[7]);
            }
        }
        asm volatile("bar.sync 1, %0;" ::"n"(kBulkConsumerWarps * 32) : "memory");
    }

    // stage rows of this warp: UNIT 1 -> rows 2w, 2w+1 (units u0 + 2w, +1); UNIT 2 -> gate row w, up row 8 + w (unit u0 + w)
    const int r0 = UNIT == 1 ? warp * 2 : warp;
    const int r1 = UNIT == 1 ? warp * 2 + 1 : kBulkStageRows / 2 + warp;
    float acc[kBulkRowsPerWarp] = {0.f, 0.f};
    for (int it = 0; it < n_iters; ++it) {
        const int s = it % kBulkStages;
        const int g = it / nkc, kc = it - g * nkc;
        if (!mbar_wait(&full[s], (it / kBulkStages) & 1, abort_flag, status)) break;
        const unsigned char* st = stages + (size_t)s * STAGE;
        const int unit0 = u_begin + g * UG + (UNIT == 1 ? warp * 2 : warp);
        if (unit0 < u_end) {
#pragma unroll
            for (int c = 0; c < kBulkKC / 512; ++c) {
                const int kk = c * 512 + lane * 16;
                const int k = kc * kBulkKC + kk;
                const uint4 h4 = *reinterpret_cast<const uint4*>(xhi + k);
                const uint4 l4 = *reinterpret_cast<const uint4*>(xlo + k);
                const float xs_b = xsc[k >> 5];
#pragma unroll
                for (int j = 0; j < kBulkRowsPerWarp; ++j) {
                    const int r = j == 0 ? r0 : r1;
                    const uint4 w = *reinterpret_cast<const uint4*>(st + r * kBulkKC + kk);
                    const ScaleT sc = *reinterpret_cast<const ScaleT*>(st + kBulkStageRows * kBulkKC + r * SCB + (kk >> 5) * sizeof(ScaleT));
                    int ah = 0, al = 0;
                    ah = dp4a_ss(w.x, h4.x, ah); al = dp4a_su(w.x, l4.x, al);
                    ah = dp4a_ss(w.y, h4.y, ah); al = dp4a_su(w.y, l4.y, al);
                    ah = dp4a_ss(w.z, h4.z, ah); al = dp4a_su(w.z, l4.z, al);
                    ah = dp4a_ss(w.w, h4.w, ah); al = dp4a_su(w.w, l4.w, al);
                    acc[j] = fmaf((float)(ah * 256 + al), to_f32<ScaleT>(sc) * xs_b, acc[j]);
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);
        if (kc == nkc - 1) {
#pragma unroll
            for (int j = 0; j < kBulkRowsPerWarp; ++j) acc[j] = warp_sum(acc[j]);
            if (lane == 0) {
                if (UNIT == 1) {
#pragma unroll
                    for (int j = 0; j < kBulkRowsPerWarp; ++j)
                        if (unit0 + j < u_end) epi.store(unit0 + j, &acc[j]);
                } else if (unit0 < u_end) {
                    epi.store(unit0, acc);
                }
            }
            acc[0] = acc[1] = 0.f;
        }
    }
}

inline bool bulk_eligible(const void* w, int K, size_t smem_optin, size_t scale_size) {
    if (K % kBulkKC != 0 || K > 16384) return false;
    if (reinterpret_cast<uintptr_t>(w) & 15) return false;
    const size_t stage = (size_t)kBulkStageRows * kBulkKC + (size_t)kBulkStageRows * (kBulkKC / 32) * scale_size;
    return kBulkStages * stage + (size_t)K * 2 + (size_t)K / 8 + 256 <= smem_optin;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return (EncodeTiledFn)p;
    }();
    return fn;
}

// rows x row_bytes matrix viewed as `esize`-byte elements; box = box_rows x box_inner elements
inline bool make_map_2d(CUtensorMap* map, CUtensorMapDataType dt, size_t esize, const void* base, uint64_t rows, uint64_t row_bytes,
                        uint32_t box_inner, uint32_t box_rows) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {row_bytes / esize, rows};
    cuuint64_t strides[1] = {row_bytes};
    cuuint32_t box[2] = {box_inner, box_rows};
    cuuint32_t estr[2] = {1, 1};
    return fn(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
              CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <class ScaleT, class Prologue, class Epilogue>
rcu_status launch_bulk(rcu_device* dev, const int8_t* qs, const void* scales, const Prologue& pro, const Epilogue& epi, int N, int K,
                       bool overlap) {
    constexpr int UNIT = Epilogue::UNIT;
    const int n_units = N / UNIT;
    CUtensorMap wmap, smap;
    const bool half_scales = sizeof(ScaleT) == 2;
    if (!make_map_2d(&wmap, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, qs, (uint64_t)N, (uint64_t)K, kBulkKC / 4, kBulkBoxRows) ||
        !make_map_2d(&smap, half_scales ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, sizeof(ScaleT), scales,
                     (uint64_t)N, (uint64_t)(K / 32) * sizeof(ScaleT), kBulkKC / 32, kBulkBoxRows))
        return rcu_fail(dev, RCU_ERR_CUDA, "gemv: cuTensorMapEncodeTiled failed for a %d x %d weight", N, K);
    const size_t smem = (size_t)kBulkStages * bulk_stage_bytes<ScaleT>() + (size_t)K * sizeof(__half) + 16 * sizeof(float) +
                        2 * kBulkStages * sizeof(uint64_t) + 16 + (size_t)(K / 32) * sizeof(float);
    auto kern = gemv_q8_bulk_kernel<ScaleT, Prologue, Epilogue>;
    RCU_CUDA(dev, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    RCU_CUDA(dev, cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
    // one CTA per SM; fewer when there is less than one stage group of units per SM
    const int per_cta = kBulkStageRows / UNIT;
    int grid = (n_units + per_cta - 1) / per_cta;
    if (grid > dev->sm_count) grid = dev->sm_count;
    if (grid < 1) grid = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kBulkThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = dev->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = overlap ? 1 : 0;
    RCU_CUDA(dev, cudaLaunchKernelEx(&cfg, kern, wmap, smap, pro, epi, n_units, N / UNIT, K, dev->d_status));
    RCU_LAUNCH_CHECK(dev);
    return RCU_OK;
}

}  // namespace gemvq8
