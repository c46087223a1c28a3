// Q8_0 GEMV with the weight stream staged through per-warp rings of shared memory.
//
// y[N] = W[N,K] . x[K] on ratchet's Q8_0 segments, as gemv_q8.cuh, but the bytes in flight live in
// shared memory instead of registers.  One CTA per SM, eight warps, and every warp is its own
// producer and consumer:
//   * a warp owns D slots of S bytes and one mbarrier per slot; lane 0 requests an item — a few whole
//     weight rows (or one K-chunk of a long row) plus their block scales — with 1-D bulk copies
//     (cp.async.bulk, completion counted in bytes on the slot's barrier; no tensor maps, no multicast);
//   * the warp waits for the oldest slot, multiplies it with the activation planes (dp4a on 16-bit
//     fixed point with 16-element scales, see gemv_q8.cuh) straight out of shared memory, and lane 0
//     re-requests the slot for the item D places ahead.  No warp ever waits for another warp, so there
//     is no CTA-wide barrier inside the stream and no separate producer warp to keep in step.
// W x D x S is sized to fill the SM's shared memory (about 200 KB in flight per SM); measured on B200
// this streams at 6.8-7.0 TB/s, against 6.5-6.65 for the register-staged kernels, and — what the
// decode step needs — the requests for the next matrix are already in flight while the warp waits for
// the activation vector of the current one.
//
// Requirements (the launcher falls back to the register kernels otherwise): K a multiple of 256, so that
// every row and every row's scales start and end on 16-byte boundaries.
// Every wait is bounded (rcu_wait_limit_ns); one that runs out raises RCU_DEVFLAG_TIMEOUT and the kernel
// runs on to its end without waiting again.
#pragma once
#include "bulk_async.cuh"
#include "gemv_q8.cuh"

namespace ringq8 {

using gemvq8::Dot16Local;
using gemvq8::mbar_expect_tx;
using gemvq8::mbar_init;
using gemvq8::mbar_try_wait;
using gemvq8::bulk_load_1d;

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kMaxDepth = 4;                 // slots per warp (mbarriers are laid out for this many)
constexpr int kSlotTarget = 9216;            // bytes of one item the geometry aims for (8192 codes + f32 scales)
constexpr int kBarBytes = kWarps * kMaxDepth * 8;

__device__ __forceinline__ unsigned long long globaltimer() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// All lanes of the warp wait for `bar`.  False when the wait (or an earlier one anywhere on the device) ran out.
__device__ __forceinline__ bool ring_wait(uint64_t* bar, unsigned parity, int* status) {
    unsigned long long t0 = 0;
    for (unsigned i = 0;; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 31u) == 31u) {
            if (*reinterpret_cast<volatile int*>(status) & RCU_DEVFLAG_TIMEOUT) return false;
            const unsigned long long t = globaltimer();
            if (t0 == 0) t0 = t;
            else if (t - t0 > rcu_wait_limit(status)) { atomicOr(status, RCU_DEVFLAG_TIMEOUT); return false; }
        }
    }
}

// How one matrix is cut into items.  A unit is an output element: one weight row (UNIT 1) or a
// (gate, up) row pair `unit_stride` rows apart (UNIT 2).  An item is `ri` consecutive units x one K chunk.
struct Job {
    const int8_t* qs;
    const unsigned char* scales;
    int n_units, unit_stride, K;
    int ri;                 // units per item (1, 2 or 4; ri * UNIT <= 4)
    int kc, nc;             // K chunk (bytes = elements) and chunks per row; kc * nc == K
    int scale_size;         // 2 or 4
};

// Host: choose the cut.  Returns false if K does not meet the alignment rules.
inline bool plan_job(Job* j, int unit, int slot_bytes) {
    const int K = j->K, ss = j->scale_size;
    if (K % 256 != 0 || K < 256) return false;
    const int row = K + K / 32 * ss;
    if (unit * row <= slot_bytes) {
        j->kc = K;
        j->nc = 1;
        int ri = slot_bytes / (unit * row);
        ri = ri >= 4 ? 4 : (ri >= 2 ? 2 : 1);
        while (ri * unit > 4) ri >>= 1;
        j->ri = ri;
        return true;
    }
    // a row does not fit: equal chunks that are multiples of 512 elements (every chunk's scales stay 16-byte aligned)
    for (int nc = 2; nc <= 64; ++nc) {
        if (K % (nc * 512) != 0) continue;
        const int kc = K / nc;
        if (unit * (kc + kc / 32 * ss) <= slot_bytes) {
            j->kc = kc;
            j->nc = nc;
            j->ri = 1;
            return true;
        }
    }
    return false;
}
inline int item_bytes(const Job& j, int unit) { return unit * j.ri * (j.kc + j.kc / 32 * j.scale_size); }

// Lane 0 of a warp: request item (group g, chunk c) of `job` into `slot`, completion on `bar`.
template <int UNIT>
__device__ __forceinline__ void issue_item(const Job& job, int g, int c, unsigned char* slot, uint64_t* bar) {
    const int u0 = g * job.ri;
    const int nr = min(job.ri, job.n_units - u0);
    const int kc = job.kc, ss = job.scale_size;
    const int sc_row = (kc >> 5) * ss;                       // scale bytes of one row chunk
    const int K = job.K;
    const size_t sc_pitch = (size_t)(K >> 5) * ss;           // scale bytes of a whole row
    unsigned char* sdst = slot + UNIT * job.ri * kc;
    // the slot was read with ordinary loads; the copies below write it through the asynchronous proxy
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    mbar_expect_tx(bar, (unsigned)(UNIT * nr * (kc + sc_row)));
#pragma unroll
    for (int b = 0; b < UNIT; ++b) {
        const size_t row0 = (size_t)u0 + (size_t)b * job.unit_stride;
        if (job.nc == 1) {
            bulk_load_1d(slot + b * job.ri * kc, job.qs + row0 * K, (uint32_t)(nr * kc), bar);
            bulk_load_1d(sdst + b * job.ri * sc_row, job.scales + row0 * sc_pitch, (uint32_t)(nr * sc_row), bar);
        } else {
            for (int r = 0; r < nr; ++r) {
                bulk_load_1d(slot + (b * job.ri + r) * kc, job.qs + (row0 + r) * K + (size_t)c * kc, (uint32_t)kc, bar);
                bulk_load_1d(sdst + (b * job.ri + r) * sc_row, job.scales + (row0 + r) * sc_pitch + (size_t)c * sc_row, (uint32_t)sc_row, bar);
            }
        }
    }
}

// The warp multiplies the RT rows of a landed item with the activation planes; acc[r] += partial sums (per lane).
// A batch of 512-element chunks is read into registers before any of it is multiplied (a warp has mostly its
// own instruction-level parallelism to hide the shared-memory latency with: there are few warps per SM).
// shared-memory loads by 32-bit shared address (the slot and plane pointers reach this code as generic pointers)
__device__ __forceinline__ uint4 lds128(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ float lds_f32(uint32_t a) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(a));
    return v;
}
template <class ScaleT> __device__ __forceinline__ float lds_scale(uint32_t a);
template <> __device__ __forceinline__ float lds_scale<float>(uint32_t a) { return lds_f32(a); }
template <> __device__ __forceinline__ float lds_scale<__half>(uint32_t a) {
    unsigned short h;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(h) : "r"(a));
    return __half2float(__ushort_as_half(h));
}

// U chunks of RT rows: everything is read into registers before any of it is multiplied.
// Shared addresses: slot (rows of kc codes, then rows of kc / 32 scales) and planes ([K hi][K lo][K / 16 scales]).
template <int RT, class ScaleT, int U>
__device__ __forceinline__ void consume_chunks(uint32_t slot, uint32_t sc, int kc, int k, uint32_t planes, int K, int kbase, float (&acc)[RT]) {
    Dot16Local d16[U];
    uint4 w[U][RT];
    float ws[U][RT];
    const int sc_row_bytes = (kc >> 5) * (int)sizeof(ScaleT);
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const int ku = k + 512 * u;
        d16[u].h = lds128(planes + kbase + ku);
        d16[u].l = lds128(planes + K + kbase + ku);
        d16[u].s = lds_f32(planes + 2 * K + ((kbase + ku) >> 4) * 4);
#pragma unroll
        for (int r = 0; r < RT; ++r) {
            w[u][r] = lds128(slot + r * kc + ku);
            ws[u][r] = lds_scale<ScaleT>(sc + r * sc_row_bytes + (ku >> 5) * (int)sizeof(ScaleT));
        }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
#pragma unroll
        for (int r = 0; r < RT; ++r) acc[r] = fmaf(d16[u].dot(w[u][r]), ws[u][r], acc[r]);
    }
}

template <int RT, class ScaleT>
__device__ __forceinline__ void consume_item(const unsigned char* slot_ptr, int kc, int kbase, const unsigned char* planes_ptr, int K, float (&acc)[RT]) {
    const int lane = threadIdx.x & 31;
    const uint32_t slot = gemvq8::smem_u32(slot_ptr), planes = gemvq8::smem_u32(planes_ptr);
    const uint32_t sc = slot + RT * kc;
    constexpr int U = RT == 4 ? 2 : 4;
    const int n_full = kc >> 9;                  // chunks every lane takes part in
    int c = 0;
    for (; c + U <= n_full; c += U) consume_chunks<RT, ScaleT, U>(slot, sc, kc, (c << 9) + (lane << 4), planes, K, kbase, acc);
    if (U > 2 && c + 2 <= n_full) {
        consume_chunks<RT, ScaleT, 2>(slot, sc, kc, (c << 9) + (lane << 4), planes, K, kbase, acc);
        c += 2;
    }
    for (; c < n_full; ++c) consume_chunks<RT, ScaleT, 1>(slot, sc, kc, (c << 9) + (lane << 4), planes, K, kbase, acc);
    if ((n_full << 9) + (lane << 4) < kc) consume_chunks<RT, ScaleT, 1>(slot, sc, kc, (n_full << 9) + (lane << 4), planes, K, kbase, acc);
}

// ------------------------------------------------------------------------------------------------
// Prologues: build the activation planes ([K high bytes][K low bytes][K/16 f32 scales]) in shared memory
// straight from the source vector.  All kThreads threads call; the caller synchronises afterwards.
// A thread owns whole groups of 16 elements: group g belongs to thread g % NT.
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void write_group(const float (&v)[16], unsigned char* planes, int K, int g) {
    float amax = 0.f;
    bool finite = true;                    // fmaxf drops a NaN operand: look for NaN / infinity separately
#pragma unroll
    for (int e = 0; e < 16; ++e) {
        amax = fmaxf(amax, fabsf(v[e]));
        finite = finite && fabsf(v[e]) <= 65504.f;
    }
    const float inv = (amax > 0.f && finite) ? 32767.f / amax : 0.f;
    uint32_t hi[4] = {0, 0, 0, 0}, lo[4] = {0, 0, 0, 0};
#pragma unroll
    for (int e = 0; e < 16; ++e) {
        const int X = __float2int_rn(finite ? v[e] * inv : 0.f);
        hi[e >> 2] |= (uint32_t)((X >> 8) & 0xFF) << (8 * (e & 3));
        lo[e >> 2] |= (uint32_t)(X & 0xFF) << (8 * (e & 3));
    }
    reinterpret_cast<uint4*>(planes)[g] = make_uint4(hi[0], hi[1], hi[2], hi[3]);
    reinterpret_cast<uint4*>(planes + K)[g] = make_uint4(lo[0], lo[1], lo[2], lo[3]);
    reinterpret_cast<float*>(planes + 2 * (size_t)K)[g] = finite ? amax / 32767.f : __int_as_float(0x7fc00000);
}

__device__ __forceinline__ void unpack16(const uint4& a, const uint4& b, float (&v)[16]) {
    const uint32_t hw[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&hw[e]));
        v[2 * e] = f.x;
        v[2 * e + 1] = f.y;
    }
}

// a group of 16 f16 values of an ordinary vector, read at L2 (another CTA or kernel produced it)
struct VecSource {
    const __half* x;
    __device__ __forceinline__ void begin() const {}
    __device__ __forceinline__ void load(int g, float (&v)[16]) const {
        const uint4 a = __ldcg(reinterpret_cast<const uint4*>(x) + 2 * g), b = __ldcg(reinterpret_cast<const uint4*>(x) + 2 * g + 1);
        unpack16(a, b, v);
    }
};

// NT = threads that stage (the first NT threads of the CTA; a kernel may run further warps that do not).
template <int NT> __device__ __forceinline__ void stage_barrier() { asm volatile("bar.sync 1, %0;" ::"n"(NT) : "memory"); }

template <class Source, int NT = kThreads> struct PlainPlanes {
    Source s;
    __device__ __forceinline__ void stage(unsigned char* planes, int K, float* /*scratch*/) {
        s.begin();
        for (int g = threadIdx.x; g < (K >> 4); g += NT) {
            float v[16];
            s.load(g, v);
            write_group(v, planes, K, g);
        }
    }
};

// RMSNorm as ratchet-nn schedules it (ratchet-nn/src/norm.rs:63-69): upcast to f32,
// y = x * (1/sqrt(mean(x^2) + eps)) * gamma (cpu/norm.rs:185-213), cast back to f16; the planes are built
// from the f16 result.  A thread keeps its groups in registers between the two passes (up to kKeep groups,
// K <= 16 * kKeep * NT); longer vectors are read a second time.
template <class Source, int NT = kThreads> struct RmsPlanes {
    Source s;
    const float* gamma;
    float eps;
    static constexpr int kKeep = 2;
    __device__ __forceinline__ void stage(unsigned char* planes, int K, float* scratch) {
        s.begin();
        const int ng = K >> 4;
        float keep[kKeep][16];
        float4 gm[kKeep][4];               // the weights of the kept groups: requested before the vector, which may have to be waited for
#pragma unroll
        for (int q = 0; q < kKeep; ++q) {
            const int g = threadIdx.x + q * NT;
            if (g < ng) {
#pragma unroll
                for (int e4 = 0; e4 < 4; ++e4) gm[q][e4] = __ldg(reinterpret_cast<const float4*>(gamma) + 4 * g + e4);
            }
        }
        float s2 = 0.f;
        int n = 0;
        for (int g = threadIdx.x; g < ng; g += NT, ++n) {
            float v[16];
            s.load(g, v);
#pragma unroll
            for (int e = 0; e < 16; ++e) s2 = fmaf(v[e], v[e], s2);
#pragma unroll
            for (int q = 0; q < kKeep; ++q)
                if (q == n) {
#pragma unroll
                    for (int e = 0; e < 16; ++e) keep[q][e] = v[e];
                }
        }
        s2 = warp_sum(s2);
        if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = s2;
        stage_barrier<NT>();
        float tot = 0.f;
#pragma unroll
        for (int w = 0; w < NT / 32; ++w) tot += scratch[w];
        const float rstd = 1.0f / sqrtf(tot / (float)K + eps);
        n = 0;
        for (int g = threadIdx.x; g < ng; g += NT, ++n) {
            float v[16];
            float4 gv[4];
            bool have = false;
#pragma unroll
            for (int q = 0; q < kKeep; ++q)
                if (q == n) {
#pragma unroll
                    for (int e = 0; e < 16; ++e) v[e] = keep[q][e];
#pragma unroll
                    for (int e4 = 0; e4 < 4; ++e4) gv[e4] = gm[q][e4];
                    have = true;
                }
            if (!have) {
                s.load(g, v);
#pragma unroll
                for (int e4 = 0; e4 < 4; ++e4) gv[e4] = __ldg(reinterpret_cast<const float4*>(gamma) + 4 * g + e4);
            }
#pragma unroll
            for (int e4 = 0; e4 < 4; ++e4) {
                v[4 * e4] = __half2float(__float2half_rn(v[4 * e4] * rstd * gv[e4].x));
                v[4 * e4 + 1] = __half2float(__float2half_rn(v[4 * e4 + 1] * rstd * gv[e4].y));
                v[4 * e4 + 2] = __half2float(__float2half_rn(v[4 * e4 + 2] * rstd * gv[e4].z));
                v[4 * e4 + 3] = __half2float(__float2half_rn(v[4 * e4 + 3] * rstd * gv[e4].w));
            }
            write_group(v, planes, K, g);
        }
    }
};

// ------------------------------------------------------------------------------------------------
// One matrix, one kernel: the ring GEMV behind rcu_matmul and rcu_gemv_q8_allgather.
// Shared memory: [mbarriers][planes: 2K + K/4][8 floats][rings: kWarps x D x S].
// ------------------------------------------------------------------------------------------------
__host__ __device__ inline size_t planes_bytes(int K) { return (size_t)2 * K + (size_t)K / 4; }

template <int UNIT, int RI, class Epilogue>
__device__ __forceinline__ void store_units(const Epilogue& epi, int u0, int n_units, float (&acc)[UNIT * RI]) {
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int r = 0; r < UNIT * RI; ++r) acc[r] = warp_sum(acc[r]);
    // unit i of the item is stored by lane i (every lane holds every sum after the butterfly)
    float s[UNIT];
#pragma unroll
    for (int j = 0; j < UNIT; ++j) s[j] = acc[j * RI];
#pragma unroll
    for (int i = 1; i < RI; ++i)
        if (lane == i) {
#pragma unroll
            for (int j = 0; j < UNIT; ++j) s[j] = acc[j * RI + i];
        }
    if (lane < RI && u0 + lane < n_units) epi.store(u0 + lane, s);
#pragma unroll
    for (int r = 0; r < UNIT * RI; ++r) acc[r] = 0.f;
}

template <class ScaleT, int RI, class Prologue, class Epilogue>
__global__ void __launch_bounds__(kThreads, 1)
gemv_q8_ring_kernel(Job job, Prologue pro, Epilogue epi, int slot_bytes, int depth, int* status) {
    constexpr int UNIT = Epilogue::UNIT;
    constexpr int RT = UNIT * RI;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int K = job.K;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem_raw);
    unsigned char* planes = smem_raw + kBarBytes;
    float* scratch = reinterpret_cast<float*>(planes + planes_bytes(K));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    unsigned char* ring = reinterpret_cast<unsigned char*>(scratch + 8) + (size_t)warp * depth * slot_bytes;
    uint64_t* bar = bars + warp * kMaxDepth;

    if (lane == 0) {
        for (int s = 0; s < depth; ++s) mbar_init(&bar[s], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();

    // groups of RI units are dealt to the warps of the grid as contiguous, balanced ranges
    const long long n_groups = (job.n_units + RI - 1) / RI;
    const long long gw = (long long)blockIdx.x * kWarps + warp, GW = (long long)gridDim.x * kWarps;
    const int g0 = (int)(gw * n_groups / GW), g1 = (int)((gw + 1) * n_groups / GW);
    const int nc = job.nc;
    const int n_items = (g1 - g0) * nc;

    // the weights do not depend on the kernel before this one: fill the ring, then wait for x
    gemvq8::pdl_launch_dependents();
    if (lane == 0)
        for (int it = 0; it < depth && it < n_items; ++it) issue_item<UNIT>(job, g0 + it / nc, it % nc, ring + (size_t)it * slot_bytes, &bar[it]);
    gemvq8::pdl_wait();
    pro.stage(planes, K, scratch);
    __syncthreads();

    float acc[RT];
#pragma unroll
    for (int r = 0; r < RT; ++r) acc[r] = 0.f;
    int slot = 0;
    unsigned parity = 0;
    for (int it = 0; it < n_items; ++it) {
        if (!ring_wait(&bar[slot], parity, status)) break;
        const int g = g0 + it / nc, c = it % nc;
        consume_item<RT, ScaleT>(ring + (size_t)slot * slot_bytes, job.kc, c * job.kc, planes, K, acc);
        if (c == nc - 1) store_units<UNIT, RI>(epi, g * RI, job.n_units, acc);
        __syncwarp();
        if (lane == 0 && it + depth < n_items) {
            const int nx = it + depth;
            issue_item<UNIT>(job, g0 + nx / nc, nx % nc, ring + (size_t)slot * slot_bytes, &bar[slot]);
        }
        if (++slot == depth) { slot = 0; parity ^= 1u; }
    }
    epi.warp_done(g0 * RI, min(job.n_units, g1 * RI));
    epi.finish();
}

struct Geometry { int slot_bytes, depth; size_t smem; };

// Slot size = this job's item (rounded up to 128 bytes); depth = what the SM's shared memory holds, at most kMaxDepth.
inline bool geometry(const rcu_device* dev, const Job& job, int unit, Geometry* g) {
    const int slot = (item_bytes(job, unit) + 127) & ~127;
    const size_t fixed = kBarBytes + planes_bytes(job.K) + 8 * sizeof(float) + 128;
    const size_t budget = (size_t)dev->smem_optin - 256;          // an epilogue may keep a few words of static shared memory
    if (fixed + (size_t)kWarps * 2 * slot > budget) return false;
    int depth = (int)((budget - fixed) / ((size_t)kWarps * slot));
    if (depth > kMaxDepth) depth = kMaxDepth;
    g->slot_bytes = slot;
    g->depth = depth;
    g->smem = fixed + (size_t)kWarps * depth * slot;
    return true;
}

// Launch on the device's stream; returns RCU_ERR_UNSUPPORTED (without a message) when the shape does not
// meet the ring's rules, so that the caller can take the register kernel.
template <class ScaleT, class Prologue, class Epilogue>
rcu_status launch(rcu_device* dev, const int8_t* qs, const void* scales, const Prologue& pro, const Epilogue& epi, int N, int K, bool overlap) {
    constexpr int UNIT = Epilogue::UNIT;
    Job job{qs, (const unsigned char*)scales, N / UNIT, N / UNIT, K, 1, K, 1, (int)sizeof(ScaleT)};
    if (!plan_job(&job, UNIT, kSlotTarget)) return RCU_ERR_UNSUPPORTED;
    Geometry geo;
    if (!geometry(dev, job, UNIT, &geo)) return RCU_ERR_UNSUPPORTED;
    const long long n_groups = (job.n_units + job.ri - 1) / job.ri;
    int grid = dev->sm_count;
    if ((long long)grid * kWarps > n_groups) grid = (int)((n_groups + kWarps - 1) / kWarps);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = geo.smem;
    cfg.stream = dev->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = overlap ? 1 : 0;
#define RCU_RING_CASE(RI_)                                                                                              \
    case RI_: {                                                                                                         \
        if constexpr (RI_ * UNIT <= 4) {                                                                                \
            auto kern = gemv_q8_ring_kernel<ScaleT, RI_, Prologue, Epilogue>;                                           \
            RCU_CUDA(dev, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)geo.smem));       \
            RCU_CUDA(dev, cudaLaunchKernelEx(&cfg, kern, job, pro, epi, geo.slot_bytes, geo.depth, dev->d_status));     \
        }                                                                                                               \
        break;                                                                                                          \
    }
    switch (job.ri) {
        RCU_RING_CASE(1)
        RCU_RING_CASE(2)
        RCU_RING_CASE(4)
    }
#undef RCU_RING_CASE
    RCU_LAUNCH_CHECK(dev);
    return RCU_OK;
}

}  // namespace ringq8
