// All transformer layers of one decode step as ONE persistent kernel.
//
// The per-kernel decode step (decode.cu, run_sequence) launches five kernels per layer; each streams
// only 10-56 MB and spends microseconds starting, staging its input vector and draining.  Here the
// CTAs stay resident for the whole step (cooperative launch, two per SM) and walk the same five phases
// per layer, separated by grid-wide barriers:
//     qkv GEMV (RMSNorm prologue) | attention | o GEMV + residual | gate/up GEMV + SiLU | down GEMV + residual
// What a phase needs that does not depend on the phase before it is requested BEFORE the barrier that
// separates them: the first two register slots of the next GEMV's weight stream, and the cached K/V
// rows of a CTA's first attention tile (cp.async into shared memory).  HBM therefore keeps streaming
// while CTAs wait for each other, which is what the separate kernels could not do.
//
// The arithmetic of every phase is that of the separate kernels: gemvq8's dot product, prologues and
// epilogues, and the split-KV attention of decode.cu (64 cached positions per work item, merged by
// the last item of a head to finish).  Data handed from one phase to the next is read with L2 loads
// (__ldcg / cp.async.cg): L1 is not coherent across the CTAs of a running kernel.
//
// Grid barrier: one monotonically increasing counter in global memory, zeroed before the launch;
// thread 0 of each CTA adds one (release) and later polls (acquire) until every CTA of the grid has.  The poll is bounded in time; a barrier that gives up sets RCU_DEVFLAG_TIMEOUT and the
// kernel runs on to its end with meaningless results instead of hanging.
#pragma once
#include "gemv_q8.cuh"

namespace persist {

using gemvq8::Dot16;
using gemvq8::kThreads;
using gemvq8::kWarps;
using gemvq8::ld_scale;
using gemvq8::Slot;

constexpr int ROWS = 4;
constexpr int UNROLL = 2;
constexpr int kTile = 64;            // cached positions per attention work item
constexpr int kMaxSplits = 128;
constexpr int kHalf = 128;           // threads per attention work item (a CTA runs two at a time)

struct LayerW {
    const int8_t* qkv; const __half* qkv_s;
    const int8_t* o; const __half* o_s;
    const int8_t* gate_up; const __half* gate_up_s;
    const int8_t* down; const __half* down_s;
    const float* attn_norm;
    const float* ffn_norm;
    __half* kc;
    __half* vc;
};

struct Params {
    const LayerW* layers;            // device array [n_layers]
    int n_layers, D, H, Hkv, ffn, max_cache, rope_dim;
    float eps, scale;
    __half* x;                       // [D]    residual stream, updated in place
    __half* qkv;                     // [(H + 2 Hkv) * HD]
    __half* attn;                    // [H * HD]
    __half* act;                     // [ffn]
    const uint32_t* d_pos;
    const float* rope_tab;
    float* partial;                  // [H][ceil(max_cache / kTile)][HD + 2]
    unsigned int* counters;          // [H], zero between steps
    unsigned int* bar;               // grid barrier counter, zero at launch
    int* status;
    int ks_qkv, ks_o, ks_gu, ks_down;   // K splits of the four GEMVs (host-chosen, powers of two <= 8)
};

// ------------------------------------------------------------------------------------------------
// The barrier comes in two halves so that work which does not depend on other CTAs (requesting the
// next phase's weights) sits between them.  Arrival is a release reduction without a return value: the
// arriving thread does not wait for the counter's old value.
__device__ __forceinline__ void grid_arrive(const Params& p) {
    __syncthreads();          // every thread's stores of this phase happen before thread 0's release
    if (threadIdx.x == 0) asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(p.bar) : "memory");
}

__device__ __forceinline__ void grid_wait(const Params& p, unsigned int& epoch) {
    if (threadIdx.x == 0) {
        const unsigned int target = (epoch + 1u) * gridDim.x;
        unsigned long long t0 = 0;
        for (unsigned int n = 0;; ++n) {
            unsigned int v;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p.bar) : "memory");
            if ((int)(v - target) >= 0) break;
            if ((n & 255u) == 255u) {
                if (*reinterpret_cast<volatile int*>(p.status) & RCU_DEVFLAG_TIMEOUT) break;
                unsigned long long t;
                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
                if (t0 == 0) t0 = t;
                else if (t - t0 > 1000000000ull) { atomicOr(p.status, RCU_DEVFLAG_TIMEOUT); break; }
            }
        }
    }
    __syncthreads();
    ++epoch;
}

// ------------------------------------------------------------------------------------------------
// Prologues with the arithmetic of gemvq8's, staging x with 16-byte L2 loads requested in pairs (in
// this kernel the weight slots of the phase are live while x is staged, so the staging loop must be
// short and its loads explicit).
template <class ActT> struct VecPlainPrologue {
    const ActT* x;
    __device__ __forceinline__ void stage(ActT* xs, int K, float* /*scratch*/) const {
        const int nvec = K / (16 / (int)sizeof(ActT));
        const uint4* src = reinterpret_cast<const uint4*>(x);
        uint4* dst = reinterpret_cast<uint4*>(xs);
        // two 16-byte loads per thread are requested before the first is stored: x comes from L2 (it was
        // produced by the previous kernel) and each trip there costs most of a microsecond
        for (int i = threadIdx.x; i < nvec; i += 2 * kThreads) {
            const bool second = i + kThreads < nvec;
            const uint4 a = __ldcg(src + i);
            uint4 b = a;
            if (second) b = __ldcg(src + i + kThreads);
            dst[i] = a;
            if (second) dst[i + kThreads] = b;
        }
    }
};

// RMSNorm prologue of gemvq8::RmsNormPrologueH with 16-byte loads.
__device__ __forceinline__ float sumsq8(const uint4& v, float s2) {
    const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const float2 f = __half22float2(h[e]);
        s2 = fmaf(f.x, f.x, s2);
        s2 = fmaf(f.y, f.y, s2);
    }
    return s2;
}

struct VecRmsNormPrologueH {
    const __half* x;
    const float* gamma;
    float eps;
    __device__ __forceinline__ void stage(__half* xs, int K, float* scratch) const {
        // one trip to L2 per pair of 16-byte loads: raw values are parked in shared memory while the sum
        // of squares is reduced
        const int nvec = K >> 3;
        const uint4* src = reinterpret_cast<const uint4*>(x);
        uint4* dst = reinterpret_cast<uint4*>(xs);
        float s2 = 0.f;
        for (int i = threadIdx.x; i < nvec; i += 2 * kThreads) {
            const bool second = i + kThreads < nvec;
            const uint4 a = __ldcg(src + i);
            uint4 b = make_uint4(0u, 0u, 0u, 0u);
            if (second) b = __ldcg(src + i + kThreads);
            dst[i] = a;
            s2 = sumsq8(a, s2);
            if (second) {
                dst[i + kThreads] = b;
                s2 = sumsq8(b, s2);
            }
        }
        s2 = warp_sum(s2);
        if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = s2;
        // the kThreads staging threads only (a kernel may run extra warps that do not stage)
        asm volatile("bar.sync 15, %0;" ::"n"(kThreads) : "memory");
        float tot = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) tot += scratch[w];
        const float rstd = 1.0f / sqrtf(tot / (float)K + eps);
        // each thread normalises the vectors it staged itself
        for (int i = threadIdx.x; i < nvec; i += kThreads) {
            uint4 v = dst[i];
            __half2* h = reinterpret_cast<__half2*>(&v);
            const float4 g0 = __ldg(reinterpret_cast<const float4*>(gamma) + 2 * i), g1 = __ldg(reinterpret_cast<const float4*>(gamma) + 2 * i + 1);
            float2 f = __half22float2(h[0]);
            h[0] = __floats2half2_rn(f.x * rstd * g0.x, f.y * rstd * g0.y);
            f = __half22float2(h[1]);
            h[1] = __floats2half2_rn(f.x * rstd * g0.z, f.y * rstd * g0.w);
            f = __half22float2(h[2]);
            h[2] = __floats2half2_rn(f.x * rstd * g1.x, f.y * rstd * g1.y);
            f = __half22float2(h[3]);
            h[3] = __floats2half2_rn(f.x * rstd * g1.z, f.y * rstd * g1.w);
            dst[i] = v;
        }
    }
};

// ------------------------------------------------------------------------------------------------
// GEMV phase: the work split and the item pipeline of gemvq8::gemv_q8_pipe_kernel with the K split as
// a run-time value (one kernel serves all four shapes).
struct Gemv {
    const int8_t* qs;
    const __half* scales;
    int n_units, K, ksplit;       // row j of unit u is u + j * n_units
};

struct WarpMap {
    int u_begin, u_end, ncg, n_items;
};

template <int UNIT>
__device__ __forceinline__ WarpMap map_warp(const Gemv& g) {
    constexpr int UPI = ROWS / UNIT;
    WarpMap m;
    const int warp = threadIdx.x >> 5;
    const int RG = kWarps / g.ksplit;
    const int rg = warp / g.ksplit, ks = warp % g.ksplit;
    const long long gw = (long long)blockIdx.x * RG + rg;
    const long long W = (long long)gridDim.x * RG;
    const long long n_groups_all = (g.n_units + UPI - 1) / UPI;       // whole groups are dealt, as in gemvq8's kernels
    m.u_begin = (int)((gw * n_groups_all) / W) * UPI;
    m.u_end = min(g.n_units, (int)(((gw + 1) * n_groups_all) / W) * UPI);
    const int nchunks = (g.K + 511) >> 9;
    const int n_groups = (m.u_end - m.u_begin + UPI - 1) / UPI;
    m.ncg = (nchunks - ks + g.ksplit * UNROLL - 1) / (g.ksplit * UNROLL);
    if (m.ncg < 0) m.ncg = 0;
    m.n_items = n_groups * m.ncg;
    return m;
}

template <int UNIT>
__device__ __forceinline__ void load_item(const Gemv& g, const WarpMap& m, int it, Slot<UNROLL, ROWS>& s) {
    constexpr int UPI = ROWS / UNIT;
    const int kl = (threadIdx.x & 31) << 4;
    const int kblocks = g.K >> 5;
    const int ks = (threadIdx.x >> 5) % g.ksplit;
    const int u0 = m.u_begin + (it / m.ncg) * UPI;
    const int c0 = ks + (it % m.ncg) * (g.ksplit * UNROLL);
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
        const int k = ((c0 + u * g.ksplit) << 9) + kl;
        const bool live = k < g.K;
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            const int un = min(u0 + r / UNIT, m.u_end - 1);     // duplicate the last unit; its result is dropped
            const size_t row = (size_t)(un + (r % UNIT) * g.n_units);
            if (live) {
                s.w[u][r] = ld_stream_v4(g.qs + row * g.K + k);
                s.sc[u][r] = ld_scale<__half>(g.scales + row * kblocks + (k >> 5));
            } else {
                s.w[u][r] = make_uint4(0x0, 0x0, 0x0, 0x0);
                s.sc[u][r] = 0.f;
            }
        }
    }
}

template <class Epi>
__device__ __forceinline__ void compute_item(const Gemv& g, const WarpMap& m, int it, const Slot<UNROLL, ROWS>& s, const __half* xs, float* red,
                                             float (&acc)[ROWS], const Epi& epi) {
    constexpr int UNIT = Epi::UNIT;
    constexpr int UPI = ROWS / UNIT;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int kl = lane << 4;
    const int rg = warp / g.ksplit, ks = warp % g.ksplit;
    const int c0 = ks + (it % m.ncg) * (g.ksplit * UNROLL);
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
        const int k = ((c0 + u * g.ksplit) << 9) + kl;
        if (k < g.K) {
            Dot16<__half, 0> d16;
            d16.load(xs, k);
#pragma unroll
            for (int r = 0; r < ROWS; ++r) acc[r] = fmaf(d16.dot(s.w[u][r]), s.sc[u][r], acc[r]);
        }
    }
    if (it % m.ncg != m.ncg - 1) return;
    // last chunk group of this unit group: reduce and store
    const int u0 = m.u_begin + (it / m.ncg) * UPI;
#pragma unroll
    for (int r = 0; r < ROWS; ++r) acc[r] = warp_sum(acc[r]);
    if (g.ksplit > 1) {
        if (lane == 0) {
#pragma unroll
            for (int r = 0; r < ROWS; ++r) red[warp * ROWS + r] = acc[r];
        }
        asm volatile("bar.sync %0, %1;" ::"r"(1 + rg), "r"(g.ksplit * 32) : "memory");
        if (ks == 0 && lane < UPI) {
            float sum[UNIT];
#pragma unroll
            for (int j = 0; j < UNIT; ++j) {
                sum[j] = 0.f;
                for (int q = 0; q < g.ksplit; ++q) sum[j] += red[(rg * g.ksplit + q) * ROWS + lane * UNIT + j];
            }
            if (u0 + lane < m.u_end) epi.store(u0 + lane, sum);
        }
        asm volatile("bar.sync %0, %1;" ::"r"(1 + rg), "r"(g.ksplit * 32) : "memory");
    } else if (lane == 0) {
#pragma unroll
        for (int i = 0; i < UPI; ++i)
            if (u0 + i < m.u_end) epi.store(u0 + i, &acc[i * UNIT]);
    }
#pragma unroll
    for (int r = 0; r < ROWS; ++r) acc[r] = 0.f;
}

// Runs a GEMV whose first two slots are already in flight.
template <class Pro, class Epi>
__device__ __forceinline__ void run_gemv(const Gemv& g, const WarpMap& m, Slot<UNROLL, ROWS>& s0, Slot<UNROLL, ROWS>& s1, const Pro& pro,
                                         const Epi& epi, __half* xs, float* red) {
    pro.stage(xs, g.K, red);
    __syncthreads();
    float acc[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) acc[r] = 0.f;
    for (int it = 0; it < m.n_items; it += 2) {
        compute_item(g, m, it, s0, xs, red, acc, epi);
        if (it + 2 < m.n_items) load_item<Epi::UNIT>(g, m, it + 2, s0);
        if (it + 1 < m.n_items) {
            compute_item(g, m, it + 1, s1, xs, red, acc, epi);
            if (it + 3 < m.n_items) load_item<Epi::UNIT>(g, m, it + 3, s1);
        }
    }
    __syncthreads();      // xs and red are free again
}

template <int UNIT>
__device__ __forceinline__ void prefetch_gemv(const Gemv& g, const WarpMap& m, Slot<UNROLL, ROWS>& s0, Slot<UNROLL, ROWS>& s1) {
    if (m.n_items > 0) load_item<UNIT>(g, m, 0, s0);
    if (m.n_items > 1) load_item<UNIT>(g, m, 1, s1);
}

// ------------------------------------------------------------------------------------------------
// Attention phase.  Work item = (head, tile of 64 cached positions); a CTA runs two items at a time,
// one per half of its threads, with named barriers 9 and 10.
template <int HD> struct AttnShared {
    __half Ks[kTile * HD];
    __half Vs[kTile * HD];
    float sc[kTile];
    float q_s[HD], k_s[HD], v_s[HD];
    float red[8];
    float o_s[4][HD];
    float wgt[kMaxSplits];
    unsigned int ticket;
    int pad[3];
};

__device__ __forceinline__ void half_sync(int half) { asm volatile("bar.sync %0, %1;" ::"r"(9 + half), "n"(kHalf) : "memory"); }

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gsrc) : "memory");
}

__device__ __forceinline__ float f16r(float v) { return __half2float(__float2half_rn(v)); }

// RoPE of one head row read from global memory at L2 (written by the phase before), as rope.cu does it
template <int HD>
__device__ __forceinline__ void rope_into(const __half* in, const float* tab, int rope_dim, float* dst, int t) {
    const int half = rope_dim >> 1;
    for (int i = t; i < HD; i += kHalf) {
        if (i < half) {
            const float x1 = __half2float(__ldcg(in + i)), x2 = __half2float(__ldcg(in + i + half));
            const float c = tab[i], s = tab[half + i];
            dst[i] = f16r(__fsub_rn(__fmul_rn(x1, c), __fmul_rn(x2, s)));
            dst[i + half] = f16r(__fadd_rn(__fmul_rn(x1, s), __fmul_rn(x2, c)));
        } else if (i >= rope_dim) {
            dst[i] = __half2float(__ldcg(in + i));
        }
    }
}

// requests the cached K and V rows of work item `item` (none if the item does not exist)
template <int HD>
__device__ __forceinline__ void attn_prefetch(const Params& p, const LayerW& L, int item, int P, AttnShared<HD>& sh, int t) {
    const int T = P + 1;
    const int nsplit = (T + kTile - 1) / kTile;
    if (item < p.H * nsplit) {
        const int h = item % p.H, s = item / p.H;
        const int kvh = h / (p.H / p.Hkv);
        const int begin = s * kTile;
        const int end = min(T, begin + kTile);
        const int n_cached = min(end, P) - begin;
        const int vecs = n_cached * (HD / 8);
        const uint4* kg = reinterpret_cast<const uint4*>(L.kc + ((size_t)kvh * p.max_cache + begin) * HD);
        const uint4* vg = reinterpret_cast<const uint4*>(L.vc + ((size_t)kvh * p.max_cache + begin) * HD);
        for (int i = t; i < vecs; i += kHalf) {
            cp_async16(reinterpret_cast<uint4*>(sh.Ks) + i, kg + i);
            cp_async16(reinterpret_cast<uint4*>(sh.Vs) + i, vg + i);
        }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
}

template <int HD>
__device__ __forceinline__ void attn_item(const Params& p, const LayerW& L, int item, int P, AttnShared<HD>& sh, int t, int half_id) {
    const int T = P + 1;
    const int nsplit = (T + kTile - 1) / kTile;
    const int max_splits = (p.max_cache + kTile - 1) / kTile;
    const int h = item % p.H, s = item / p.H;
    const int group = p.H / p.Hkv;
    const int kvh = h / group;
    const int begin = s * kTile;
    const int end = min(T, begin + kTile);
    const int n = end - begin;
    const bool owns_new = P < end;
    const int qkv_k = p.H * HD, qkv_v = (p.H + p.Hkv) * HD;
    rope_into<HD>(p.qkv + (size_t)h * HD, p.rope_tab, p.rope_dim, sh.q_s, t);
    if (owns_new) {
        rope_into<HD>(p.qkv + qkv_k + (size_t)kvh * HD, p.rope_tab, p.rope_dim, sh.k_s, t);
        for (int i = t; i < HD; i += kHalf) sh.v_s[i] = __half2float(__ldcg(p.qkv + qkv_v + (size_t)kvh * HD + i));
    }
    half_sync(half_id);
    if (owns_new) {
        const int row = P - begin;
        __half* K = L.kc + (size_t)kvh * p.max_cache * HD;
        __half* V = L.vc + (size_t)kvh * p.max_cache * HD;
        for (int i = t; i < HD; i += kHalf) {
            const __half kh = __float2half_rn(sh.k_s[i]), vh = __float2half_rn(sh.v_s[i]);
            sh.Ks[row * HD + i] = kh;
            sh.Vs[row * HD + i] = vh;
            if (h % group == 0) {
                K[(size_t)P * HD + i] = kh;
                V[(size_t)P * HD + i] = vh;
            }
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    half_sync(half_id);

    // scores: four lanes per position, HD/4 dims each
    constexpr int DPL = HD / 4;
    const int sub = t & 3;
    float qreg[DPL];
#pragma unroll
    for (int i = 0; i < DPL; ++i) qreg[i] = sh.q_s[sub * DPL + i];
#pragma unroll
    for (int pl0 = 0; pl0 < kTile; pl0 += kHalf / 4) {
        const int pl = pl0 + (t >> 2);
        float dot = 0.f;
        if (pl < n) {
            const uint4* kp = reinterpret_cast<const uint4*>(sh.Ks + pl * HD + sub * DPL);
#pragma unroll
            for (int v = 0; v < DPL / 8; ++v) {
                const uint4 w = kp[v];
                const __half2* hp = reinterpret_cast<const __half2*>(&w);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 f = __half22float2(hp[j]);
                    dot = fmaf(qreg[v * 8 + 2 * j], f.x, dot);
                    dot = fmaf(qreg[v * 8 + 2 * j + 1], f.y, dot);
                }
            }
        }
        dot += __shfl_xor_sync(0xffffffffu, dot, 1);
        dot += __shfl_xor_sync(0xffffffffu, dot, 2);
        if (pl < n && sub == 0) sh.sc[pl] = f16r(dot * p.scale);
    }
    half_sync(half_id);

    float m = t < n ? sh.sc[t] : -INFINITY;
    m = warp_max(m);
    if ((t & 31) == 0) sh.red[t >> 5] = m;
    half_sync(half_id);
    m = fmaxf(fmaxf(sh.red[0], sh.red[1]), fmaxf(sh.red[2], sh.red[3]));
    half_sync(half_id);
    float l = 0.f;
    if (t < n) {
        const float e = expf(sh.sc[t] - m);
        sh.sc[t] = e;
        l = e;
    }
    l = warp_sum(l);
    if ((t & 31) == 0) sh.red[t >> 5] = l;
    half_sync(half_id);
    l = sh.red[0] + sh.red[1] + sh.red[2] + sh.red[3];

    constexpr int HP = HD / 2;
    constexpr int G = kHalf / HP;
    const int dp = t % HP, g = t / HP;
    if (g < G) {
        float2 acc = make_float2(0.f, 0.f);
#pragma unroll 4
        for (int j = g; j < n; j += G) {
            const float2 v = __half22float2(*reinterpret_cast<const __half2*>(sh.Vs + j * HD + 2 * dp));
            const float pj = sh.sc[j];
            acc.x = fmaf(pj, v.x, acc.x);
            acc.y = fmaf(pj, v.y, acc.y);
        }
        sh.o_s[g][2 * dp] = acc.x;
        sh.o_s[g][2 * dp + 1] = acc.y;
    }
    half_sync(half_id);
    float* part = p.partial + ((size_t)h * max_splits + s) * (HD + 2);
    for (int d = t; d < HD; d += kHalf) {
        float o = 0.f;
#pragma unroll
        for (int gg = 0; gg < G; ++gg) o += sh.o_s[gg][d];
        part[2 + d] = o;
    }
    if (t == 0) { part[0] = m; part[1] = l; }

    // merge: the last item of this head to finish
    __threadfence();
    half_sync(half_id);
    if (t == 0) sh.ticket = atomicAdd(&p.counters[h], 1u);
    half_sync(half_id);
    if (sh.ticket == (unsigned int)nsplit - 1) {
        __threadfence();
        const float* hp = p.partial + (size_t)h * max_splits * (HD + 2);
        float mj = -INFINITY, lj = 0.f;
        if (t < nsplit) {
            mj = __ldcg(hp + t * (HD + 2));
            lj = __ldcg(hp + t * (HD + 2) + 1);
        }
        float M = warp_max(mj);
        if ((t & 31) == 0) sh.red[t >> 5] = M;
        half_sync(half_id);
        M = fmaxf(fmaxf(sh.red[0], sh.red[1]), fmaxf(sh.red[2], sh.red[3]));
        half_sync(half_id);
        const float wj = t < nsplit ? expf(mj - M) : 0.f;
        if (t < nsplit) sh.wgt[t] = wj;
        float Lsum = warp_sum(lj * wj);
        if ((t & 31) == 0) sh.red[t >> 5] = Lsum;
        half_sync(half_id);
        Lsum = sh.red[0] + sh.red[1] + sh.red[2] + sh.red[3];
        for (int d = t; d < HD; d += kHalf) {
            float o = 0.f;
#pragma unroll 8
            for (int j = 0; j < nsplit; ++j) o = fmaf(__ldcg(hp + j * (HD + 2) + 2 + d), sh.wgt[j], o);
            p.attn[(size_t)h * HD + d] = __float2half_rn(o / Lsum);
        }
        if (t == 0) p.counters[h] = 0;
    }
    half_sync(half_id);      // the item's shared memory is free again
}

// ------------------------------------------------------------------------------------------------
template <int HD>
__global__ void __launch_bounds__(kThreads, 2) decode_layers_kernel(const Params p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int kmax = max(max(p.D, p.ffn), p.H * HD);
    __half* xs = reinterpret_cast<__half*>(smem_raw);
    float* red = reinterpret_cast<float*>(smem_raw + (size_t)kmax * sizeof(__half));
    AttnShared<HD>* ash = reinterpret_cast<AttnShared<HD>*>(smem_raw + (((size_t)kmax * sizeof(__half) + kWarps * ROWS * sizeof(float) + 15) & ~(size_t)15));

    const int half_id = threadIdx.x / kHalf, t = threadIdx.x % kHalf;
    const int P = (int)*p.d_pos;
    const int T = P + 1;
    const int nsplit = (T + kTile - 1) / kTile;
    const int n_attn_items = p.H * nsplit;
    const int qkv_n = (p.H + 2 * p.Hkv) * HD;
    unsigned int epoch = 0;
    Slot<UNROLL, ROWS> s0, s1;

    Gemv g{p.layers[0].qkv, p.layers[0].qkv_s, qkv_n, p.D, p.ks_qkv};
    WarpMap m = map_warp<1>(g);
    prefetch_gemv<1>(g, m, s0, s1);
    for (int li = 0; li < p.n_layers; ++li) {
        const LayerW L = p.layers[li];
        // ---- qkv = W_qkv . rmsnorm(x)
        run_gemv(g, m, s0, s1, VecRmsNormPrologueH{p.x, L.attn_norm, p.eps}, gemvq8::PlainEpilogue<__half>{nullptr, p.qkv}, xs, red);
        grid_arrive(p);
        const int first_item = blockIdx.x * 2 + half_id;
        attn_prefetch<HD>(p, L, first_item, P, ash[half_id], t);
        grid_wait(p, epoch);
        // ---- attention over this layer's cache (no weights are requested across it: it needs the registers)
        for (int item = first_item; item < n_attn_items; item += gridDim.x * 2) {
            if (item != first_item) attn_prefetch<HD>(p, L, item, P, ash[half_id], t);
            attn_item<HD>(p, L, item, P, ash[half_id], t, half_id);
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        grid_arrive(p);
        g = Gemv{L.o, L.o_s, p.D, p.H * HD, p.ks_o};
        m = map_warp<1>(g);
        prefetch_gemv<1>(g, m, s0, s1);
        grid_wait(p, epoch);
        // ---- x += W_o . attn
        run_gemv(g, m, s0, s1, VecPlainPrologue<__half>{p.attn}, gemvq8::ResidualEpilogueH{p.x, p.x}, xs, red);
        grid_arrive(p);
        g = Gemv{L.gate_up, L.gate_up_s, p.ffn, p.D, p.ks_gu};
        m = map_warp<2>(g);
        prefetch_gemv<2>(g, m, s0, s1);
        grid_wait(p, epoch);
        // ---- act = up * silu(gate)
        run_gemv(g, m, s0, s1, VecRmsNormPrologueH{p.x, L.ffn_norm, p.eps}, gemvq8::SiluGateEpilogueH{p.act}, xs, red);
        grid_arrive(p);
        g = Gemv{L.down, L.down_s, p.D, p.ffn, p.ks_down};
        m = map_warp<1>(g);
        prefetch_gemv<1>(g, m, s0, s1);
        grid_wait(p, epoch);
        // ---- x += W_down . act
        run_gemv(g, m, s0, s1, VecPlainPrologue<__half>{p.act}, gemvq8::ResidualEpilogueH{p.x, p.x}, xs, red);
        grid_arrive(p);
        if (li + 1 < p.n_layers) {
            g = Gemv{p.layers[li + 1].qkv, p.layers[li + 1].qkv_s, qkv_n, p.D, p.ks_qkv};
            m = map_warp<1>(g);
            prefetch_gemv<1>(g, m, s0, s1);
        }
        grid_wait(p, epoch);
    }
}

}  // namespace persist
