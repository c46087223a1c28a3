// Fused decode step for a decoder-only transformer at sequence length 1, and its attention kernel.
//
// What ratchet-models' Phi3::schedule (phi3/model.rs:134-156) builds per token as ~43 lazy nodes
// per layer (phi3/attn.rs:88-159, phi3/mlp.rs:31-39, ratchet-nn/src/norm.rs:63-69) runs here as
// five kernels per layer, replayed from a CUDA graph:
//   qkv GEMV with the RMSNorm folded into its activation staging,
//   attention (RoPE on q/k, KV append, split-KV softmax(q.K^T).V with an in-kernel combine),
//   o GEMV + residual add, gate_up GEMV with RMSNorm prologue and SiLU-gate epilogue,
//   down GEMV + residual add.
// Rounding points of the reference graph that matter at the 1e-2 parity bar are kept: activations
// are f16 between ops, norms/rope/softmax are evaluated in f32 from f16 inputs, scores are rounded
// to f16 after scaling (attn.rs:145), Linear outputs are rounded to f16 before the residual add.
//
// Every kernel is HBM-bound at batch 1: the GEMVs stream the Q8_0 weights once (gemv_q8.cuh); the
// attention kernel streams the K and V rows of the populated cache once, 16 CTAs per head so that
// 32 heads fill the 148 SMs.
#include <atomic>
#include <cmath>
#include <cstdlib>
#include <mutex>

#include <cooperative_groups.h>

#include "comm.cuh"
#include "decode_flow.cuh"

namespace {

constexpr int kTile = 64;           // cache positions per CTA (split-KV): CTA s of a head owns positions [64 s, 64 s + 64)
constexpr int kMaxSplits = 128;     // the merge step assigns one thread per split: max_cache <= 8192
constexpr int kAttnThreads = 128;
constexpr int kClusterCtas = 16;    // CTAs of one head in the cluster variant of the attention kernel

struct AttnParams {
    const __half* qkv;
    __half* kc;
    __half* vc;
    int H, Hkv, max_cache, rope_dim;
    const uint32_t* d_pos;         // entries already in the cache = position of this token
    const float* rope_tab;         // cos[rope_dim/2] then sin[rope_dim/2] for this position
    float scale;
    float* partial;                // [H][ceil(max_cache / kTile)][HD + 2]: m, l, unnormalised o
    unsigned int* counters;        // [H], zero between launches
    __half* out;                   // [H * HD]
    gemvq8::LLPush ll;             // ll.local != nullptr: the head outputs go to every rank's window instead of `out`
};

__device__ __forceinline__ float f16r(float v) { return __half2float(__float2half_rn(v)); }

// cos/sin of theta = pos * inv_f[i], evaluated as rope.cu does (cpu/rope.rs:23-61)
__global__ void rope_table_kernel(const uint32_t* d_pos, float ln_base, int half, float* tab) {
    const int i = threadIdx.x;
    if (i >= half) return;
    const float e = -(float)i * ln_base / (float)half;
    const float inv = (float)exp((double)e);
    const float th = (float)(*d_pos) * inv;
    double sd, cd;
    sincos((double)th, &sd, &cd);
    tab[i] = (float)cd;
    tab[half + i] = (float)sd;
}

template <int HD>
__device__ __forceinline__ void rope_into(const __half* in, const float* tab, int rope_dim, float* dst) {
    const int half = rope_dim >> 1;
    for (int i = threadIdx.x; i < HD; i += kAttnThreads) {
        if (i < half) {
            const float x1 = __half2float(in[i]), x2 = __half2float(in[i + half]);
            const float c = tab[i], s = tab[half + i];
            // f32 rope with each product rounded (no fma contraction), then `.cast(f16)` (attn.rs:118-130)
            dst[i] = f16r(__fsub_rn(__fmul_rn(x1, c), __fmul_rn(x2, s)));
            dst[i + half] = f16r(__fadd_rn(__fmul_rn(x1, s), __fmul_rn(x2, c)));
        } else if (i >= rope_dim) {
            dst[i] = __half2float(in[i]);
        }
    }
}

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gsrc) : "memory");
}

inline int attn_splits(int max_cache) { return (max_cache + kTile - 1) / kTile; }

// grid = (H, ceil(max_cache / kTile)): fixed by the cache capacity, so a captured launch stays valid as
// the position advances; CTAs whose tile lies beyond the current position leave at once (heads are
// the fast grid axis, so the working CTAs of all heads are scheduled before the idle ones).  A working CTA
// starts by copying its 64 cached K rows and V rows into shared memory with 16-byte asynchronous
// copies (every byte it will read is requested before anything is computed), applies RoPE to q (and to
// the new k row if the tile holds the current position) while they arrive, then computes scores,
// tile-local softmax statistics and the unnormalised output from shared memory.  The last CTA of a
// head to finish merges the head's partial results.
template <int HD>
__global__ void __launch_bounds__(kAttnThreads) attn_decode_kernel(AttnParams p) {
    __shared__ __align__(16) __half Ks[kTile * HD];
    __shared__ __align__(16) __half Vs[kTile * HD];
    __shared__ float sc[kTile];                     // scores / probabilities of this CTA's tile
    __shared__ float q_s[HD], k_s[HD], v_s[HD];
    __shared__ float red[kAttnThreads / 32 + 2];
    __shared__ float o_s[4][HD];
    __shared__ float wgt_s[kMaxSplits];
    __shared__ unsigned int ticket;

    // everything this kernel reads was produced by kernels before it in the stream; the kernel after
    // it may begin launching (it only prefetches weights until this one has finished)
    gemvq8::pdl_launch_dependents();
    gemvq8::pdl_wait();
    const int tid = threadIdx.x;
    const int h = blockIdx.x, s = blockIdx.y;
    const int P = (int)*p.d_pos;
    const int T = P + 1;
    const int nsplit = (T + kTile - 1) / kTile;
    if (s >= nsplit) return;
    const int group = p.H / p.Hkv;
    const int kvh = h / group;
    const int begin = s * kTile;
    const int end = min(T, begin + kTile);
    const int n = end - begin;
    __half* K = p.kc + (size_t)kvh * p.max_cache * HD;
    __half* V = p.vc + (size_t)kvh * p.max_cache * HD;
    const bool owns_new = P < end;                  // P >= begin always holds for a working CTA's last tile
    {
        // rows already in the cache: [begin, min(end, P))
        const int n_cached = min(end, P) - begin;
        const int vecs = n_cached * (HD / 8);
        const uint4* kg = reinterpret_cast<const uint4*>(K + (size_t)begin * HD);
        const uint4* vg = reinterpret_cast<const uint4*>(V + (size_t)begin * HD);
        for (int i = tid; i < vecs; i += kAttnThreads) {
            cp_async16(reinterpret_cast<uint4*>(Ks) + i, kg + i);
            cp_async16(reinterpret_cast<uint4*>(Vs) + i, vg + i);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    const __half* q_in = p.qkv + (size_t)h * HD;
    const __half* k_in = p.qkv + (size_t)(p.H + kvh) * HD;
    const __half* v_in = p.qkv + (size_t)(p.H + p.Hkv + kvh) * HD;
    rope_into<HD>(q_in, p.rope_tab, p.rope_dim, q_s);
    if (owns_new) {
        rope_into<HD>(k_in, p.rope_tab, p.rope_dim, k_s);
        for (int i = tid; i < HD; i += kAttnThreads) v_s[i] = __half2float(v_in[i]);
    }
    __syncthreads();
    if (owns_new) {
        // Cache op (ops/cache.rs:73-103): the new row goes into the cache for later steps (written by
        // one of the query heads that share this kv head); this step reads it from the tile.
        const int row = P - begin;
        for (int i = tid; i < HD; i += kAttnThreads) {
            const __half kh = __float2half_rn(k_s[i]), vh = __float2half_rn(v_s[i]);   // exact: both hold f16 values
            Ks[row * HD + i] = kh;
            Vs[row * HD + i] = vh;
            if (h % group == 0) {
                K[(size_t)P * HD + i] = kh;
                V[(size_t)P * HD + i] = vh;
            }
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();

    // ---- phase 1: scores. four lanes per position, HD/4 dims each
    constexpr int DPL = HD / 4;
    const int sub = tid & 3;
    float qreg[DPL];
#pragma unroll
    for (int i = 0; i < DPL; ++i) qreg[i] = q_s[sub * DPL + i];
#pragma unroll
    for (int pl0 = 0; pl0 < kTile; pl0 += kAttnThreads / 4) {
        const int pl = pl0 + (tid >> 2);
        float dot = 0.f;
        if (pl < n) {
            const uint4* kp = reinterpret_cast<const uint4*>(Ks + pl * HD + sub * DPL);
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
        if (pl < n && sub == 0) sc[pl] = f16r(dot * p.scale);   // `.mul(scale).cast(f16)` (attn.rs:142-146)
    }
    __syncthreads();

    // ---- phase 2: tile-local softmax statistics
    float m = tid < n ? sc[tid] : -INFINITY;        // kTile <= kAttnThreads
    m = warp_max(m);
    if ((tid & 31) == 0) red[tid >> 5] = m;
    __syncthreads();
    m = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
    __syncthreads();
    float l = 0.f;
    if (tid < n) {
        const float e = expf(sc[tid] - m);
        sc[tid] = e;
        l = e;
    }
    l = warp_sum(l);
    if ((tid & 31) == 0) red[tid >> 5] = l;
    __syncthreads();
    l = red[0] + red[1] + red[2] + red[3];

    // ---- phase 3: o = sum_j p_j V_j. thread -> (dim pair, position group)
    constexpr int HP = HD / 2;
    constexpr int G = kAttnThreads / HP;            // position groups (2 for HD 96/128, 4 for 64)
    const int dp = tid % HP, g = tid / HP;
    if (g < G) {
        float2 acc = make_float2(0.f, 0.f);
#pragma unroll 4
        for (int j = g; j < n; j += G) {
            const float2 v = __half22float2(*reinterpret_cast<const __half2*>(Vs + j * HD + 2 * dp));
            const float pj = sc[j];
            acc.x = fmaf(pj, v.x, acc.x);
            acc.y = fmaf(pj, v.y, acc.y);
        }
        o_s[g][2 * dp] = acc.x;
        o_s[g][2 * dp + 1] = acc.y;
    }
    __syncthreads();
    const int max_splits = gridDim.y;
    float* part = p.partial + ((size_t)h * max_splits + s) * (HD + 2);
    for (int d = tid; d < HD; d += kAttnThreads) {
        float o = 0.f;
#pragma unroll
        for (int gg = 0; gg < G; ++gg) o += o_s[gg][d];
        part[2 + d] = o;
    }
    if (tid == 0) { part[0] = m; part[1] = l; }

    // ---- combine: the last working CTA of this head to finish merges the head's partials
    __threadfence();
    __syncthreads();
    if (tid == 0) ticket = atomicAdd(&p.counters[h], 1u);
    __syncthreads();
    if (ticket != (unsigned int)nsplit - 1) return;
    __threadfence();
    const float* hp = p.partial + (size_t)h * max_splits * (HD + 2);
    // one thread per split fetches its (m, l): all loads of the merge are in flight together
    float mj = -INFINITY, lj = 0.f;
    if (tid < nsplit) {
        mj = __ldcg(hp + tid * (HD + 2));
        lj = __ldcg(hp + tid * (HD + 2) + 1);
    }
    float M = warp_max(mj);
    if ((tid & 31) == 0) red[tid >> 5] = M;
    __syncthreads();
    M = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
    __syncthreads();
    const float wj = tid < nsplit ? expf(mj - M) : 0.f;
    if (tid < nsplit) wgt_s[tid] = wj;
    float L = warp_sum(lj * wj);
    if ((tid & 31) == 0) red[tid >> 5] = L;
    __syncthreads();
    L = red[0] + red[1] + red[2] + red[3];
    for (int d = tid; d < HD; d += kAttnThreads) {
        float o = 0.f;
#pragma unroll 8
        for (int j = 0; j < nsplit; ++j) o = fmaf(__ldcg(hp + j * (HD + 2) + 2 + d), wgt_s[j], o);
        const __half r = __float2half_rn(o / L);
        if (p.ll.local) p.ll.put(h * HD + d, r);     // sharded decoder: this rank's heads -> every rank
        else p.out[(size_t)h * HD + d] = r;
    }
    if (tid == 0) p.counters[h] = 0;                 // ready for the next launch
}

// ------------------------------------------------------------------------------------------------
// The same attention with one thread-block cluster per head.
//
// Sixteen CTAs form the cluster of a head (grid = (H, 16), cluster dimension (1, 16)).  The 64-position
// tiles of the cache go round-robin to the cluster's CTAs; a warp owns 16 positions of a tile and keeps
// them in registers: the K rows as (position, half row) per lane, the V rows as four features per lane,
// every load requested before anything is computed and nothing staged in shared memory.  Scores need one
// shuffle, softmax statistics are per warp (online across tiles), the weighted V sum needs no
// cross-lane reduction.  The four warps of a CTA merge through shared memory, the sixteen CTAs of the
// head through distributed shared memory: each writes its (m, l, o) into the leader CTA's shared
// memory, one cluster barrier, and the leader writes the head's output.  No global scratch, no
// fence, no atomic ticket, no second pass over partial results in L2.
// ------------------------------------------------------------------------------------------------
template <int HD, bool CLUSTER>
__global__ void __launch_bounds__(kAttnThreads) attn_cluster_kernel(AttnParams p) {
    namespace cg = cooperative_groups;
    constexpr int KV4 = HD / 16;                    // 16-byte K loads per lane: half a row
    constexpr int VL = HD / 4;                      // lanes that hold V features (four each)
    __shared__ float q_s[HD], k_s[HD], v_s[HD];
    __shared__ float wm[4], wl[4];
    __shared__ float wo[4][HD];
    __shared__ float cl_m[kClusterCtas], cl_l[kClusterCtas];     // leader only: one slot per CTA of the cluster
    __shared__ float cl_o[kClusterCtas][HD];

    gemvq8::pdl_launch_dependents();
    gemvq8::pdl_wait();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int h = blockIdx.x;
    // CLUSTER: tiles go round-robin to the 16 CTAs of the head's cluster.  Otherwise CTA y owns tile y
    // alone and the head's CTAs merge through global memory (last one to finish, as attn_decode_kernel).
    constexpr int kStride = CLUSTER ? kClusterCtas : (1 << 30);
    const int rank = CLUSTER ? (int)cg::this_cluster().block_rank() : (int)blockIdx.y;
    const int P = (int)*p.d_pos;
    const int T = P + 1;
    const int ntiles = (T + kTile - 1) / kTile;
    if (!CLUSTER && rank >= ntiles) return;
    const int group = p.H / p.Hkv;
    const int kvh = h / group;
    const __half* K = p.kc + (size_t)kvh * p.max_cache * HD;
    const __half* V = p.vc + (size_t)kvh * p.max_cache * HD;
    __half* Kw = p.kc + (size_t)kvh * p.max_cache * HD;
    __half* Vw = p.vc + (size_t)kvh * p.max_cache * HD;
    const int pos16 = lane >> 1, half = lane & 1;

    // first tile's loads go out before RoPE (they do not depend on it)
    uint4 kreg[KV4];
    uint2 vreg[16];
    auto request = [&](int tile) {
        const int base = tile * kTile + warp * 16;
        const int kp = base + pos16;
        if (kp < P) {
            const uint4* src = reinterpret_cast<const uint4*>(K + (size_t)kp * HD + half * (HD / 2));
#pragma unroll
            for (int v = 0; v < KV4; ++v) kreg[v] = ld_stream_v4(src + v);
        }
        if (lane < VL) {
#pragma unroll
            for (int j = 0; j < 16; ++j)
                if (base + j < P) vreg[j] = *reinterpret_cast<const uint2*>(V + (size_t)(base + j) * HD + 4 * lane);
        }
    };
    int tile = rank;
    if (tile < ntiles) request(tile);

    const bool owns_new = CLUSTER ? (ntiles - 1) % kClusterCtas == rank : ntiles - 1 == rank;   // the CTA whose tile holds position P
    rope_into<HD>(p.qkv + (size_t)h * HD, p.rope_tab, p.rope_dim, q_s);
    if (owns_new) {
        rope_into<HD>(p.qkv + (size_t)(p.H + kvh) * HD, p.rope_tab, p.rope_dim, k_s);
        for (int i = tid; i < HD; i += kAttnThreads) v_s[i] = __half2float(p.qkv[(size_t)(p.H + p.Hkv + kvh) * HD + i]);
    }
    __syncthreads();
    if (owns_new && h % group == 0) {
        // Cache op (ops/cache.rs:73-103): the new row goes into the cache for later steps
        for (int i = tid; i < HD; i += kAttnThreads) {
            Kw[(size_t)P * HD + i] = __float2half_rn(k_s[i]);
            Vw[(size_t)P * HD + i] = __float2half_rn(v_s[i]);
        }
    }

    // running softmax state of this warp; o: four features per lane
    float m_run = -INFINITY, l_run = 0.f;
    float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
    for (; tile < ntiles; tile += kStride) {
        const int base = tile * kTile + warp * 16;
        const int kp = base + pos16;
        // ---- scores of the warp's 16 positions
        float dot = 0.f;
        if (kp < T) {
            const float* q = q_s + half * (HD / 2);
            if (kp == P) {
                const float* kk = k_s + half * (HD / 2);
#pragma unroll 8
                for (int i = 0; i < HD / 2; ++i) dot = fmaf(q[i], kk[i], dot);
            } else {
#pragma unroll
                for (int v = 0; v < KV4; ++v) {
                    const __half2* hp = reinterpret_cast<const __half2*>(&kreg[v]);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float2 f = __half22float2(hp[j]);
                        dot = fmaf(q[v * 8 + 2 * j], f.x, dot);
                        dot = fmaf(q[v * 8 + 2 * j + 1], f.y, dot);
                    }
                }
            }
        }
        dot += __shfl_xor_sync(0xffffffffu, dot, 1);
        const float sc = kp < T ? f16r(dot * p.scale) : -INFINITY;     // `.mul(scale).cast(f16)` (attn.rs:142-146)
        const float m_tile = warp_max(sc);
        if (m_tile > -INFINITY) {                                       // the warp has at least one position in this tile
            const float m_new = fmaxf(m_run, m_tile);
            const float corr = expf(m_run - m_new);                     // 0 on the first tile (m_run = -inf)
            const float pe = kp < T ? expf(sc - m_new) : 0.f;
            l_run = l_run * corr + 0.5f * warp_sum(pe);                 // every position sits in two lanes
            o0 *= corr; o1 *= corr; o2 *= corr; o3 *= corr;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const float pj = __shfl_sync(0xffffffffu, pe, 2 * j);
                if (lane < VL && base + j < T) {
                    float2 a, b;
                    if (base + j == P) {
                        a = make_float2(v_s[4 * lane], v_s[4 * lane + 1]);
                        b = make_float2(v_s[4 * lane + 2], v_s[4 * lane + 3]);
                    } else {
                        a = __half22float2(*reinterpret_cast<const __half2*>(&vreg[j].x));
                        b = __half22float2(*reinterpret_cast<const __half2*>(&vreg[j].y));
                    }
                    o0 = fmaf(pj, a.x, o0); o1 = fmaf(pj, a.y, o1);
                    o2 = fmaf(pj, b.x, o2); o3 = fmaf(pj, b.y, o3);
                }
            }
            m_run = m_new;
        }
        if (CLUSTER && tile + kClusterCtas < ntiles) request(tile + kClusterCtas);
    }

    // ---- the four warps of the CTA
    if (lane == 0) { wm[warp] = m_run; wl[warp] = l_run; }
    if (lane < VL) {
        wo[warp][4 * lane] = o0; wo[warp][4 * lane + 1] = o1;
        wo[warp][4 * lane + 2] = o2; wo[warp][4 * lane + 3] = o3;
    }
    __syncthreads();
    const float Mc = fmaxf(fmaxf(wm[0], wm[1]), fmaxf(wm[2], wm[3]));
    float e[4];
#pragma unroll
    for (int w = 0; w < 4; ++w) e[w] = wm[w] > -INFINITY ? expf(wm[w] - Mc) : 0.f;
    if (!CLUSTER) {
        // ---- this CTA's partial to global memory; the last CTA of the head to finish merges
        __shared__ unsigned int ticket;
        __shared__ float wgt_s[kMaxSplits];
        __shared__ float red[4];
        const int max_splits = gridDim.y;
        float* part = p.partial + ((size_t)h * max_splits + rank) * (HD + 2);
        if (tid == 0) {
            part[0] = Mc;
            part[1] = wl[0] * e[0] + wl[1] * e[1] + wl[2] * e[2] + wl[3] * e[3];
        }
        for (int d = tid; d < HD; d += kAttnThreads) part[2 + d] = wo[0][d] * e[0] + wo[1][d] * e[1] + wo[2][d] * e[2] + wo[3][d] * e[3];
        __threadfence();
        __syncthreads();
        if (tid == 0) ticket = atomicAdd(&p.counters[h], 1u);
        __syncthreads();
        if (ticket != (unsigned int)ntiles - 1) return;
        __threadfence();
        const float* hp = p.partial + (size_t)h * max_splits * (HD + 2);
        float mj = -INFINITY, lj = 0.f;
        if (tid < ntiles) {
            mj = __ldcg(hp + tid * (HD + 2));
            lj = __ldcg(hp + tid * (HD + 2) + 1);
        }
        float M = warp_max(mj);
        if (lane == 0) red[warp] = M;
        __syncthreads();
        M = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
        __syncthreads();
        const float wj = tid < ntiles ? expf(mj - M) : 0.f;
        if (tid < ntiles) wgt_s[tid] = wj;
        float L = warp_sum(lj * wj);
        if (lane == 0) red[warp] = L;
        __syncthreads();
        L = red[0] + red[1] + red[2] + red[3];
        for (int d = tid; d < HD; d += kAttnThreads) {
            float o = 0.f;
#pragma unroll 8
            for (int j = 0; j < ntiles; ++j) o = fmaf(__ldcg(hp + j * (HD + 2) + 2 + d), wgt_s[j], o);
            const __half r = __float2half_rn(o / L);
            if (p.ll.local) p.ll.put(h * HD + d, r);
            else p.out[(size_t)h * HD + d] = r;
        }
        if (tid == 0) p.counters[h] = 0;
        return;
    }
    // ---- into the leader's shared memory
    cg::cluster_group cluster = cg::this_cluster();
    float* lm = cluster.map_shared_rank(cl_m, 0);
    float* ll_ = cluster.map_shared_rank(cl_l, 0);
    float* lo = cluster.map_shared_rank(&cl_o[0][0], 0);
    if (tid == 0) {
        lm[rank] = Mc;
        ll_[rank] = wl[0] * e[0] + wl[1] * e[1] + wl[2] * e[2] + wl[3] * e[3];
    }
    for (int d = tid; d < HD; d += kAttnThreads)
        lo[rank * HD + d] = wo[0][d] * e[0] + wo[1][d] * e[1] + wo[2][d] * e[2] + wo[3][d] * e[3];
    cluster.sync();
    if (rank != 0) return;
    float M = -INFINITY;
#pragma unroll
    for (int c = 0; c < kClusterCtas; ++c) M = fmaxf(M, cl_m[c]);
    float L = 0.f;
    float wgt[kClusterCtas];
#pragma unroll
    for (int c = 0; c < kClusterCtas; ++c) {
        wgt[c] = cl_m[c] > -INFINITY ? expf(cl_m[c] - M) : 0.f;
        L = fmaf(cl_l[c], wgt[c], L);
    }
    for (int d = tid; d < HD; d += kAttnThreads) {
        float o = 0.f;
#pragma unroll
        for (int c = 0; c < kClusterCtas; ++c) o = fmaf(cl_o[c][d], wgt[c], o);
        const __half r = __float2half_rn(o / L);
        if (p.ll.local) p.ll.put(h * HD + d, r);     // sharded decoder: this rank's heads -> every rank
        else p.out[(size_t)h * HD + d] = r;
    }
}

__global__ void set_u32_kernel(uint32_t* p, uint32_t v);
__global__ void argmax_advance_kernel(const __half* logits, int n, int32_t* out, uint32_t* d_pos);

// Which attention kernel serves a step at `position` cached entries: 2 = one 16-CTA cluster per head with
// tiles in registers (fastest while a CTA has at most two tiles, i.e. up to 2048 positions), 0 = one CTA
// per tile staged in shared memory (more CTAs in flight for long caches), 1 = tiles in registers with the
// global merge.
int attn_variant(uint32_t position) {
    return position + 1 <= 2u * kClusterCtas * kTile ? 2 : 0;
}

rcu_status launch_attn(rcu_device* dev, const AttnParams& p, int head_dim, bool overlap, int which) {
    if (attn_splits(p.max_cache) > kMaxSplits)
        return rcu_fail(dev, RCU_ERR_UNSUPPORTED, "attn_decode: max_cache %d exceeds %d positions", p.max_cache, kMaxSplits * kTile);
    const size_t smem = 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.H, attn_splits(p.max_cache));
    cfg.blockDim = dim3(kAttnThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = dev->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = overlap ? 1 : 0;
    // Same shared-memory carve-out as the GEMVs around it: an SM that has to change its L1/shared split
    // between consecutive kernels drains first, which costs microseconds per kernel in a decode step.
    static std::once_flag carveout_once;        // handles of different devices may be driven from different host threads
    std::call_once(carveout_once, [] {
        cudaFuncSetAttribute(attn_decode_kernel<64>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        cudaFuncSetAttribute(attn_decode_kernel<96>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        cudaFuncSetAttribute(attn_decode_kernel<128>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        cudaFuncSetAttribute(rope_table_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        cudaFuncSetAttribute(argmax_advance_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        cudaFuncSetAttribute(set_u32_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    });
    if (head_dim != 64 && head_dim != 96 && head_dim != 128)
        return rcu_fail(dev, RCU_ERR_UNSUPPORTED, "attn_decode: head_dim %d (supported: 64, 96, 128)", head_dim);
    static std::atomic<bool> cluster_ok{true};
    if (which == 1 || (which == 2 && cluster_ok.load())) {
        static std::once_flag cluster_once;
        std::call_once(cluster_once, [] {
            cudaFuncSetAttribute(attn_cluster_kernel<64, true>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
            cudaFuncSetAttribute(attn_cluster_kernel<96, true>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
            cudaFuncSetAttribute(attn_cluster_kernel<128, true>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        });
        cudaLaunchConfig_t cc = cfg;
        cudaLaunchAttribute ca[2];
        int na = 0;
        if (which == 2) {
            cc.gridDim = dim3(p.H, kClusterCtas);
            ca[na].id = cudaLaunchAttributeClusterDimension;
            ca[na].val.clusterDim.x = 1;
            ca[na].val.clusterDim.y = kClusterCtas;
            ca[na].val.clusterDim.z = 1;
            ++na;
        }
        if (overlap) ca[na++] = attr[0];
        cc.attrs = ca;
        cc.numAttrs = na;
        cudaError_t e;
        if (which == 2)
            e = head_dim == 64 ? cudaLaunchKernelEx(&cc, attn_cluster_kernel<64, true>, p)
                : head_dim == 96 ? cudaLaunchKernelEx(&cc, attn_cluster_kernel<96, true>, p)
                                 : cudaLaunchKernelEx(&cc, attn_cluster_kernel<128, true>, p);
        else
            e = head_dim == 64 ? cudaLaunchKernelEx(&cc, attn_cluster_kernel<64, false>, p)
                : head_dim == 96 ? cudaLaunchKernelEx(&cc, attn_cluster_kernel<96, false>, p)
                                 : cudaLaunchKernelEx(&cc, attn_cluster_kernel<128, false>, p);
        if (e == cudaSuccess) {
            RCU_LAUNCH_CHECK(dev);
            return RCU_OK;
        }
        cudaGetLastError();          // clusters of 16 not available here: use the staged kernel from now on
        cluster_ok.store(false);
    }
    switch (head_dim) {
        case 64: RCU_CUDA(dev, cudaLaunchKernelEx(&cfg, attn_decode_kernel<64>, p)); break;
        case 96: RCU_CUDA(dev, cudaLaunchKernelEx(&cfg, attn_decode_kernel<96>, p)); break;
        default: RCU_CUDA(dev, cudaLaunchKernelEx(&cfg, attn_decode_kernel<128>, p)); break;
    }
    RCU_LAUNCH_CHECK(dev);
    return RCU_OK;
}

__global__ void set_u32_kernel(uint32_t* p, uint32_t v) { *p = v; }

__device__ __forceinline__ void argmax_advance_body(const __half* logits, int n, int32_t* out, uint32_t* d_pos);

// arg-max over f16 logits (first maximum wins, as the host loop in phi3/generate.rs:103-108) and
// position advance (KVCache::update(1)).
__global__ void __launch_bounds__(1024) argmax_advance_kernel(const __half* logits, int n, int32_t* out, uint32_t* d_pos) {
    argmax_advance_body(logits, n, out, d_pos);
}

// The sharded decoder's last kernel: takes every rank's slice of the logits from the exchange window
// (waiting for the words still in flight), writes the gathered vector to the caller's buffer, takes
// the arg-max and advances the position and the step counter.
__global__ void __launch_bounds__(1024) argmax_advance_gathered_kernel(gemvq8::LLSource src, __half* logits_out, int n, int32_t* out,
                                                                        uint32_t* d_pos, unsigned int* d_step) {
    const uint32_t tag = src.seq.tag();
    const int nvec = n >> 2;                     // n % 8 == 0 (checked at creation)
    for (int i = threadIdx.x; i < nvec; i += 2 * blockDim.x) {
        const bool second = i + (int)blockDim.x < nvec;
        uint4 a = gemvq8::ll_load4(src.words + 4 * i);
        uint4 b = a;
        if (second) b = gemvq8::ll_load4(src.words + 4 * (i + blockDim.x));
        gemvq8::ll_wait4(src.words, i, tag, src.status, a);
        reinterpret_cast<uint2*>(logits_out)[i] = gemvq8::ll_pack4(a);
        if (second) {
            gemvq8::ll_wait4(src.words, i + blockDim.x, tag, src.status, b);
            reinterpret_cast<uint2*>(logits_out)[i + blockDim.x] = gemvq8::ll_pack4(b);
        }
    }
    __syncthreads();
    argmax_advance_body(logits_out, n, out, d_pos);
    __syncthreads();          // every thread has read the step counter (through tag()) before it moves
    if (threadIdx.x == 0) *d_step += 1;
}

__device__ __forceinline__ void argmax_advance_body(const __half* logits, int n, int32_t* out, uint32_t* d_pos) {
    __shared__ float bv[32];
    __shared__ int bi[32];
    if (out) {
        float best = -INFINITY;
        int idx = 0x7fffffff;
        for (int i = threadIdx.x; i < n; i += blockDim.x) {
            const float v = __half2float(logits[i]);
            if (v > best || (v == best && i < idx)) { best = v; idx = i; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
            if (ov > best || (ov == best && oi < idx)) { best = ov; idx = oi; }
        }
        if ((threadIdx.x & 31) == 0) { bv[threadIdx.x >> 5] = best; bi[threadIdx.x >> 5] = idx; }
        __syncthreads();
        if (threadIdx.x < 32) {
            best = threadIdx.x < (blockDim.x >> 5) ? bv[threadIdx.x] : -INFINITY;
            idx = threadIdx.x < (blockDim.x >> 5) ? bi[threadIdx.x] : 0x7fffffff;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, best, o);
                const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
                if (ov > best || (ov == best && oi < idx)) { best = ov; idx = oi; }
            }
            if (threadIdx.x == 0) *out = idx;
        }
    }
    if (threadIdx.x == 0) *d_pos += 1;
}

// Programmatic dependent launch between the kernels of a step (RCU_NO_PDL=1 turns it off).
bool pdl_enabled() {
    static bool on = std::getenv("RCU_NO_PDL") == nullptr;
    return on;
}

template <class Pro, class Epi>
rcu_status gemv(rcu_device* dev, int weight_dt, const void* w, const Pro& pro, const Epi& epi, int N, int K) {
    const int8_t* qs = (const int8_t*)w;
    const void* sc = (const char*)w + align256((uint64_t)N * K);
    const bool ov = pdl_enabled();
    if (weight_dt == RCU_Q8_0H) return gemvq8::launch<__half, __half, 2>(dev, qs, sc, pro, epi, N, K, ov, 2, true);
    return gemvq8::launch<float, __half, 2>(dev, qs, sc, pro, epi, N, K, ov, 2, true);
}

// per-device scratch for the standalone attention entry point
struct AttnScratch {
    float* partial = nullptr;
    unsigned int* counters = nullptr;
    float* rope_tab = nullptr;
    uint32_t* d_pos = nullptr;
    size_t partial_floats = 0;
    int heads = 0;                 // entries of `counters`
};

void free_attn_scratch(void* p) {
    AttnScratch* s = (AttnScratch*)p;
    cudaFree(s->partial);
    cudaFree(s->counters);
    cudaFree(s->rope_tab);
    cudaFree(s->d_pos);
    delete s;
}

rcu_status alloc_attn_scratch(rcu_device* dev, int H, size_t partial_floats, AttnScratch* s) {
    s->partial_floats = partial_floats;
    s->heads = H;
    RCU_CUDA(dev, cudaMalloc(&s->partial, s->partial_floats * sizeof(float)));
    RCU_CUDA(dev, cudaMalloc(&s->counters, (size_t)H * sizeof(unsigned int)));
    RCU_CUDA(dev, cudaMalloc(&s->rope_tab, 256 * sizeof(float)));
    RCU_CUDA(dev, cudaMalloc(&s->d_pos, sizeof(uint32_t)));
    RCU_CUDA(dev, cudaMemsetAsync(s->counters, 0, (size_t)H * sizeof(unsigned int), dev->stream));
    return RCU_OK;
}

}  // namespace

struct rcu_decoder {
    rcu_device* dev;
    rcu_decoder_config cfg;
    std::vector<rcu_decoder_layer> layers;
    const void* tok_embd;
    const void* out_norm;
    const void* lm_head;
    AttnScratch scratch;
    __half *x = nullptr, *qkv = nullptr, *attn = nullptr, *act = nullptr;
    uint32_t position = 0;
    uint32_t kernels_per_step = 0;
    uint64_t steps = 0;
    // sharded across the GPUs of a node (null: single GPU).  cfg holds the whole model's sizes.
    rcu_comm* comm = nullptr;
    unsigned int* d_step = nullptr;       // steps taken, on the device: the exchanges' sequence numbers derive from it
    // all layers and the lm_head as one persistent data-flow kernel (decode_flow.cuh); flow_grid == 0: not in use
    flow::LayerPtrs* d_layer_ptrs = nullptr;
    flow::Params fp;
    int flow_grid = 0, flow_kmax = 0, flow_warps = 0;
    size_t flow_smem = 0;
    uint32_t* own_window = nullptr;       // single GPU: the exchange window lives here (no peers)
    size_t slot_words = 0;
    unsigned long long* flow_partial = nullptr;
    unsigned long long* d_prof = nullptr; // per-job time stamps of one step (rcu_decoder_profile)
    // captured step
    cudaGraphExec_t graph_exec = nullptr;
    const int32_t* cap_token = nullptr;
    void* cap_logits = nullptr;
    int32_t* cap_argmax = nullptr;
    int cap_variant = -1;                 // attention kernel the captured step launches (it depends on the cached length)
};

namespace {

// Embedding row -> tagged words of the x exchange (the flow kernel's first input), this rank only.
__global__ void publish_words_kernel(const __half* x, int n, gemvq8::LLPush push) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) push.put(i, x[i]);
}

template <int HD, class ScaleT, int NW>
bool flow_fits_t(size_t smem) {
    auto kern = flow::decode_flow_kernel<HD, ScaleT, NW>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return false;
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, (NW + 1) * 32, smem) != cudaSuccess) return false;
    return n >= 1;
}

// Instantiations of the data-flow kernel: head_dim 64 / 96 / 128, f16 or f32 block scales.  Seven consumer warps:
// with the requester warp that is eight warps, which leaves a thread 255 registers (nine warps are allotted
// registers as twelve, 168 per thread, and the item loops spill: measured 630 tokens/s against 730).
constexpr int kFlowWarps = 7;
#define RCU_FLOW_DISPATCH(HD_, HALF_, NW_, CALL) RCU_FLOW_DISPATCH_HD(HD_, HALF_, kFlowWarps, CALL)
#define RCU_FLOW_DISPATCH_HD(HD_, HALF_, NWC, CALL)                                                         \
    do {                                                                                                    \
        if ((HD_) == 64) { if (HALF_) { CALL(64, __half, NWC); } else { CALL(64, float, NWC); } }           \
        else if ((HD_) == 96) { if (HALF_) { CALL(96, __half, NWC); } else { CALL(96, float, NWC); } }      \
        else { if (HALF_) { CALL(128, __half, NWC); } else { CALL(128, float, NWC); } }                     \
    } while (0)

template <int HD> size_t flow_union_bytes(int kmax, int nw) {
    (void)nw;
    return flow::union_bytes<HD, kFlowWarps>(kmax);
}

// Exchange slots of the window (each slot_words 32-bit words): the residual stream alternates between two.
enum { SLOT_X0 = 0, SLOT_X1 = 1, SLOT_Q = 2, SLOT_A = 3, SLOT_F = 4, SLOT_LOGITS = 5 };

// Describes the decode step to the data-flow kernel if this model and device allow it: rows of whole
// 256-element runs (the rings' alignment rule), every matrix with at least one item group per CTA, at least
// eight warps per local head, cooperative launch.  Otherwise the decoder keeps the kernel-per-phase step.
void setup_flow(rcu_decoder* d) {
    rcu_device* dev = d->dev;
    const rcu_decoder_config& c = d->cfg;
    const int W = d->comm ? d->comm->world : 1, r = d->comm ? d->comm->rank : 0;
    const int HD = (int)c.head_dim, L = (int)c.n_layers;
    const int D = (int)c.d_model, Dl = D / W, ffn = (int)c.ffn, ffnl = ffn / W, Vl = (int)c.vocab / W;
    const int H = (int)c.n_heads, Hl = H / W, Hkvl = (int)c.n_kv_heads / W;
    const int qkv_nl = (Hl + 2 * Hkvl) * HD, A = H * HD;
    const int ss = c.weight_dt == RCU_Q8_0H ? 2 : 4;
    // RCU_DECODE_FLOW=0 forces the kernel-per-phase step, =1 the data-flow kernel wherever it is eligible.  By default
    // eight ranks and more take the kernel-per-phase step: a rank then streams only 2 us of weights per layer, and what
    // one persistent kernel saves on launches no longer pays for its hand-overs across NVLink (measured on Phi-3-mini:
    // 821 tokens/s for the data-flow kernel on 8 ranks against 964; on 4 ranks 948 against 941).
    static const int mode = [] { const char* e = std::getenv("RCU_DECODE_FLOW"); return e ? std::atoi(e) : -1; }();
    if (mode == 0 || (mode < 0 && W >= 8)) return;
    int coop = 0;
    if (cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev->ordinal) != cudaSuccess || !coop) return;
    const int grid = dev->sm_count;
    const int NW = kFlowWarps;
    const long long GW = (long long)grid * NW;
    if (Hl < 1 || Hl > grid || (int)c.rope_dim > flow::kMaxRope || L > flow::kMaxLayersShared) return;
    if (Dl % 4 || ffnl % 4 || Vl % 4 || (Hl * HD) % 4) return;          // consumers take four words per load
    const size_t widest = (size_t)std::max(std::max(D, ffn), std::max((int)c.vocab, std::max(A, qkv_nl)));
    const size_t slot_words = d->comm ? d->comm->local.slot_bytes / 4 : widest;
    if (slot_words < widest) return;

    auto off_of = [&](int slot, size_t elem) { return (uint32_t)((size_t)slot * slot_words + elem); };
    flow::Params& p = d->fp;
    p = flow::Params{};
    bool ok = true;
    int kmax = std::max(std::max(D, ffn), A), slot_bytes = 2 * 16 * HD * 2;      // an attention item: 16 positions of K and V
    // shared memory left for the rings, and the item size that lets every warp hold two items
    const size_t ub0 = HD == 64 ? flow_union_bytes<64>(kmax, NW) : HD == 96 ? flow_union_bytes<96>(kmax, NW) : flow_union_bytes<128>(kmax, NW);
    const size_t fixed = flow::union_off(NW, L) + ub0;
    if (fixed + (size_t)NW * 2 * slot_bytes > (size_t)dev->smem_optin) return;
    const int slot_target = (int)(((size_t)dev->smem_optin - fixed) / ((size_t)NW * 2)) & ~127;
    auto describe = [&](int kind, int n_units, int rows, int K, int unit, bool rms) {
        flow::KindDesc& k = p.kd[kind];
        ringq8::Job j{nullptr, nullptr, n_units, n_units, K, 1, K, 1, ss};
        if (!ringq8::plan_job(&j, unit, slot_target)) { ok = false; return; }
        while (j.ri > 1 && (n_units + j.ri - 1) / j.ri < grid) j.ri >>= 1;                   // every CTA takes part in every matrix
        const long long n_groups = (n_units + j.ri - 1) / j.ri;
        if (n_groups < grid || n_groups * GW >= (1ll << 31)) ok = false;
        if ((kind == flow::K_O || kind == flow::K_DOWN) && ((n_groups + GW - 1) / GW + 1) * j.ri > 32) ok = false;   // a lane per residual
        k.n_units = n_units; k.K = K; k.ri = j.ri; k.kc = j.kc; k.nc = j.nc; k.unit = unit;
        k.scales_off = (uint32_t)align256((uint64_t)rows * K);
        if (align256((uint64_t)rows * K) >= (1ull << 32)) ok = false;
        k.rms = rms ? 1 : 0;
        slot_bytes = std::max(slot_bytes, ringq8::item_bytes(j, unit));
    };
    const uint32_t per_x0 = (uint32_t)L + 1u, per = (uint32_t)L;
    describe(flow::K_QKV, qkv_nl, qkv_nl, D, 1, true);
    describe(flow::K_O, Dl, Dl, A, 1, false);
    describe(flow::K_GATE_UP, ffnl, 2 * ffnl, D, 2, true);
    describe(flow::K_DOWN, Dl, Dl, ffn, 1, false);
    describe(flow::K_HEAD, Vl, Vl, D, 1, true);
    if (!ok) return;
    {
        flow::KindDesc& q = p.kd[flow::K_QKV];       // x (embedding or the previous layer's down) -> this rank's qkv rows
        q.in_off = off_of(SLOT_X0, 0); q.in_per_step = per_x0; q.in_mul = 1; q.in_add = 0;
        q.out_off = off_of(SLOT_Q, 0); q.out_per_step = per; q.out_mul = 1; q.out_add = 0;
        flow::KindDesc& o = p.kd[flow::K_O];         // head outputs -> x + o (second x slot)
        o.in_off = off_of(SLOT_A, 0); o.in_per_step = per; o.in_mul = 1; o.in_add = 0;
        o.out_off = off_of(SLOT_X1, (size_t)r * Dl); o.out_per_step = per; o.out_mul = 1; o.out_add = 0;
        o.res_off = off_of(SLOT_X0, (size_t)r * Dl);
        o.push = 1;
        flow::KindDesc& g = p.kd[flow::K_GATE_UP];
        g.in_off = off_of(SLOT_X1, 0); g.in_per_step = per; g.in_mul = 1; g.in_add = 0;
        g.out_off = off_of(SLOT_F, (size_t)r * ffnl); g.out_per_step = per; g.out_mul = 1; g.out_add = 0;
        g.push = 1;
        flow::KindDesc& dn = p.kd[flow::K_DOWN];     // MLP activations -> x + down (first x slot again: the next layer's input)
        dn.in_off = off_of(SLOT_F, 0); dn.in_per_step = per; dn.in_mul = 1; dn.in_add = 0;
        dn.out_off = off_of(SLOT_X0, (size_t)r * Dl); dn.out_per_step = per_x0; dn.out_mul = 1; dn.out_add = 1;
        dn.res_off = off_of(SLOT_X1, (size_t)r * Dl);
        dn.push = 1;
        flow::KindDesc& hd = p.kd[flow::K_HEAD];
        hd.in_off = off_of(SLOT_X0, 0); hd.in_per_step = per_x0; hd.in_mul = 0; hd.in_add = L;
        hd.out_off = off_of(SLOT_LOGITS, (size_t)r * Vl); hd.out_per_step = 1; hd.out_mul = 0; hd.out_add = 0;
        hd.push = 1;
    }
    slot_bytes = (slot_bytes + 127) & ~127;
    if (fixed + (size_t)NW * 2 * slot_bytes > (size_t)dev->smem_optin) return;
    int depth = (int)(((size_t)dev->smem_optin - fixed) / ((size_t)NW * slot_bytes));
    depth = std::min(depth, ringq8::kMaxDepth);
    const size_t smem = fixed + (size_t)NW * depth * slot_bytes;
    const bool half = c.weight_dt == RCU_Q8_0H;
    bool fits = false;
#define RCU_FLOW_FITS(HD_, T_, NW_) fits = flow_fits_t<HD_, T_, NW_>(smem)
    RCU_FLOW_DISPATCH(HD, half, NW, RCU_FLOW_FITS);
#undef RCU_FLOW_FITS
    if (!fits) { cudaGetLastError(); return; }

    const int part_stride = std::min(grid / Hl, flow::kMaxCtasPerHead);       // a head spreads over at most this many CTAs
    const size_t part_words = (size_t)Hl * part_stride * (HD + 2);
    std::vector<flow::LayerPtrs> host(L);
    for (int li = 0; li < L; ++li) {
        const rcu_decoder_layer& Lw = d->layers[li];
        host[li] = flow::LayerPtrs{{(const int8_t*)Lw.qkv, (const int8_t*)Lw.o, (const int8_t*)Lw.gate_up, (const int8_t*)Lw.down},
                                   (const float*)Lw.attn_norm, (const float*)Lw.ffn_norm, (__half*)Lw.k_cache, (__half*)Lw.v_cache};
    }
    if (!d->comm) {
        if (cudaMalloc(&d->own_window, (size_t)rcu_window::kSlots * slot_words * 4) != cudaSuccess) { cudaGetLastError(); return; }
        cudaMemsetAsync(d->own_window, 0, (size_t)rcu_window::kSlots * slot_words * 4, dev->stream);
    }
    if (cudaMalloc(&d->d_layer_ptrs, host.size() * sizeof(flow::LayerPtrs)) != cudaSuccess || cudaMalloc(&d->flow_partial, part_words * sizeof(unsigned long long)) != cudaSuccess) {
        cudaGetLastError();
        return;
    }
    cudaMemsetAsync(d->flow_partial, 0, part_words * sizeof(unsigned long long), dev->stream);
    cudaMemcpyAsync(d->d_layer_ptrs, host.data(), host.size() * sizeof(flow::LayerPtrs), cudaMemcpyHostToDevice, dev->stream);
    cudaStreamSynchronize(dev->stream);     // `host` goes out of scope
    p.layers = d->d_layer_ptrs;
    p.n_layers = L;
    p.head_w = (const int8_t*)d->lm_head;
    p.out_norm = (const float*)d->out_norm;
    p.win = d->comm ? reinterpret_cast<uint32_t*>(d->comm->local.base) : d->own_window;
    p.n_peers = 0;
    for (int q = 0; q < W; ++q)
        if (q != r) p.peer_win[p.n_peers++] = reinterpret_cast<uint32_t*>(d->comm->peers[q].base);
    p.d_step = d->d_step;
    p.status = dev->d_status;
    p.scale_size = ss;
    p.H = Hl; p.Hkv = Hkvl; p.max_cache = (int)c.max_cache; p.rope_dim = (int)c.rope_dim;
    p.scale = 1.0f / sqrtf((float)HD);
    p.d_pos = d->scratch.d_pos;
    p.rope_tab = d->scratch.rope_tab;
    p.q_off = off_of(SLOT_Q, 0); p.q_per_step = per;
    p.a_off = off_of(SLOT_A, 0); p.a_per_step = per;
    p.a_rank_off = r * Hl * HD;
    p.partial = d->flow_partial;
    p.part_stride = part_stride;
    p.slot_bytes = slot_bytes;
    p.depth = depth;
    p.eps = c.rms_eps;
    p.prof = nullptr;
    d->slot_words = slot_words;
    d->flow_grid = grid;
    d->flow_warps = NW;
    d->flow_kmax = kmax;
    d->flow_smem = smem;
}

template <int HD, class ScaleT, int NW>
rcu_status launch_flow_t(rcu_decoder* d) {
    rcu_device* dev = d->dev;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(d->flow_grid);
    cfg.blockDim = dim3((NW + 1) * 32);
    cfg.dynamicSmemBytes = d->flow_smem;
    cfg.stream = dev->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;      // every CTA resident at once: they wait for each other's results
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    RCU_CUDA(dev, cudaLaunchKernelEx(&cfg, flow::decode_flow_kernel<HD, ScaleT, NW>, d->fp, d->flow_kmax));
    RCU_LAUNCH_CHECK(dev);
    return RCU_OK;
}

rcu_status launch_flow(rcu_decoder* d) {
    const bool half = d->cfg.weight_dt == RCU_Q8_0H;
    rcu_status st = RCU_OK;
#define RCU_FLOW_LAUNCH(HD_, T_, NW_) st = launch_flow_t<HD_, T_, NW_>(d)
    RCU_FLOW_DISPATCH((int)d->cfg.head_dim, half, d->flow_warps, RCU_FLOW_LAUNCH);
#undef RCU_FLOW_LAUNCH
    return st;
}

// One decode step through the data-flow kernel: rope table, embedding row -> tagged words, the kernel
// (all layers and the lm_head), then the gathered logits, arg-max and the position / step counters.
rcu_status run_sequence_flow(rcu_decoder* d, const int32_t* token_dev, void* logits_dev, int32_t* argmax_dev) {
    rcu_device* dev = d->dev;
    const rcu_decoder_config& c = d->cfg;
    rope_table_kernel<<<1, 128, 0, dev->stream>>>(d->scratch.d_pos, logf(c.rope_base), (int)c.rope_dim / 2, d->scratch.rope_tab);
    RCU_LAUNCH_CHECK(dev);
    rcu_tensor table{c.weight_dt, 2, {c.vocab, c.d_model, 1, 1}, const_cast<void*>(d->tok_embd)};
    rcu_tensor ids{RCU_I32, 1, {1, 1, 1, 1}, const_cast<int32_t*>(token_dev)};
    rcu_tensor xrow{RCU_F16, 2, {1, c.d_model, 1, 1}, d->x};
    rcu_status st;
    if (c.weight_dt == RCU_Q8_0H) {
        st = rcu_index_select(dev, &table, &ids, 0, &xrow);
    } else {
        rcu_tensor x32{RCU_F32, 2, {1, c.d_model, 1, 1}, d->act};
        st = rcu_index_select(dev, &table, &ids, 0, &x32);
        if (st == RCU_OK) st = rcu_cast(dev, &x32, &xrow);
    }
    if (st != RCU_OK) return st;
    gemvq8::LLPush emb{};
    emb.local = d->fp.win + (size_t)SLOT_X0 * d->slot_words;
    emb.n_peers = 0;
    emb.seq = gemvq8::LLSeq{d->d_step, c.n_layers + 1u, 0u};
    publish_words_kernel<<<(c.d_model + 255) / 256, 256, 0, dev->stream>>>(d->x, (int)c.d_model, emb);
    RCU_LAUNCH_CHECK(dev);
    st = launch_flow(d);
    if (st != RCU_OK) return st;
    gemvq8::LLSource lg{d->fp.win + (size_t)SLOT_LOGITS * d->slot_words, gemvq8::LLSeq{d->d_step, 1u, 0u}, dev->d_status};
    argmax_advance_gathered_kernel<<<1, 1024, 0, dev->stream>>>(lg, (__half*)logits_dev, (int)c.vocab, argmax_dev, d->scratch.d_pos, d->d_step);
    RCU_LAUNCH_CHECK(dev);
    return RCU_OK;
}

rcu_status run_sequence(rcu_decoder* d, const int32_t* token_dev, void* logits_dev, int32_t* argmax_dev) {
    rcu_device* dev = d->dev;
    const rcu_decoder_config& c = d->cfg;
    const int D = (int)c.d_model, H = (int)c.n_heads, Hkv = (int)c.n_kv_heads, HD = (int)c.head_dim;
    const int qkv_n = (H + 2 * Hkv) * HD;
    rope_table_kernel<<<1, 128, 0, dev->stream>>>(d->scratch.d_pos, logf(c.rope_base), (int)c.rope_dim / 2, d->scratch.rope_tab);
    RCU_LAUNCH_CHECK(dev);
    // embedding: dequantising row gather (ratchet-nn/src/embedding.rs:15-25)
    rcu_tensor table{c.weight_dt, 2, {c.vocab, c.d_model, 1, 1}, const_cast<void*>(d->tok_embd)};
    rcu_tensor ids{RCU_I32, 1, {1, 1, 1, 1}, const_cast<int32_t*>(token_dev)};
    rcu_tensor xrow{RCU_F16, 2, {1, c.d_model, 1, 1}, d->x};
    rcu_status st;
    if (c.weight_dt == RCU_Q8_0H) {
        st = rcu_index_select(dev, &table, &ids, 0, &xrow);
    } else {
        // Q8_0F tables gather to f32 (DType::activation_dt); stage through qkv's buffer and cast
        rcu_tensor x32{RCU_F32, 2, {1, c.d_model, 1, 1}, d->act};
        st = rcu_index_select(dev, &table, &ids, 0, &x32);
        if (st == RCU_OK) st = rcu_cast(dev, &x32, &xrow);
    }
    if (st != RCU_OK) return st;
    {
        for (uint32_t li = 0; li < c.n_layers; ++li) {
            const rcu_decoder_layer& L = d->layers[li];
            st = gemv(dev, c.weight_dt, L.qkv, gemvq8::RmsNormPrologueH{d->x, (const float*)L.attn_norm, c.rms_eps},
                      gemvq8::PlainEpilogue<__half>{nullptr, d->qkv}, qkv_n, D);
            if (st != RCU_OK) return st;
            AttnParams ap{d->qkv, (__half*)L.k_cache, (__half*)L.v_cache, H, Hkv, (int)c.max_cache, (int)c.rope_dim,
                          d->scratch.d_pos, d->scratch.rope_tab, 1.0f / sqrtf((float)HD), d->scratch.partial, d->scratch.counters, d->attn};
            st = launch_attn(dev, ap, HD, pdl_enabled(), attn_variant(d->position));
            if (st != RCU_OK) return st;
            st = gemv(dev, c.weight_dt, L.o, gemvq8::PlainPrologue<__half>{d->attn}, gemvq8::ResidualEpilogueH{d->x, d->x}, D, H * HD);
            if (st != RCU_OK) return st;
            st = gemv(dev, c.weight_dt, L.gate_up, gemvq8::RmsNormPrologueH{d->x, (const float*)L.ffn_norm, c.rms_eps},
                      gemvq8::SiluGateEpilogueH{d->act}, 2 * (int)c.ffn, D);
            if (st != RCU_OK) return st;
            st = gemv(dev, c.weight_dt, L.down, gemvq8::PlainPrologue<__half>{d->act}, gemvq8::ResidualEpilogueH{d->x, d->x}, D, (int)c.ffn);
            if (st != RCU_OK) return st;
        }
    }
    st = gemv(dev, c.weight_dt, d->lm_head, gemvq8::RmsNormPrologueH{d->x, (const float*)d->out_norm, c.rms_eps},
              gemvq8::PlainEpilogue<__half>{nullptr, (__half*)logits_dev}, (int)c.vocab, D);
    if (st != RCU_OK) return st;
    argmax_advance_kernel<<<1, 1024, 0, dev->stream>>>((const __half*)logits_dev, (int)c.vocab, argmax_dev, d->scratch.d_pos);
    RCU_LAUNCH_CHECK(dev);
    return RCU_OK;
}

// One decode step with every Linear sharded by output rows over the ranks of `d->comm`.  Each output
// vector is all-gathered by the kernel that produces it: results go, element by element, as tagged
// words into every rank's window (gemvq8::LLPush), and the next kernel's prologue takes them from its
// own window, waiting for the words still in flight (gemvq8::LL*PrologueH):
//   qkv rows of this rank's heads -> attention on those heads (its own slice of the KV cache)
//     -> head outputs to all ranks        [slot 1, exchange 2 li]
//   o rows + residual    -> x to all      [slot 0, exchange 2 li]
//   gate/up rows + SiLU  -> act to all    [slot 1, exchange 2 li + 1]
//   down rows + residual -> x to all      [slot 0, exchange 2 li + 1]
//   lm_head rows         -> logits to all [slot 2, one exchange per step]
// Every output element is computed by one rank with the arithmetic of the single-GPU step, so the
// gathered vectors are bit-identical to it.  Slot 0 always holds x: a rank updates its own rows in
// place and peers overwrite only theirs.  A place in a window is rewritten only by an exchange that
// cannot start before every reader of its previous contents has finished: each exchange needs results
// from all CTAs of the producing kernel on every rank, and a CTA reads its inputs before it produces.
rcu_status run_sequence_sharded(rcu_decoder* d, const int32_t* token_dev, void* logits_dev, int32_t* argmax_dev) {
    rcu_device* dev = d->dev;
    rcu_comm* cm = d->comm;
    const rcu_decoder_config& c = d->cfg;
    const int W = cm->world, r = cm->rank;
    const int D = (int)c.d_model, HD = (int)c.head_dim, L = (int)c.n_layers;
    const int H = (int)c.n_heads, Hl = H / W, Hkvl = (int)c.n_kv_heads / W;
    const int qkv_nl = (Hl + 2 * Hkvl) * HD, Dl = D / W, ffn = (int)c.ffn, ffnl = ffn / W, Vl = (int)c.vocab / W;
    auto words = [&](const rcu_window::Window& w, int slot) { return reinterpret_cast<uint32_t*>(w.slot(slot)); };
    auto make_push = [&](int slot, size_t elem_off, unsigned per_step, unsigned idx) {
        gemvq8::LLPush p{};
        p.local = words(cm->local, slot) + elem_off;
        p.n_peers = 0;
        for (int q = 0; q < W; ++q)
            if (q != r) p.peer[p.n_peers++] = words(cm->peers[q], slot) + elem_off;
        p.seq = gemvq8::LLSeq{d->d_step, per_step, idx};
        return p;
    };
    auto make_src = [&](int slot, unsigned per_step, unsigned idx) {
        return gemvq8::LLSource{words(cm->local, slot), gemvq8::LLSeq{d->d_step, per_step, idx}, dev->d_status};
    };
    const unsigned per = 2u * L;      // exchanges per step on slot 0 and on slot 1
    rope_table_kernel<<<1, 128, 0, dev->stream>>>(d->scratch.d_pos, logf(c.rope_base), (int)c.rope_dim / 2, d->scratch.rope_tab);
    RCU_LAUNCH_CHECK(dev);
    // embedding: every rank holds the table and gathers the same row into its own x
    rcu_tensor table{c.weight_dt, 2, {c.vocab, c.d_model, 1, 1}, const_cast<void*>(d->tok_embd)};
    rcu_tensor ids{RCU_I32, 1, {1, 1, 1, 1}, const_cast<int32_t*>(token_dev)};
    rcu_tensor xrow{RCU_F16, 2, {1, c.d_model, 1, 1}, d->x};
    rcu_status st;
    if (c.weight_dt == RCU_Q8_0H) {
        st = rcu_index_select(dev, &table, &ids, 0, &xrow);
    } else {
        rcu_tensor x32{RCU_F32, 2, {1, c.d_model, 1, 1}, d->act};
        st = rcu_index_select(dev, &table, &ids, 0, &x32);
        if (st == RCU_OK) st = rcu_cast(dev, &x32, &xrow);
    }
    if (st != RCU_OK) return st;
    for (int li = 0; li < L; ++li) {
        const rcu_decoder_layer& Lw = d->layers[li];
        const gemvq8::PlainEpilogue<__half> to_qkv{nullptr, d->qkv};
        if (li == 0)   // x is the embedding row, an ordinary vector
            st = gemv(dev, c.weight_dt, Lw.qkv, gemvq8::RmsNormPrologueH{d->x, (const float*)Lw.attn_norm, c.rms_eps}, to_qkv, qkv_nl, D);
        else
            st = gemv(dev, c.weight_dt, Lw.qkv,
                      gemvq8::LLRmsNormPrologueH{make_src(0, per, 2u * (li - 1) + 1u), (const float*)Lw.attn_norm, c.rms_eps}, to_qkv, qkv_nl, D);
        if (st != RCU_OK) return st;
        AttnParams ap{d->qkv, (__half*)Lw.k_cache, (__half*)Lw.v_cache, Hl, Hkvl, (int)c.max_cache, (int)c.rope_dim,
                      d->scratch.d_pos, d->scratch.rope_tab, 1.0f / sqrtf((float)HD), d->scratch.partial, d->scratch.counters,
                      nullptr, make_push(1, (size_t)r * Hl * HD, per, 2u * li)};
        st = launch_attn(dev, ap, HD, pdl_enabled(), attn_variant(d->position));
        if (st != RCU_OK) return st;
        {
            gemvq8::LLResidualEpilogueH epi{li == 0 ? d->x + (size_t)r * Dl : nullptr, words(cm->local, 0) + (size_t)r * Dl,
                                            make_push(0, (size_t)r * Dl, per, 2u * li)};
            st = gemv(dev, c.weight_dt, Lw.o, gemvq8::LLPlainPrologueH{make_src(1, per, 2u * li)}, epi, Dl, H * HD);
            if (st != RCU_OK) return st;
        }
        {
            gemvq8::LLSiluGateEpilogueH epi{make_push(1, (size_t)r * ffnl, per, 2u * li + 1u)};
            st = gemv(dev, c.weight_dt, Lw.gate_up, gemvq8::LLRmsNormPrologueH{make_src(0, per, 2u * li), (const float*)Lw.ffn_norm, c.rms_eps},
                      epi, 2 * ffnl, D);
            if (st != RCU_OK) return st;
        }
        {
            gemvq8::LLResidualEpilogueH epi{nullptr, words(cm->local, 0) + (size_t)r * Dl, make_push(0, (size_t)r * Dl, per, 2u * li + 1u)};
            st = gemv(dev, c.weight_dt, Lw.down, gemvq8::LLPlainPrologueH{make_src(1, per, 2u * li + 1u)}, epi, Dl, ffn);
            if (st != RCU_OK) return st;
        }
    }
    {
        gemvq8::LLPlainEpilogueH epi{make_push(2, (size_t)r * Vl, 1u, 0u)};
        st = gemv(dev, c.weight_dt, d->lm_head,
                  gemvq8::LLRmsNormPrologueH{make_src(0, per, 2u * (L - 1) + 1u), (const float*)d->out_norm, c.rms_eps}, epi, Vl, D);
        if (st != RCU_OK) return st;
    }
    argmax_advance_gathered_kernel<<<1, 1024, 0, dev->stream>>>(make_src(2, 1u, 0u), (__half*)logits_dev, (int)c.vocab, argmax_dev,
                                                                 d->scratch.d_pos, d->d_step);
    RCU_LAUNCH_CHECK(dev);
    return RCU_OK;
}

rcu_status run_step(rcu_decoder* d, const int32_t* token_dev, void* logits_dev, int32_t* argmax_dev) {
    if (d->flow_grid > 0) return run_sequence_flow(d, token_dev, logits_dev, argmax_dev);
    return d->comm ? run_sequence_sharded(d, token_dev, logits_dev, argmax_dev) : run_sequence(d, token_dev, logits_dev, argmax_dev);
}

// Validation and buffers shared by the single-GPU and the sharded decoder (`cfg` holds this rank's head counts).
rcu_status decoder_alloc(rcu_device* dev, const rcu_decoder_config* cfg, const rcu_decoder_layer* layers, const void* tok_embd,
                         const void* out_norm, const void* lm_head, rcu_decoder** out) {
    if (!dev || !cfg || !layers || !tok_embd || !out_norm || !lm_head || !out) return RCU_ERR_INVALID_ARG;
    RCU_REQUIRE(dev, cfg->weight_dt == RCU_Q8_0H || cfg->weight_dt == RCU_Q8_0F, "decoder: weights must be Q8_0H or Q8_0F");
    RCU_REQUIRE(dev, cfg->head_dim == 64 || cfg->head_dim == 96 || cfg->head_dim == 128, "decoder: head_dim must be 64, 96 or 128");
    RCU_REQUIRE(dev, cfg->n_kv_heads > 0 && cfg->n_heads % cfg->n_kv_heads == 0, "decoder: n_heads must be a multiple of n_kv_heads");
    RCU_REQUIRE(dev, cfg->d_model % 32 == 0 && cfg->ffn % 32 == 0 && (cfg->n_heads * cfg->head_dim) % 32 == 0, "decoder: Q8_0 rows need whole 32-element blocks");
    RCU_REQUIRE(dev, cfg->rope_dim % 2 == 0 && cfg->rope_dim <= cfg->head_dim && cfg->rope_dim <= 256, "decoder: bad rope_dim");
    RCU_REQUIRE(dev, cfg->max_cache >= 1 && cfg->n_layers >= 1, "decoder: empty model");
    RCU_REQUIRE(dev, cfg->max_cache <= (uint32_t)(kMaxSplits * kTile), "decoder: max_cache %u exceeds %d positions", cfg->max_cache, kMaxSplits * kTile);
    DevGuard g(dev->ordinal);
    rcu_decoder* d = new rcu_decoder();
    d->dev = dev;
    d->cfg = *cfg;
    d->layers.assign(layers, layers + cfg->n_layers);
    d->tok_embd = tok_embd;
    d->out_norm = out_norm;
    d->lm_head = lm_head;
    rcu_status st = alloc_attn_scratch(dev, (int)cfg->n_heads, (size_t)cfg->n_heads * attn_splits((int)cfg->max_cache) * (cfg->head_dim + 2), &d->scratch);
    const size_t qkv_n = (size_t)(cfg->n_heads + 2 * cfg->n_kv_heads) * cfg->head_dim;
    const size_t act_n = std::max<size_t>(cfg->ffn, 2 * (size_t)cfg->d_model);   // also stages an f32 embedding row
    if (st == RCU_OK && (cudaMalloc(&d->x, cfg->d_model * sizeof(__half)) != cudaSuccess || cudaMalloc(&d->qkv, qkv_n * sizeof(__half)) != cudaSuccess ||
                         cudaMalloc(&d->attn, (size_t)cfg->n_heads * cfg->head_dim * sizeof(__half)) != cudaSuccess ||
                         cudaMalloc(&d->act, act_n * sizeof(__half)) != cudaSuccess || cudaMalloc(&d->d_step, sizeof(unsigned int)) != cudaSuccess))
        st = rcu_fail(dev, RCU_ERR_OOM, "decoder: activation buffers");
    if (st != RCU_OK) { rcu_decoder_destroy(d); return st; }
    cudaMemsetAsync(d->d_step, 0, sizeof(unsigned int), dev->stream);
    st = rcu_decoder_set_position(d, 0);
    if (st != RCU_OK) { rcu_decoder_destroy(d); return st; }
    *out = d;
    return RCU_OK;
}

}  // namespace

extern "C" {

rcu_status rcu_decoder_create(rcu_device* dev, const rcu_decoder_config* cfg, const rcu_decoder_layer* layers, const void* tok_embd,
                              const void* out_norm, const void* lm_head, rcu_decoder** out) {
    rcu_decoder* d = nullptr;
    const rcu_status st = decoder_alloc(dev, cfg, layers, tok_embd, out_norm, lm_head, &d);
    if (st != RCU_OK) return st;
    DevGuard g(dev->ordinal);
    setup_flow(d);
    *out = d;
    return RCU_OK;
}

rcu_status rcu_decoder_create_sharded(rcu_device* dev, rcu_comm* comm, const rcu_decoder_config* cfg, const rcu_decoder_layer* layers,
                                      const void* tok_embd, const void* out_norm, const void* lm_head, rcu_decoder** out) {
    if (!dev || !comm || !cfg || !layers || !tok_embd || !out_norm || !lm_head || !out) return RCU_ERR_INVALID_ARG;
    const uint32_t W = (uint32_t)comm->world;
    RCU_REQUIRE(dev, comm->dev == dev, "sharded decoder: the window belongs to another device");
    RCU_REQUIRE(dev, !comm->bound && comm->seq == 0, "sharded decoder: the window must be fresh (its flags count this decoder's steps)");
    for (int p = 0; p < comm->world; ++p)
        RCU_REQUIRE(dev, p == comm->rank || comm->opened[p] || comm->linked[p], "sharded decoder: peer %d has not been imported", p);
    RCU_REQUIRE(dev, cfg->n_heads % W == 0 && cfg->n_kv_heads % W == 0, "sharded decoder: heads (%u, %u kv) must divide over %u ranks",
                cfg->n_heads, cfg->n_kv_heads, W);
    // slices travel as 16-byte vectors and GEMV rows come in groups of 8
    RCU_REQUIRE(dev, (cfg->d_model / W) % 8 == 0 && cfg->d_model % W == 0 && cfg->ffn % W == 0 && (cfg->ffn / W) % 8 == 0 &&
                         cfg->vocab % W == 0 && (cfg->vocab / W) % 8 == 0 && (cfg->n_heads / W * cfg->head_dim) % 8 == 0,
                "sharded decoder: d_model, ffn and vocab must split over %u ranks into multiples of 8 rows", W);
    const size_t need = 4 * (size_t)std::max(std::max(std::max(cfg->d_model, cfg->ffn), std::max(cfg->vocab, cfg->n_heads * cfg->head_dim)),
                                             (cfg->n_heads + 2 * cfg->n_kv_heads) / W * cfg->head_dim);   // one word per element
    RCU_REQUIRE(dev, comm->local.slot_bytes >= need, "sharded decoder: window slots hold %zu bytes, %zu needed", comm->local.slot_bytes, need);
    rcu_decoder_config local = *cfg;   // per-rank sizes for the shared validation and buffers
    local.n_heads = cfg->n_heads / W;
    local.n_kv_heads = cfg->n_kv_heads / W;
    rcu_decoder* d = nullptr;
    rcu_status st = decoder_alloc(dev, &local, layers, tok_embd, out_norm, lm_head, &d);
    if (st != RCU_OK) return st;
    d->cfg = *cfg;                     // the step works from the whole model's sizes
    DevGuard g(dev->ordinal);
    d->comm = comm;
    comm->bound = true;
    setup_flow(d);
    *out = d;
    return RCU_OK;
}

void rcu_decoder_destroy(rcu_decoder* d) {
    if (!d) return;
    DevGuard g(d->dev->ordinal);
    cudaStreamSynchronize(d->dev->stream);
    if (d->graph_exec) cudaGraphExecDestroy(d->graph_exec);
    cudaFree(d->scratch.partial);
    cudaFree(d->scratch.counters);
    cudaFree(d->scratch.rope_tab);
    cudaFree(d->scratch.d_pos);
    cudaFree(d->x);
    cudaFree(d->qkv);
    cudaFree(d->attn);
    cudaFree(d->act);
    cudaFree(d->d_step);
    cudaFree(d->d_layer_ptrs);
    cudaFree(d->own_window);
    cudaFree(d->flow_partial);
    cudaFree(d->d_prof);
    delete d;
}

rcu_status rcu_decoder_set_position(rcu_decoder* d, uint32_t position) {
    if (!d) return RCU_ERR_INVALID_ARG;
    RCU_REQUIRE(d->dev, position < d->cfg.max_cache, "decoder: position %u is outside the cache (%u)", position, d->cfg.max_cache);
    DevGuard g(d->dev->ordinal);
    set_u32_kernel<<<1, 1, 0, d->dev->stream>>>(d->scratch.d_pos, position);
    RCU_LAUNCH_CHECK(d->dev);
    d->position = position;
    return RCU_OK;
}

uint32_t rcu_decoder_position(const rcu_decoder* d) { return d ? d->position : 0; }
uint32_t rcu_decoder_kernels_per_step(const rcu_decoder* d) { return d ? d->kernels_per_step : 0; }

rcu_status rcu_decoder_step(rcu_decoder* d, const int32_t* token_dev, void* logits_dev, int32_t* argmax_dev) {
    if (!d || !token_dev || !logits_dev) return RCU_ERR_INVALID_ARG;
    rcu_device* dev = d->dev;
    RCU_REQUIRE(dev, d->position < d->cfg.max_cache, "decoder: the KV cache is full (%u entries)", d->cfg.max_cache);
    DevGuard g(dev->ordinal);
    // stream capture is not available on the legacy default stream: run the sequence eagerly there
    const bool use_graph = std::getenv("RCU_NO_GRAPH") == nullptr && dev->stream != nullptr;
    rcu_status st = RCU_OK;
    if (!use_graph || d->steps == 0) {
        // first step runs eagerly: sets kernel attributes and counts the launches
        const uint64_t l0 = dev->launches;
        st = run_step(d, token_dev, logits_dev, argmax_dev);
        d->kernels_per_step = (uint32_t)(dev->launches - l0);
    } else {
        if (!d->graph_exec || d->cap_token != token_dev || d->cap_logits != logits_dev || d->cap_argmax != argmax_dev ||
            d->cap_variant != attn_variant(d->position)) {
            if (d->graph_exec) { cudaGraphExecDestroy(d->graph_exec); d->graph_exec = nullptr; }
            cudaGraph_t graph = nullptr;
            const uint64_t l0 = dev->launches;
            RCU_CUDA(dev, cudaStreamBeginCapture(dev->stream, cudaStreamCaptureModeThreadLocal));
            st = run_step(d, token_dev, logits_dev, argmax_dev);
            cudaError_t e = cudaStreamEndCapture(dev->stream, &graph);
            dev->launches = l0;   // capture launched nothing
            if (st != RCU_OK) { if (graph) cudaGraphDestroy(graph); return st; }
            if (e != cudaSuccess) return rcu_fail(dev, RCU_ERR_CUDA, "decoder: graph capture failed: %s", cudaGetErrorString(e));
            e = cudaGraphInstantiate(&d->graph_exec, graph, 0);
            cudaGraphDestroy(graph);
            if (e != cudaSuccess) return rcu_fail(dev, RCU_ERR_CUDA, "decoder: graph instantiation failed: %s", cudaGetErrorString(e));
            d->cap_token = token_dev; d->cap_logits = logits_dev; d->cap_argmax = argmax_dev;
            d->cap_variant = attn_variant(d->position);
        }
        RCU_CUDA(dev, cudaGraphLaunch(d->graph_exec, dev->stream));
        dev->launches += d->kernels_per_step;
    }
    if (st != RCU_OK) return st;
    d->steps++;
    d->position++;
    return RCU_OK;
}

rcu_status rcu_decoder_profile_step(rcu_decoder* d, const int32_t* token_dev, void* logits_dev, uint64_t* stamps_ns, uint32_t capacity,
                                    uint32_t* n_stamps) {
    if (!d || !token_dev || !logits_dev || !stamps_ns || !n_stamps) return RCU_ERR_INVALID_ARG;
    rcu_device* dev = d->dev;
    RCU_REQUIRE(dev, d->flow_grid > 0, "decoder: this decoder runs kernel by kernel; per-job time stamps exist only for the data-flow kernel");
    RCU_REQUIRE(dev, d->position < d->cfg.max_cache, "decoder: the KV cache is full (%u entries)", d->cfg.max_cache);
    const uint32_t n = 2u * (5u * (uint32_t)d->fp.n_layers + 1u) + 1u + 24u;
    RCU_REQUIRE(dev, capacity >= n, "decoder: %u time stamps needed, room for %u", n, capacity);
    DevGuard g(dev->ordinal);
    if (!d->d_prof) RCU_CUDA(dev, cudaMalloc(&d->d_prof, n * sizeof(unsigned long long)));
    RCU_CUDA(dev, cudaMemsetAsync(d->d_prof, 0, n * sizeof(unsigned long long), dev->stream));
    d->fp.prof = d->d_prof;
    const rcu_status st = run_sequence_flow(d, token_dev, logits_dev, nullptr);
    d->fp.prof = nullptr;
    if (st != RCU_OK) return st;
    d->steps++;
    d->position++;
    static_assert(sizeof(unsigned long long) == sizeof(uint64_t), "time stamps are 64-bit");
    const rcu_status sd = rcu_d2h(dev, stamps_ns, d->d_prof, n * sizeof(uint64_t));
    *n_stamps = n;
    return sd;
}

rcu_status rcu_attn_decode(rcu_device* dev, const void* qkv, void* k_cache, void* v_cache, uint32_t n_heads, uint32_t n_kv_heads,
                           uint32_t head_dim, uint32_t max_cache, uint32_t rope_dim, float rope_base, uint32_t position, void* out) {
    if (!dev || !qkv || !k_cache || !v_cache || !out) return RCU_ERR_INVALID_ARG;
    RCU_REQUIRE(dev, n_kv_heads > 0 && n_heads % n_kv_heads == 0, "attn_decode: n_heads must be a multiple of n_kv_heads");
    RCU_REQUIRE(dev, n_heads <= 65535u, "attn_decode: n_heads %u exceeds the grid limit", n_heads);
    RCU_REQUIRE(dev, max_cache <= (uint32_t)(kMaxSplits * kTile), "attn_decode: max_cache %u exceeds %d positions", max_cache, kMaxSplits * kTile);
    RCU_REQUIRE(dev, position < max_cache, "attn_decode: position %u outside the cache (%u)", position, max_cache);
    RCU_REQUIRE(dev, rope_dim % 2 == 0 && rope_dim <= head_dim && rope_dim <= 256, "attn_decode: bad rope_dim");
    DevGuard g(dev->ordinal);
    // per-device scratch, allocated on first use (and re-allocated if a later call needs more)
    static std::mutex mu;
    static std::unordered_map<rcu_device*, AttnScratch*> table;
    AttnScratch* s = nullptr;
    {
        std::lock_guard<std::mutex> lock(mu);
        auto it = table.find(dev);
        if (it != table.end()) s = it->second;
    }
    const size_t need = (size_t)n_heads * attn_splits((int)max_cache) * (head_dim + 2);
    if (!s || s->partial_floats < need || s->heads < (int)n_heads) {   // the counters hold one word per head
        AttnScratch* ns = new AttnScratch();
        // never shrink either part: a later call may bring back the larger shape
        rcu_status st = alloc_attn_scratch(dev, std::max((int)n_heads, s ? s->heads : 0), std::max(need, s ? s->partial_floats : (size_t)0), ns);
        if (st != RCU_OK) { delete ns; return st; }
        {
            std::lock_guard<std::mutex> lock(mu);
            table[dev] = ns;
        }
        dev->cleanup.push_back({[](void* p) {
                                    std::lock_guard<std::mutex> lock(mu);
                                    for (auto it = table.begin(); it != table.end();)
                                        it = it->second == p ? table.erase(it) : std::next(it);
                                    free_attn_scratch(p);
                                },
                                ns});
        s = ns;
    }
    set_u32_kernel<<<1, 1, 0, dev->stream>>>(s->d_pos, position);
    RCU_LAUNCH_CHECK(dev);
    rope_table_kernel<<<1, 128, 0, dev->stream>>>(s->d_pos, logf(rope_base), (int)rope_dim / 2, s->rope_tab);
    RCU_LAUNCH_CHECK(dev);
    AttnParams ap{(const __half*)qkv, (__half*)k_cache, (__half*)v_cache, (int)n_heads, (int)n_kv_heads, (int)max_cache, (int)rope_dim,
                  s->d_pos, s->rope_tab, 1.0f / sqrtf((float)head_dim), s->partial, s->counters, (__half*)out};
    return launch_attn(dev, ap, (int)head_dim, false, attn_variant(position));
}

}  // extern "C"

// ------------------------------------------------------------------------------------------------
// Allocation-free variant of rcu_attn_decode.
//
// Some callers may not allocate device memory at the moment they need attention: code running
// inside a host framework that owns the whole device heap and forbids foreign cudaMalloc calls, a
// real-time serving loop whose latency budget cannot absorb an allocation (cudaMalloc synchronises
// the device), or a process that has already handed all free memory to its KV caches.  For them
// the split-KV scratch (per-head partial results, the per-head completion counters, the RoPE table
// and the position word) lives in a fixed array in the library's own device image instead of in
// memory obtained at run time.  Every GPU that loads the library carries these 2.04 MiB until the
// process exits.
//
// The array is shared by every call on a device and keeps what the previous call left in it: the
// counters are cleared at the start of each call, everything else is fully rewritten before it is
// read.  Two calls that overlap on the GPU (different streams, or different host threads using
// handles of the same device) race on it; callers must keep such calls ordered.
// ------------------------------------------------------------------------------------------------
namespace {
constexpr int kStaticMaxHeads = 64;
constexpr int kStaticMaxHeadDim = 128;
constexpr int kStaticMaxSplits = 64;                                                              // 64 heads of 128 dims up to 4096 cached positions
constexpr size_t kStaticPartialFloats = (size_t)kStaticMaxHeads * kStaticMaxSplits * (kStaticMaxHeadDim + 2);
constexpr size_t kStaticPartialBytes = kStaticPartialFloats * sizeof(float);                      // 2129920
constexpr size_t kStaticCountersOff = kStaticPartialBytes;                                        // 64 x u32
constexpr size_t kStaticRopeOff = kStaticCountersOff + 256;                                       // 256 x f32
constexpr size_t kStaticPosOff = kStaticRopeOff + 256 * sizeof(float);
constexpr size_t kStaticScratchBytes = kStaticPosOff + 256;

static __device__ __align__(256) unsigned char g_attn_static_scratch[kStaticScratchBytes];

// Device address of the array, per CUDA device ordinal.  In host code the symbol's name is only a
// handle for the runtime, never a pointer a kernel could use, so the address is looked up once per
// device (with that device current) and cached here.
constexpr int kMaxDeviceOrdinals = 64;
void* g_attn_static_addr[kMaxDeviceOrdinals] = {};
std::mutex g_attn_static_mu;
}  // namespace

extern "C" rcu_status rcu_attn_decode_static(rcu_device* dev, const void* qkv, void* k_cache, void* v_cache, uint32_t n_heads,
                                             uint32_t n_kv_heads, uint32_t head_dim, uint32_t max_cache, uint32_t rope_dim,
                                             float rope_base, uint32_t position, void* out) {
    if (!dev || !qkv || !k_cache || !v_cache || !out) return RCU_ERR_INVALID_ARG;
    RCU_REQUIRE(dev, n_heads >= 1 && n_heads <= (uint32_t)kStaticMaxHeads,
                "attn_decode_static: n_heads %u exceeds the built-in scratch (at most %d heads); use rcu_attn_decode", n_heads, kStaticMaxHeads);
    RCU_REQUIRE(dev, head_dim <= (uint32_t)kStaticMaxHeadDim,
                "attn_decode_static: head_dim %u exceeds the built-in scratch (at most %d); use rcu_attn_decode", head_dim, kStaticMaxHeadDim);
    RCU_REQUIRE(dev, max_cache <= (uint32_t)(kStaticMaxSplits * kTile),
                "attn_decode_static: max_cache %u exceeds the built-in scratch (at most %d positions); use rcu_attn_decode", max_cache,
                kStaticMaxSplits * kTile);
    RCU_REQUIRE(dev, n_kv_heads > 0 && n_heads % n_kv_heads == 0, "attn_decode_static: n_heads must be a multiple of n_kv_heads");
    RCU_REQUIRE(dev, position < max_cache, "attn_decode_static: position %u outside the cache (%u)", position, max_cache);
    RCU_REQUIRE(dev, rope_dim % 2 == 0 && rope_dim <= head_dim && rope_dim <= 256, "attn_decode_static: bad rope_dim");
    RCU_REQUIRE(dev, dev->ordinal >= 0 && dev->ordinal < kMaxDeviceOrdinals, "attn_decode_static: device ordinal %d not supported", dev->ordinal);
    DevGuard g(dev->ordinal);
    unsigned char* base = nullptr;
    {
        // first call on this device: resolve the array's device address (do this before any stream capture)
        std::lock_guard<std::mutex> lock(g_attn_static_mu);
        if (!g_attn_static_addr[dev->ordinal]) {
            void* p = nullptr;
            RCU_CUDA(dev, cudaGetSymbolAddress(&p, g_attn_static_scratch));
            g_attn_static_addr[dev->ordinal] = p;
        }
        base = (unsigned char*)g_attn_static_addr[dev->ordinal];
    }
    float* partial = reinterpret_cast<float*>(base);
    unsigned int* counters = reinterpret_cast<unsigned int*>(base + kStaticCountersOff);
    float* rope_tab = reinterpret_cast<float*>(base + kStaticRopeOff);
    uint32_t* d_pos = reinterpret_cast<uint32_t*>(base + kStaticPosOff);
    // the completion counters must start at zero whatever an earlier (possibly failed) call left behind
    RCU_CUDA(dev, cudaMemsetAsync(counters, 0, (size_t)kStaticMaxHeads * sizeof(unsigned int), dev->stream));
    set_u32_kernel<<<1, 1, 0, dev->stream>>>(d_pos, position);
    RCU_LAUNCH_CHECK(dev);
    rope_table_kernel<<<1, 128, 0, dev->stream>>>(d_pos, logf(rope_base), (int)rope_dim / 2, rope_tab);
    RCU_LAUNCH_CHECK(dev);
    AttnParams ap{(const __half*)qkv, (__half*)k_cache, (__half*)v_cache, (int)n_heads, (int)n_kv_heads, (int)max_cache, (int)rope_dim,
                  d_pos, rope_tab, 1.0f / sqrtf((float)head_dim), partial, counters, (__half*)out};
    return launch_attn(dev, ap, (int)head_dim, false, attn_variant(position));
}
