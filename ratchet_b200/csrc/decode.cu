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
#include <cmath>
#include <cstdlib>

#include <cooperative_groups.h>

#include "comm.cuh"
#include "decode_persist.cuh"
#include "gemv_q8_bulk.cuh"

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
// global merge.  RCU_ATTN_KERNEL forces one.
int attn_variant(uint32_t position) {
    static const int forced = [] { const char* e = std::getenv("RCU_ATTN_KERNEL"); return e ? std::atoi(e) : -1; }();
    if (forced >= 0) return forced;
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
    static bool carveout_set = false;
    if (!carveout_set) {
        cudaFuncSetAttribute(attn_decode_kernel<64>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        cudaFuncSetAttribute(attn_decode_kernel<96>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        cudaFuncSetAttribute(attn_decode_kernel<128>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        cudaFuncSetAttribute(rope_table_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        cudaFuncSetAttribute(argmax_advance_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        cudaFuncSetAttribute(set_u32_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        carveout_set = true;
    }
    if (head_dim != 64 && head_dim != 96 && head_dim != 128)
        return rcu_fail(dev, RCU_ERR_UNSUPPORTED, "attn_decode: head_dim %d (supported: 64, 96, 128)", head_dim);
    static bool cluster_ok = true;
    if (which == 1 || (which == 2 && cluster_ok)) {
        static bool attr_set = false;
        if (!attr_set) {
            cudaFuncSetAttribute(attn_cluster_kernel<64, true>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
            cudaFuncSetAttribute(attn_cluster_kernel<96, true>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
            cudaFuncSetAttribute(attn_cluster_kernel<128, true>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
            attr_set = true;
        }
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
        cluster_ok = false;
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

// Inner product of the step's GEMVs: 2 (default) = dp4a on fixed-point activation planes with 16-element
// scales, 0 = packed f16 with the mixed-precision fma, 1 = f32 FFMA (RCU_GEMV_MODE, tuning aid).
int q8_mode() {
    static int mode = [] {
        const char* e = std::getenv("RCU_GEMV_MODE");
        return e ? std::atoi(e) : 2;
    }();
    return mode;
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
    const int mode = q8_mode();
    const bool ov = pdl_enabled();
    static const int ctas = [] { const char* e = std::getenv("RCU_DECODE_CTAS"); const int n = e ? std::atoi(e) : 3; return n < 1 ? 1 : (n > 3 ? 3 : n); }();
    // shared-memory ring fed by TMA tile copies: opt-in with RCU_GEMV_BULK=1 (the register kernel measures faster on cold weights)
    static const bool bulk = std::getenv("RCU_GEMV_BULK") != nullptr;
    if (bulk && gemvq8::bulk_eligible(qs, K, (size_t)dev->smem_optin, weight_dt == RCU_Q8_0H ? 2 : 4)) {
        if (weight_dt == RCU_Q8_0H) return gemvq8::launch_bulk<__half>(dev, qs, sc, pro, epi, N, K, ov);
        return gemvq8::launch_bulk<float>(dev, qs, sc, pro, epi, N, K, ov);
    }
    if (weight_dt == RCU_Q8_0H) {
        if (mode == 1) return gemvq8::launch<__half, __half, 1>(dev, qs, sc, pro, epi, N, K, ov, ctas, true);
        if (mode == 2) return gemvq8::launch<__half, __half, 2>(dev, qs, sc, pro, epi, N, K, ov, ctas, true);
        return gemvq8::launch<__half, __half, 0>(dev, qs, sc, pro, epi, N, K, ov, ctas, true);
    }
    if (mode == 1) return gemvq8::launch<float, __half, 1>(dev, qs, sc, pro, epi, N, K, ov, ctas, true);
    if (mode == 2) return gemvq8::launch<float, __half, 2>(dev, qs, sc, pro, epi, N, K, ov, ctas, true);
    return gemvq8::launch<float, __half, 0>(dev, qs, sc, pro, epi, N, K, ov, ctas, true);
}

// per-device scratch for the standalone attention entry point
struct AttnScratch {
    float* partial = nullptr;
    unsigned int* counters = nullptr;
    float* rope_tab = nullptr;
    uint32_t* d_pos = nullptr;
    size_t partial_floats = 0;
};

void free_attn_scratch(void* p) {
    AttnScratch* s = (AttnScratch*)p;
    cudaFree(s->partial);
    cudaFree(s->counters);
    cudaFree(s->rope_tab);
    cudaFree(s->d_pos);
    delete s;
}

rcu_status alloc_attn_scratch(rcu_device* dev, int H, int head_dim, int max_cache, AttnScratch* s) {
    s->partial_floats = (size_t)H * attn_splits(max_cache) * (head_dim + 2);
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
    // all layers as one persistent cooperative kernel (decode_persist.cuh); null when not in use
    persist::LayerW* d_layers = nullptr;
    unsigned int* d_bar = nullptr;
    int persist_grid = 0;
    size_t persist_smem = 0;
    persist::Params pp;
    // captured step
    cudaGraphExec_t graph_exec = nullptr;
    const int32_t* cap_token = nullptr;
    void* cap_logits = nullptr;
    int32_t* cap_argmax = nullptr;
    int cap_variant = -1;                 // attention kernel the captured step launches (it depends on the cached length)
};

namespace {

template <int HD>
rcu_status launch_persistent_hd(rcu_decoder* d) {
    rcu_device* dev = d->dev;
    RCU_CUDA(dev, cudaMemsetAsync(d->d_bar, 0, sizeof(unsigned int), dev->stream));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(d->persist_grid);
    cfg.blockDim = dim3(gemvq8::kThreads);
    cfg.dynamicSmemBytes = d->persist_smem;
    cfg.stream = dev->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;      // every CTA resident at once: the grid barriers need it
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    RCU_CUDA(dev, cudaLaunchKernelEx(&cfg, persist::decode_layers_kernel<HD>, d->pp));
    RCU_LAUNCH_CHECK(dev);
    return RCU_OK;
}

rcu_status launch_persistent_layers(rcu_decoder* d) {
    switch (d->cfg.head_dim) {
        case 64: return launch_persistent_hd<64>(d);
        case 96: return launch_persistent_hd<96>(d);
        default: return launch_persistent_hd<128>(d);
    }
}

// K split of a GEMV on the persistent grid: the rule of gemvq8::plan for a fixed number of warps.
int persistent_ksplit(int n_units, int unit, int K, int grid) {
    const long long groups = (n_units + 4 / unit - 1) / (4 / unit);
    const long long warps = (long long)grid * gemvq8::kWarps;
    int ks = 1;
    while (ks < 8 && groups * ks * 2 <= warps && (K / (ks * 2)) >= 1024) ks *= 2;
    return ks;
}

template <int HD>
bool persistent_fit(rcu_decoder* d, size_t smem, int* ctas_per_sm) {
    auto kern = persist::decode_layers_kernel<HD>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return false;
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, gemvq8::kThreads, smem) != cudaSuccess) return false;
    *ctas_per_sm = n;
    return n >= 1;
}

// Sets up the persistent-kernel path when asked for (RCU_DECODE_PERSISTENT=1) and this model and device
// allow it (Q8_0H weights, one GPU, cooperative launch, cache short enough for the merge step).  It is
// not the default: with a grid barrier of about 2 us between phases it measures slower than the
// kernel-per-phase step, whose kernels hand over through programmatic dependent launch.
void setup_persistent(rcu_decoder* d) {
    rcu_device* dev = d->dev;
    const rcu_decoder_config& c = d->cfg;
    const char* env = std::getenv("RCU_DECODE_PERSISTENT");
    if (!env || std::atoi(env) == 0) return;
    if (c.weight_dt != RCU_Q8_0H || d->comm) return;
    if ((c.max_cache + persist::kTile - 1) / persist::kTile > persist::kMaxSplits) return;
    int coop = 0;
    if (cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev->ordinal) != cudaSuccess || !coop) return;
    const int HD = (int)c.head_dim;
    const size_t kmax = std::max(std::max((size_t)c.d_model, (size_t)c.ffn), (size_t)c.n_heads * HD);
    const size_t attn_bytes = HD == 64 ? sizeof(persist::AttnShared<64>) : HD == 96 ? sizeof(persist::AttnShared<96>) : sizeof(persist::AttnShared<128>);
    const size_t smem = ((kmax * 2 + gemvq8::kWarps * 4 * sizeof(float) + 15) & ~(size_t)15) + 2 * attn_bytes;
    if (smem > (size_t)dev->smem_optin) return;
    int per_sm = 0;
    const bool ok = HD == 64 ? persistent_fit<64>(d, smem, &per_sm) : HD == 96 ? persistent_fit<96>(d, smem, &per_sm) : persistent_fit<128>(d, smem, &per_sm);
    if (!ok) { cudaGetLastError(); return; }
    per_sm = std::min(per_sm, 2);
    const int grid = per_sm * dev->sm_count;
    std::vector<persist::LayerW> host(c.n_layers);
    const uint64_t D = c.d_model, F = c.ffn, Q = (uint64_t)(c.n_heads + 2 * c.n_kv_heads) * HD, A = (uint64_t)c.n_heads * HD;
    auto scales = [](const void* w, uint64_t n) { return (const __half*)((const char*)w + align256(n)); };
    for (uint32_t i = 0; i < c.n_layers; ++i) {
        const rcu_decoder_layer& L = d->layers[i];
        host[i] = persist::LayerW{(const int8_t*)L.qkv, scales(L.qkv, Q * D), (const int8_t*)L.o, scales(L.o, D * A),
                                  (const int8_t*)L.gate_up, scales(L.gate_up, 2 * F * D), (const int8_t*)L.down, scales(L.down, D * F),
                                  (const float*)L.attn_norm, (const float*)L.ffn_norm, (__half*)L.k_cache, (__half*)L.v_cache};
    }
    if (cudaMalloc(&d->d_layers, host.size() * sizeof(persist::LayerW)) != cudaSuccess || cudaMalloc(&d->d_bar, sizeof(unsigned int)) != cudaSuccess) {
        cudaGetLastError();
        return;
    }
    cudaMemcpyAsync(d->d_layers, host.data(), host.size() * sizeof(persist::LayerW), cudaMemcpyHostToDevice, dev->stream);
    cudaStreamSynchronize(dev->stream);     // `host` goes out of scope
    persist::Params& p = d->pp;
    p.layers = d->d_layers;
    p.n_layers = (int)c.n_layers; p.D = (int)D; p.H = (int)c.n_heads; p.Hkv = (int)c.n_kv_heads; p.ffn = (int)F;
    p.max_cache = (int)c.max_cache; p.rope_dim = (int)c.rope_dim;
    p.eps = c.rms_eps; p.scale = 1.0f / sqrtf((float)HD);
    p.x = d->x; p.qkv = d->qkv; p.attn = d->attn; p.act = d->act;
    p.d_pos = d->scratch.d_pos; p.rope_tab = d->scratch.rope_tab;
    p.partial = d->scratch.partial; p.counters = d->scratch.counters;
    p.bar = d->d_bar; p.status = dev->d_status;
    p.ks_qkv = persistent_ksplit((int)Q, 1, (int)D, grid);
    p.ks_o = persistent_ksplit((int)D, 1, (int)A, grid);
    p.ks_gu = persistent_ksplit((int)F, 2, (int)D, grid);
    p.ks_down = persistent_ksplit((int)D, 1, (int)F, grid);
    d->persist_grid = grid;
    d->persist_smem = smem;
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
    if (d->persist_grid > 0) {
        st = launch_persistent_layers(d);
        if (st != RCU_OK) return st;
    } else {
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

}  // namespace

extern "C" {

rcu_status rcu_decoder_create(rcu_device* dev, const rcu_decoder_config* cfg, const rcu_decoder_layer* layers, const void* tok_embd,
                              const void* out_norm, const void* lm_head, rcu_decoder** out) {
    if (!dev || !cfg || !layers || !tok_embd || !out_norm || !lm_head || !out) return RCU_ERR_INVALID_ARG;
    RCU_REQUIRE(dev, cfg->weight_dt == RCU_Q8_0H || cfg->weight_dt == RCU_Q8_0F, "decoder: weights must be Q8_0H or Q8_0F");
    RCU_REQUIRE(dev, cfg->head_dim == 64 || cfg->head_dim == 96 || cfg->head_dim == 128, "decoder: head_dim must be 64, 96 or 128");
    RCU_REQUIRE(dev, cfg->n_kv_heads > 0 && cfg->n_heads % cfg->n_kv_heads == 0, "decoder: n_heads must be a multiple of n_kv_heads");
    RCU_REQUIRE(dev, cfg->d_model % 32 == 0 && cfg->ffn % 32 == 0 && (cfg->n_heads * cfg->head_dim) % 32 == 0, "decoder: Q8_0 rows need whole 32-element blocks");
    RCU_REQUIRE(dev, cfg->rope_dim % 2 == 0 && cfg->rope_dim <= cfg->head_dim && cfg->rope_dim <= 256, "decoder: bad rope_dim");
    RCU_REQUIRE(dev, cfg->max_cache >= 1 && cfg->n_layers >= 1, "decoder: empty model");
    DevGuard g(dev->ordinal);
    rcu_decoder* d = new rcu_decoder();
    d->dev = dev;
    d->cfg = *cfg;
    d->layers.assign(layers, layers + cfg->n_layers);
    d->tok_embd = tok_embd;
    d->out_norm = out_norm;
    d->lm_head = lm_head;
    rcu_status st = alloc_attn_scratch(dev, (int)cfg->n_heads, (int)cfg->head_dim, (int)cfg->max_cache, &d->scratch);
    const size_t qkv_n = (size_t)(cfg->n_heads + 2 * cfg->n_kv_heads) * cfg->head_dim;
    const size_t act_n = std::max<size_t>(cfg->ffn, 2 * (size_t)cfg->d_model);   // also stages an f32 embedding row
    if (st == RCU_OK && (cudaMalloc(&d->x, cfg->d_model * sizeof(__half)) != cudaSuccess || cudaMalloc(&d->qkv, qkv_n * sizeof(__half)) != cudaSuccess ||
                         cudaMalloc(&d->attn, (size_t)cfg->n_heads * cfg->head_dim * sizeof(__half)) != cudaSuccess ||
                         cudaMalloc(&d->act, act_n * sizeof(__half)) != cudaSuccess))
        st = rcu_fail(dev, RCU_ERR_OOM, "decoder: activation buffers");
    if (st != RCU_OK) { rcu_decoder_destroy(d); return st; }
    setup_persistent(d);
    st = rcu_decoder_set_position(d, 0);
    if (st != RCU_OK) { rcu_decoder_destroy(d); return st; }
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
        RCU_REQUIRE(dev, p == comm->rank || comm->opened[p], "sharded decoder: peer %d has not been imported", p);
    RCU_REQUIRE(dev, cfg->n_heads % W == 0 && cfg->n_kv_heads % W == 0, "sharded decoder: heads (%u, %u kv) must divide over %u ranks",
                cfg->n_heads, cfg->n_kv_heads, W);
    // slices travel as 16-byte vectors and GEMV rows come in groups of 8
    RCU_REQUIRE(dev, (cfg->d_model / W) % 8 == 0 && cfg->d_model % W == 0 && cfg->ffn % W == 0 && (cfg->ffn / W) % 8 == 0 &&
                         cfg->vocab % W == 0 && (cfg->vocab / W) % 8 == 0 && (cfg->n_heads / W * cfg->head_dim) % 8 == 0,
                "sharded decoder: d_model, ffn and vocab must split over %u ranks into multiples of 8 rows", W);
    const size_t need = 4 * (size_t)std::max(std::max(cfg->d_model, cfg->ffn), std::max(cfg->vocab, cfg->n_heads * cfg->head_dim));   // one word per element
    RCU_REQUIRE(dev, comm->local.slot_bytes >= need, "sharded decoder: window slots hold %zu bytes, %zu needed", comm->local.slot_bytes, need);
    rcu_decoder_config local = *cfg;   // per-rank sizes for the shared validation and buffers
    local.n_heads = cfg->n_heads / W;
    local.n_kv_heads = cfg->n_kv_heads / W;
    rcu_decoder* d = nullptr;
    rcu_status st = rcu_decoder_create(dev, &local, layers, tok_embd, out_norm, lm_head, &d);
    if (st != RCU_OK) return st;
    d->cfg = *cfg;                     // the step works from the whole model's sizes
    d->persist_grid = 0;               // the sharded step runs kernel by kernel
    DevGuard g(dev->ordinal);
    if (cudaMalloc(&d->d_step, sizeof(unsigned int)) != cudaSuccess) {
        rcu_decoder_destroy(d);
        return rcu_fail(dev, RCU_ERR_OOM, "sharded decoder: step counter");
    }
    cudaMemsetAsync(d->d_step, 0, sizeof(unsigned int), dev->stream);
    d->comm = comm;
    comm->bound = true;
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
    cudaFree(d->d_layers);
    cudaFree(d->d_bar);
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
        st = d->comm ? run_sequence_sharded(d, token_dev, logits_dev, argmax_dev) : run_sequence(d, token_dev, logits_dev, argmax_dev);
        d->kernels_per_step = (uint32_t)(dev->launches - l0);
    } else {
        if (!d->graph_exec || d->cap_token != token_dev || d->cap_logits != logits_dev || d->cap_argmax != argmax_dev ||
            d->cap_variant != attn_variant(d->position)) {
            if (d->graph_exec) { cudaGraphExecDestroy(d->graph_exec); d->graph_exec = nullptr; }
            cudaGraph_t graph = nullptr;
            const uint64_t l0 = dev->launches;
            RCU_CUDA(dev, cudaStreamBeginCapture(dev->stream, cudaStreamCaptureModeThreadLocal));
            st = d->comm ? run_sequence_sharded(d, token_dev, logits_dev, argmax_dev) : run_sequence(d, token_dev, logits_dev, argmax_dev);
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

rcu_status rcu_attn_decode(rcu_device* dev, const void* qkv, void* k_cache, void* v_cache, uint32_t n_heads, uint32_t n_kv_heads,
                           uint32_t head_dim, uint32_t max_cache, uint32_t rope_dim, float rope_base, uint32_t position, void* out) {
    if (!dev || !qkv || !k_cache || !v_cache || !out) return RCU_ERR_INVALID_ARG;
    RCU_REQUIRE(dev, n_kv_heads > 0 && n_heads % n_kv_heads == 0, "attn_decode: n_heads must be a multiple of n_kv_heads");
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
    if (!s || s->partial_floats < need) {
        AttnScratch* ns = new AttnScratch();
        rcu_status st = alloc_attn_scratch(dev, (int)n_heads, (int)head_dim, (int)max_cache, ns);
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
    RCU_REQUIRE(dev, attn_splits((int)max_cache) <= kStaticMaxSplits,
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
