// One decode step's layers as ONE persistent data-flow kernel.
//
// The kernel-per-phase decode step (decode.cu, run_sequence) launches five kernels per layer; each of
// them streams only 10-56 MB and pays microseconds of start, activation staging and drain, and the
// weight stream stops at every kernel boundary.  Here one CTA per SM stays resident for the whole step
// (cooperative launch) and walks a fixed list of jobs:
//     per layer:  qkv GEMV (RMSNorm) | attention | o GEMV + residual | gate/up GEMV + SiLU | down GEMV + residual
//     then:       lm_head GEMV (RMSNorm)
// Two things make it a data flow rather than a sequence of phases behind grid barriers:
//   * every vector that one job hands to the next travels as tagged 32-bit words (sequence number in the
//     high half, f16 value in the low half, as gemvq8::LLPush does between GPUs) in an exchange window, on
//     one GPU as well as across the GPUs of a sharded decoder.  A producer stores a result the moment it
//     has it; a consumer polls exactly the words it needs.  There is no barrier object and no CTA that
//     waits for a CTA it does not depend on;
//   * the weights, and the cached K/V rows, do not depend on activations.  Every consumer warp owns a
//     ring of shared-memory slots; one more warp per CTA, the requester, walks each consumer's sequence
//     of items through the whole job list and keeps its ring full with 1-D bulk copies (ring.cuh; no
//     tensor maps, no multicast), asking L2 for the items a few places further on.  While a warp waits
//     for the activation vector of one matrix, its slots fill with rows of that matrix and of the next,
//     so HBM keeps streaming across the hand-overs.
// Arithmetic and rounding points are those of the per-kernel step: gemvq8's dp4a inner product on
// 16-bit fixed-point planes, its prologues and epilogues, and split-KV attention with f16-rounded
// scores (phi3/attn.rs:142-157).
//
// Attention: the warps of the grid are dealt to the local heads (wph warps per head), a warp owns a
// contiguous run of 16-position tiles of one head and folds them with an online softmax; the warps of a
// head inside one CTA merge through shared memory, the (at most few) CTAs of a head through a small
// global scratch and a per-head ticket; the last one publishes the head's output as tagged words.
//
// Every wait (mbarrier, tagged word) is bounded by the device's wait limit; a wait that runs out raises
// RCU_DEVFLAG_TIMEOUT, after which every other wait returns at once and the kernel runs to its end
// with meaningless results instead of hanging.
#pragma once
#include "ring.cuh"

namespace flow {

constexpr int kTileP = 16;               // cached positions per attention item
constexpr int kMaxRope = 256;
constexpr int kMaxLayersShared = 48;     // layer pointer tables up to this many layers are kept in shared memory
constexpr int kMaxDepth = ringq8::kMaxDepth;

// Job j of the list is (layer j / 5, kind j % 5) for j < 5 L, then the lm_head.  Layers have the same
// shapes, so a job is described by its kind (constant memory, part of the kernel's parameters) plus the
// layer's pointers (shared memory): a warp never goes to global memory to learn what to do next.
enum Kind : int { K_QKV = 0, K_ATTN = 1, K_O = 2, K_GATE_UP = 3, K_DOWN = 4, K_HEAD = 5, kKinds = 6 };

// Window offsets are in 32-bit words from the start of the window.  An exchange's sequence number is
// step * per_step + (layer * idx_mul + idx_add) + 1 (as gemvq8::LLSeq).
struct KindDesc {
    int n_units, K, ri, kc, nc, unit;    // the matrix and its cut into items (ringq8::Job); unit: 1, or 2 for (gate, up) row pairs
    uint32_t scales_off;                 // bytes from the matrix's first byte to its scale segment
    int rms;                             // the prologue normalises (RMSNorm) with the layer's weights
    uint32_t in_off, in_per_step;
    int in_mul, in_add;
    uint32_t out_off, out_per_step;      // out_off already points at this rank's rows
    int out_mul, out_add;
    uint32_t res_off;                    // words holding the residual for this rank's rows (K_O, K_DOWN)
    int push;                            // outputs also go to the peers' windows
};

struct LayerPtrs {
    const int8_t* w[4];                  // qkv, o, gate_up, down
    const float* attn_norm;
    const float* ffn_norm;
    __half* kc;
    __half* vc;
};

struct Params {
    KindDesc kd[kKinds];
    const LayerPtrs* layers;             // device array [n_layers]
    int n_layers;
    const int8_t* head_w;
    const float* out_norm;
    uint32_t* win;                       // this rank's exchange window
    uint32_t* peer_win[gemvq8::kMaxPeers];
    int n_peers;
    const unsigned int* d_step;          // steps taken so far (sequence numbers derive from it)
    int* status;
    int scale_size;                      // bytes of a block scale (2 or 4)
    // attention
    int H, Hkv, max_cache, rope_dim;     // heads on this rank
    float scale;
    const uint32_t* d_pos;
    const float* rope_tab;               // cos[rope_dim/2], sin[rope_dim/2] for this position
    uint32_t q_off, q_per_step;          // exchange holding this rank's qkv rows
    uint32_t a_off, a_per_step;          // exchange the head outputs go to (start of the whole vector)
    int a_rank_off;                      // first element of this rank's heads in it
    float* partial;                      // [H][max CTAs per head][HD + 2]
    unsigned int* counters;              // [H], zero between steps
    int part_stride;                     // CTAs per head the scratch is laid out for
    // ring
    int slot_bytes, depth;
    int l2_ahead;                        // items beyond the ring the requester asks L2 for (0: none)
    int prof_job;                        // with prof_cta: the job whose per-CTA times are recorded
    unsigned long long* prof_cta;        // optional: [3 x grid] per CTA: job begun, input staged, items done (job prof_job)
    float eps;
    unsigned long long* prof;            // optional (nullptr: off): [2 n_jobs + 1] time stamps of CTA 0 (job begun, input staged; end), then
                                         // per job kind four sums of SM clock cycles of the grid's first warp: slot wait, multiply, store, release
};

__device__ __forceinline__ uint32_t make_tag(unsigned step, uint32_t per_step, uint32_t idx) { return ((step * per_step + idx + 1u) & 0xFFFFu) << 16; }

__device__ __forceinline__ float f16r(float v) { return __half2float(__float2half_rn(v)); }

__device__ __forceinline__ int n_jobs_of(const Params& p) { return 5 * p.n_layers + 1; }
__device__ __forceinline__ void split_job(const Params& p, int j, int& li, int& kind) {
    if (j >= 5 * p.n_layers) { li = p.n_layers; kind = K_HEAD; }
    else { li = j / 5; kind = j - 5 * li; }
}
__device__ __forceinline__ const int8_t* weights_of(const Params& p, const LayerPtrs* lp, int li, int kind) {
    return kind == K_HEAD ? p.head_w : lp[li].w[kind == K_QKV ? 0 : kind - 1];       // K_O 2 -> 1, K_GATE_UP 3 -> 2, K_DOWN 4 -> 3
}
__device__ __forceinline__ ringq8::Job job_of(const Params& p, const KindDesc& k, const int8_t* w) {
    return ringq8::Job{w, reinterpret_cast<const unsigned char*>(w) + k.scales_off, k.n_units, k.n_units, k.K, k.ri, k.kc, k.nc, p.scale_size};
}

// ------------------------------------------------------------------------------------------------
// The items of one consumer warp in one job.  NW = consumer warps per CTA.
struct Range { int first, count; };      // GEMV: first group, groups x nc items.  Attention: first tile, tiles.

template <int NW>
__device__ __forceinline__ Range gemv_range(const KindDesc& k, int warp) {      // host checks that groups x warps stays below 2^31
    const unsigned n_groups = (unsigned)((k.n_units + k.ri - 1) / k.ri);
    const unsigned gw = blockIdx.x * NW + warp, GW = gridDim.x * NW;
    const int g0 = (int)(gw * n_groups / GW), g1 = (int)((gw + 1u) * n_groups / GW);
    return Range{g0, (g1 - g0) * k.nc};
}

// warps per head; warp gw serves head gw / wph (none if that is >= H), segment gw % wph of its tiles
template <int NW> __device__ __forceinline__ int warps_per_head(int H) { return (int)((gridDim.x * NW) / H); }

template <int NW>
__device__ __forceinline__ Range attn_range(int H, int n_tiles, int warp, int* head) {
    const int gw = blockIdx.x * NW + warp;
    const int wph = warps_per_head<NW>(H);
    const int h = gw / wph;
    *head = h;
    if (h >= H) return Range{0, 0};
    const int s = gw - h * wph;
    const int t0 = s * n_tiles / wph, t1 = (s + 1) * n_tiles / wph;
    return Range{t0, t1 - t0};
}

// The per-kind ranges of a warp are the same in every layer: computed once, kept in shared memory (they are
// indexed by a run-time kind), and a cursor only counts.
struct Ranges {
    Range r[kKinds];
    int head;            // of this warp's attention tiles
};
struct Cursor {
    int job, li, kind, idx;
};

__device__ __forceinline__ void seek(const Params& p, const Ranges& rg, Cursor& c) {   // to the first job from c.job on that has items
    c.idx = 0;
    const int n = n_jobs_of(p);
    for (; c.job < n; ++c.job) {
        split_job(p, c.job, c.li, c.kind);
        if (rg.r[c.kind].count > 0) return;
    }
}
__device__ __forceinline__ void advance(const Params& p, const Ranges& rg, Cursor& c) {
    if (++c.idx < rg.r[c.kind].count) return;
    ++c.job;
    seek(p, rg, c);
}

__device__ __forceinline__ void l2_prefetch(const void* src, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}

// One thread: request the item at `c` into `slot` (completion on `bar`), or, with slot == nullptr, only ask L2 for it.
template <int HD>
__device__ __forceinline__ void issue(const Params& p, const LayerPtrs* lp, const Ranges& rg, const Cursor& c, int P, unsigned char* slot, uint64_t* bar) {
    if (c.kind == K_ATTN) {
        const int h = rg.head, kvh = h / (p.H / p.Hkv);
        const int begin = (rg.r[K_ATTN].first + c.idx) * kTileP;
        const int n_cached = min(kTileP, P - begin);                     // rows already in the cache (the tile may also hold position P)
        const unsigned bytes = n_cached > 0 ? (unsigned)n_cached * HD * 2u : 0u;
        const __half* kc = lp[c.li].kc + ((size_t)kvh * p.max_cache + begin) * HD;
        const __half* vc = lp[c.li].vc + ((size_t)kvh * p.max_cache + begin) * HD;
        if (!slot) {
            if (bytes) { l2_prefetch(kc, bytes); l2_prefetch(vc, bytes); }
            return;
        }
        gemvq8::mbar_expect_tx(bar, 2u * bytes);
        if (bytes) {
            gemvq8::bulk_load_1d(slot, kc, bytes, bar);
            gemvq8::bulk_load_1d(slot + kTileP * HD * 2, vc, bytes, bar);
        }
        return;
    }
    const KindDesc& k = p.kd[c.kind];
    const int8_t* w = weights_of(p, lp, c.li, c.kind);
    int g = rg.r[c.kind].first, ch = 0;
    if (k.nc == 1) g += c.idx;
    else { g += c.idx / k.nc; ch = c.idx % k.nc; }
    const int u0 = g * k.ri;
    const int nr = min(k.ri, k.n_units - u0);
    const int sc_row = (k.kc >> 5) * p.scale_size;                  // scale bytes of one row chunk
    const size_t sc_pitch = (size_t)(k.K >> 5) * p.scale_size;      // scale bytes of a whole row
    const unsigned char* scales = reinterpret_cast<const unsigned char*>(w) + k.scales_off;
    if (slot) gemvq8::mbar_expect_tx(bar, (unsigned)(k.unit * nr * (k.kc + sc_row)));
    unsigned char* sdst = slot + k.unit * k.ri * k.kc;
    for (int b = 0; b < k.unit; ++b) {
        const size_t row0 = (size_t)u0 + (size_t)b * k.n_units;    // the up rows follow the gate rows
        if (k.nc == 1) {
            if (slot) {
                gemvq8::bulk_load_1d(slot + b * k.ri * k.kc, w + row0 * k.K, (uint32_t)(nr * k.kc), bar);
                gemvq8::bulk_load_1d(sdst + b * k.ri * sc_row, scales + row0 * sc_pitch, (uint32_t)(nr * sc_row), bar);
            } else {
                l2_prefetch(w + row0 * k.K, (uint32_t)(nr * k.kc));
                l2_prefetch(scales + row0 * sc_pitch, (uint32_t)(nr * sc_row));
            }
        } else {
            for (int r = 0; r < nr; ++r) {
                const int8_t* qsrc = w + (row0 + r) * k.K + (size_t)ch * k.kc;
                const unsigned char* ssrc = scales + (row0 + r) * sc_pitch + (size_t)ch * sc_row;
                if (slot) {
                    gemvq8::bulk_load_1d(slot + (b * k.ri + r) * k.kc, qsrc, (uint32_t)k.kc, bar);
                    gemvq8::bulk_load_1d(sdst + (b * k.ri + r) * sc_row, ssrc, (uint32_t)sc_row, bar);
                } else {
                    l2_prefetch(qsrc, (uint32_t)k.kc);
                    l2_prefetch(ssrc, (uint32_t)sc_row);
                }
            }
        }
    }
}

// ------------------------------------------------------------------------------------------------
// The requester warp: lane w keeps consumer warp w's ring full.  A slot is requested again once the consumer
// has arrived on its `empty` barrier (the consumer's reads of the slot are ordered before that arrival, and
// this thread's copies after its wait, as in any TMA producer / consumer pipeline).
template <int HD, int NW>
__device__ __forceinline__ void requester(const Params& p, const LayerPtrs* lp, const Ranges* rgs, int P, unsigned char* rings, uint64_t* full_bars,
                                          uint64_t* empty_bars) {
    const int w = threadIdx.x & 31;
    if (w >= NW) return;
    const Ranges& rg = rgs[w];
    unsigned char* ring = rings + (size_t)w * p.depth * p.slot_bytes;
    uint64_t* full = full_bars + w * kMaxDepth;
    uint64_t* empty = empty_bars + w * kMaxDepth;
    const int n_jobs = n_jobs_of(p);
    Cursor pc{0, 0, 0, 0};
    seek(p, rg, pc);
    Cursor lc = pc;                                    // runs l2_ahead items ahead of pc
    for (int i = 0; i < p.depth + p.l2_ahead && lc.job < n_jobs; ++i) {
        if (i >= p.depth) issue<HD>(p, lp, rg, lc, P, nullptr, nullptr);
        advance(p, rg, lc);
    }
    int slot = 0, round = 0;
    unsigned long long t0 = 0;
    unsigned spins = 0;
    while (pc.job < n_jobs) {
        bool is_free = round == 0;
        if (!is_free) is_free = gemvq8::mbar_test_wait(&empty[slot], (unsigned)(round - 1) & 1u);
        if (is_free) {
            issue<HD>(p, lp, rg, pc, P, ring + (size_t)slot * p.slot_bytes, &full[slot]);
            advance(p, rg, pc);
            if (p.l2_ahead > 0 && lc.job < n_jobs) {
                issue<HD>(p, lp, rg, lc, P, nullptr, nullptr);
                advance(p, rg, lc);
            }
            if (++slot == p.depth) { slot = 0; ++round; }
            spins = 0;
            t0 = 0;
        } else if ((++spins & 127u) == 0u) {
            if (*reinterpret_cast<volatile int*>(p.status) & RCU_DEVFLAG_TIMEOUT) break;
            const unsigned long long t = ringq8::globaltimer();
            if (t0 == 0) t0 = t;
            else if (t - t0 > rcu_wait_limit(p.status)) { atomicOr(p.status, RCU_DEVFLAG_TIMEOUT); break; }
        }
    }
}

// ------------------------------------------------------------------------------------------------
// Epilogue of a GEMV item: lane i stores unit i as a tagged word to this rank's window and its peers'
// (the window pointers stay in the kernel's parameters; only the offset travels in registers).
struct Out {
    uint32_t off;        // words from the start of a window to the exchange's first element on this rank
    int n_peers;
    uint32_t tag;
    int kind;
    __device__ __forceinline__ void put(const Params& p, int u, __half v) const {
        const uint32_t word = tag | (uint32_t)__half_as_ushort(v);
        p.win[off + u] = word;
#pragma unroll
        for (int q = 0; q < gemvq8::kMaxPeers; ++q)
            if (q < n_peers) p.peer_win[q][off + u] = word;
    }
};

__device__ __forceinline__ Out make_out(const Params& p, uint32_t off, bool push, uint32_t tag, int kind) {
    return Out{off, push ? p.n_peers : 0, tag, kind};
}

__device__ __forceinline__ void store_unit(const Params& p, const Out& o, int u, const float* s, float res) {
    __half r;
    if (o.kind == K_GATE_UP) {
        // phi3/mlp.rs:31-39: up * f16(silu(f32(gate))), silu(x) = x / (1 + exp(-x)) (cpu/unary.rs:64)
        const float gate = f16r(s[0]), up = f16r(s[1]);
        const float act = f16r(gate / (1.0f + expf(-gate)));
        r = __float2half_rn(up * act);
    } else if (o.kind == K_O || o.kind == K_DOWN) {
        // phi3/model.rs:110-116: the Linear output is rounded to f16, then added to the residual in f16
        r = __float2half_rn(f16r(s[0]) + res);
    } else {
        r = __float2half_rn(s[0]);
    }
    o.put(p, u, r);
}

// `resv`: lane i holds the residual of the warp's i-th unit of this job (loaded when the job began); `first_unit`
// is the warp's first unit.
template <int UNIT, int RI>
__device__ __forceinline__ void store_item(const Params& p, const Out& o, int u0, int n_units, float (&acc)[UNIT * RI], float resv, int first_unit) {
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int r = 0; r < UNIT * RI; ++r) acc[r] = warp_sum(acc[r]);
    float s[UNIT];
#pragma unroll
    for (int j = 0; j < UNIT; ++j) s[j] = acc[j * RI];
#pragma unroll
    for (int i = 1; i < RI; ++i)
        if (lane == i) {
#pragma unroll
            for (int j = 0; j < UNIT; ++j) s[j] = acc[j * RI + i];
        }
    const float res = __shfl_sync(0xffffffffu, resv, (u0 + lane - first_unit) & 31);
    if (lane < RI && u0 + lane < n_units) store_unit(p, o, u0 + lane, s, res);
#pragma unroll
    for (int r = 0; r < UNIT * RI; ++r) acc[r] = 0.f;
}

// What a consumer warp carries through the kernel.
struct WarpState {
    Cursor cc;
    int slot;
    unsigned parity;
    bool alive;
};

// The slot just read goes back to the requester.
__device__ __forceinline__ void release_slot(const Params& p, const Ranges& rg, WarpState& ws, uint64_t* empty) {
    __syncwarp();
    if ((threadIdx.x & 31) == 0) gemvq8::mbar_arrive(&empty[ws.slot]);
    advance(p, rg, ws.cc);
    if (++ws.slot == p.depth) { ws.slot = 0; ws.parity ^= 1u; }
}

// All items of this warp in the GEMV job at ws.cc, out of the ring.
template <int UNIT, int RI, class ScaleT>
__device__ __forceinline__ void run_gemv_items(const Params& p, const Ranges& rg, const KindDesc& k, const Out& out, WarpState& ws,
                                               unsigned char* ring, uint64_t* full, uint64_t* empty, const unsigned char* planes, float resv) {
    constexpr int RT = UNIT * RI;
    const int lane = threadIdx.x & 31;
    const int jid = ws.cc.job, kind = ws.cc.kind;
    const int g_first = rg.r[kind].first;
    float acc[RT];
#pragma unroll
    for (int r = 0; r < RT; ++r) acc[r] = 0.f;
    // optional split of this warp's time (first warp of the grid only): waiting for a slot, multiplying, storing, releasing
    const bool timed = p.prof != nullptr && blockIdx.x == 0 && threadIdx.x < 32;
    long long t_wait = 0, t_mul = 0, t_store = 0, t_rel = 0;
    while (ws.cc.job == jid) {
        const long long t0 = timed ? clock64() : 0;
        if (ws.alive && !ringq8::ring_wait(&full[ws.slot], ws.parity, p.status)) ws.alive = false;
        const long long t1 = timed ? clock64() : 0;
        int g = g_first, ch = 0;
        if (k.nc == 1) g += ws.cc.idx;
        else { g += ws.cc.idx / k.nc; ch = ws.cc.idx % k.nc; }
        long long t2 = t1;
        if (ws.alive) {
            ringq8::consume_item<RT, ScaleT>(ring + (size_t)ws.slot * p.slot_bytes, k.kc, ch * k.kc, planes, k.K, acc);
            if (timed) t2 = clock64();
            if (ch == k.nc - 1) store_item<UNIT, RI>(p, out, g * RI, k.n_units, acc, resv, g_first * RI);
        }
        const long long t3 = timed ? clock64() : 0;
        release_slot(p, rg, ws, empty);
        if (timed) {
            const long long t4 = clock64();
            t_wait += t1 - t0; t_mul += t2 - t1; t_store += t3 - t2; t_rel += t4 - t3;
        }
    }
    if (timed && lane == 0) {
        unsigned long long* acc_t = p.prof + 2 * n_jobs_of(p) + 1 + 4 * kind;
        acc_t[0] += (unsigned long long)t_wait; acc_t[1] += (unsigned long long)t_mul;
        acc_t[2] += (unsigned long long)t_store; acc_t[3] += (unsigned long long)t_rel;
    }
}

// ------------------------------------------------------------------------------------------------
// Attention.  Per-warp scratch in shared memory: a raw row and the rotated q, HD floats each.
template <int HD> struct WarpAttn {
    float raw[HD];
    float q[HD];
};
// Partial result of one warp / one CTA for a head: m, l, unnormalised o.
template <int HD> struct Part {
    float m, l;
    float o[HD];
};
template <int HD, int NW> struct AttnShared {
    WarpAttn<HD> w[NW];
    Part<HD> part[2][NW];                // [head slot of this CTA][warp]
};

// HD tagged words starting at word `off` -> floats in `dst` (all lanes; HD / 4 lanes carry four values each)
template <int HD>
__device__ __forceinline__ void fetch_row(const Params& p, uint32_t off, uint32_t tag, float* dst) {
    const int lane = threadIdx.x & 31;
    if (lane < HD / 4) {
        const uint32_t* words = p.win + off;
        uint4 w = gemvq8::ll_load4(words + 4 * lane);
        gemvq8::ll_wait4(words, lane, tag, p.status, w);
        const uint2 h = gemvq8::ll_pack4(w);
        const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&h.x));
        const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&h.y));
        dst[4 * lane] = f0.x; dst[4 * lane + 1] = f0.y; dst[4 * lane + 2] = f1.x; dst[4 * lane + 3] = f1.y;
    }
    __syncwarp();
}

// RoPE of one head row as rope.cu / decode.cu do it (cpu/rope.rs:63-143): f32 products rounded one by one, result cast to f16
template <int HD>
__device__ __forceinline__ void rope_row(const float* in, const float* tab, int rope_dim, float* dst) {
    const int lane = threadIdx.x & 31;
    const int half = rope_dim >> 1;
    for (int i = lane; i < HD; i += 32) {
        if (i < half) {
            const float x1 = in[i], x2 = in[i + half];
            const float c = tab[i], s = tab[half + i];
            dst[i] = f16r(__fsub_rn(__fmul_rn(x1, c), __fmul_rn(x2, s)));
            dst[i + half] = f16r(__fadd_rn(__fmul_rn(x1, s), __fmul_rn(x2, c)));
        } else if (i >= rope_dim) {
            dst[i] = in[i];
        }
    }
    __syncwarp();
}

// The same, written as f16 (the rotated values are f16-rounded already) to a tile row and, if asked, to the cache row.
template <int HD>
__device__ __forceinline__ void rope_row_half(const float* in, const float* tab, int rope_dim, __half* dst, __half* cache) {
    const int lane = threadIdx.x & 31;
    const int half = rope_dim >> 1;
    for (int i = lane; i < HD; i += 32) {
        if (i < half) {
            const float x1 = in[i], x2 = in[i + half];
            const float c = tab[i], s = tab[half + i];
            const __half a = __float2half_rn(__fsub_rn(__fmul_rn(x1, c), __fmul_rn(x2, s)));
            const __half b = __float2half_rn(__fadd_rn(__fmul_rn(x1, s), __fmul_rn(x2, c)));
            dst[i] = a;
            dst[i + half] = b;
            if (cache) { cache[i] = a; cache[i + half] = b; }
        } else if (i >= rope_dim) {
            const __half a = __float2half_rn(in[i]);
            dst[i] = a;
            if (cache) cache[i] = a;
        }
    }
    __syncwarp();
}

// Running softmax state of a warp over its tiles: lane l holds output features 2l, 2l+1 and (l < HD/2 - 32) 64+2l, 64+2l+1.
struct Running {
    float m, l;
    float o0, o1, o2, o3;
};

// One landed tile (K rows then V rows in `slot`) folded into the running state.
template <int HD>
__device__ __forceinline__ void attn_tile(const Params& p, const LayerPtrs& lw, int h, int tile, int P, unsigned char* slot, WarpAttn<HD>& ws,
                                          const float* tab, uint32_t qtag, Running& st) {
    const int lane = threadIdx.x & 31;
    const int group = p.H / p.Hkv, kvh = h / group;
    const int begin = tile * kTileP;
    const int T = P + 1;
    __half* Ks = reinterpret_cast<__half*>(slot);
    __half* Vs = Ks + kTileP * HD;
    if (P >= begin && P < begin + kTileP) {
        // this tile holds the new position: rotate k, append both rows to the cache (ops/cache.rs:73-103) and to the tile
        const int row = P - begin;
        const bool to_cache = h % group == 0;
        fetch_row<HD>(p, p.q_off + (uint32_t)(p.H + kvh) * HD, qtag, ws.raw);
        rope_row_half<HD>(ws.raw, tab, p.rope_dim, Ks + row * HD, to_cache ? lw.kc + ((size_t)kvh * p.max_cache + P) * HD : nullptr);
        fetch_row<HD>(p, p.q_off + (uint32_t)(p.H + p.Hkv + kvh) * HD, qtag, ws.raw);
        for (int i = lane; i < HD; i += 32) {
            const __half vh = __float2half_rn(ws.raw[i]);                 // exact: the value was an f16
            Vs[row * HD + i] = vh;
            if (to_cache) lw.vc[((size_t)kvh * p.max_cache + P) * HD + i] = vh;
        }
        __syncwarp();
    }
    // scores: two lanes per position, half a row each
    const int pos = lane >> 1, hf = lane & 1;
    float dot = 0.f;
    if (begin + pos < T) {
        const uint4* kp = reinterpret_cast<const uint4*>(Ks + pos * HD + hf * (HD / 2));
        const float* q = ws.q + hf * (HD / 2);
#pragma unroll
        for (int v = 0; v < HD / 16; ++v) {
            const uint4 w = kp[v];
            const __half2* hp = reinterpret_cast<const __half2*>(&w);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f = __half22float2(hp[j]);
                dot = fmaf(q[v * 8 + 2 * j], f.x, dot);
                dot = fmaf(q[v * 8 + 2 * j + 1], f.y, dot);
            }
        }
    }
    dot += __shfl_xor_sync(0xffffffffu, dot, 1);
    const float sc = begin + pos < T ? f16r(dot * p.scale) : -INFINITY;      // `.mul(scale).cast(f16)` (attn.rs:142-146)
    const float m_tile = warp_max(sc);
    const float m_new = fmaxf(st.m, m_tile);                                  // finite: the tile holds at least one position
    const float corr = expf(st.m - m_new);                                    // 0 on the first tile (m = -inf)
    const float pe = begin + pos < T ? expf(sc - m_new) : 0.f;
    st.l = st.l * corr + 0.5f * warp_sum(pe);                                 // every position sits in two lanes
    st.o0 *= corr; st.o1 *= corr; st.o2 *= corr; st.o3 *= corr;
    const int n = min(kTileP, T - begin);
#pragma unroll
    for (int j = 0; j < kTileP; ++j) {
        const float pj = __shfl_sync(0xffffffffu, pe, 2 * j);
        if (j < n) {
            const __half2* vr = reinterpret_cast<const __half2*>(Vs + j * HD);
            const float2 a = __half22float2(vr[lane]);
            st.o0 = fmaf(pj, a.x, st.o0);
            st.o1 = fmaf(pj, a.y, st.o1);
            if (HD > 64 && lane < HD / 2 - 32) {
                const float2 b = __half22float2(vr[32 + lane]);
                st.o2 = fmaf(pj, b.x, st.o2);
                st.o3 = fmaf(pj, b.y, st.o3);
            }
        }
    }
    st.m = m_new;
}

template <int HD>
__device__ __forceinline__ void write_part(Part<HD>& dst, const Running& st) {
    const int lane = threadIdx.x & 31;
    if (lane == 0) { dst.m = st.m; dst.l = st.l; }
    dst.o[2 * lane] = st.o0;
    dst.o[2 * lane + 1] = st.o1;
    if (HD > 64 && lane < HD / 2 - 32) {
        dst.o[64 + 2 * lane] = st.o2;
        dst.o[64 + 2 * lane + 1] = st.o3;
    }
}

// One warp: merge n partial results (m, l, o[HD]; `stride` floats apart) into (M, L, o); every lane ends with its features.
template <int HD, bool GLOBAL>
__device__ __forceinline__ void merge_parts(const float* parts, int n, int stride, Running& out) {
    const int lane = threadIdx.x & 31;
    auto ld = [&](const float* q) { return GLOBAL ? __ldcg(q) : *q; };
    float M = -INFINITY;
    for (int j = 0; j < n; ++j) M = fmaxf(M, ld(parts + (size_t)j * stride));
    Running r{M, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < n; ++j) {
        const float* q = parts + (size_t)j * stride;
        const float mj = ld(q);
        const float w = mj > -INFINITY ? expf(mj - M) : 0.f;
        r.l = fmaf(ld(q + 1), w, r.l);
        r.o0 = fmaf(ld(q + 2 + 2 * lane), w, r.o0);
        r.o1 = fmaf(ld(q + 2 + 2 * lane + 1), w, r.o1);
        if (HD > 64 && lane < HD / 2 - 32) {
            r.o2 = fmaf(ld(q + 2 + 64 + 2 * lane), w, r.o2);
            r.o3 = fmaf(ld(q + 2 + 64 + 2 * lane + 1), w, r.o3);
        }
    }
    out = r;
}

// The head's output, normalised, as tagged words to every rank.
template <int HD>
__device__ __forceinline__ void publish_head(const Params& p, int h, const Running& r, uint32_t tag) {
    const int lane = threadIdx.x & 31;
    const Out out = make_out(p, p.a_off + (uint32_t)p.a_rank_off, true, tag, K_ATTN);
    const float inv = 1.0f / r.l;
    out.put(p, h * HD + 2 * lane, __float2half_rn(r.o0 * inv));
    out.put(p, h * HD + 2 * lane + 1, __float2half_rn(r.o1 * inv));
    if (HD > 64 && lane < HD / 2 - 32) {
        out.put(p, h * HD + 64 + 2 * lane, __float2half_rn(r.o2 * inv));
        out.put(p, h * HD + 64 + 2 * lane + 1, __float2half_rn(r.o3 * inv));
    }
}

// ------------------------------------------------------------------------------------------------
// Shared memory: [full and empty mbarriers][rope table][16 floats][item ranges of the warps][layer pointers]
// [union: activation planes | attention scratch][rings: NW x depth x slot_bytes].  The host computes the same offsets.
__host__ __device__ constexpr size_t round128(size_t n) { return (n + 127) & ~(size_t)127; }
__host__ __device__ constexpr size_t bars_bytes(int nw) { return (size_t)2 * nw * kMaxDepth * 8; }
__host__ __device__ constexpr size_t ranges_off(int nw) { return bars_bytes(nw) + kMaxRope * sizeof(float) + 16 * sizeof(float); }
__host__ __device__ constexpr size_t layer_ptrs_off(int nw) { return (ranges_off(nw) + nw * sizeof(Ranges) + 15) & ~(size_t)15; }
__host__ __device__ constexpr size_t union_off(int nw, int n_layers) { return round128(layer_ptrs_off(nw) + (size_t)n_layers * sizeof(LayerPtrs)); }
template <int HD, int NW> __host__ __device__ constexpr size_t union_bytes(int kmax) {
    return round128(sizeof(AttnShared<HD, NW>) > (size_t)2 * kmax + (size_t)kmax / 4 ? sizeof(AttnShared<HD, NW>) : (size_t)2 * kmax + (size_t)kmax / 4);
}

// plane-building prologue reading tagged words with a tag computed once.  A thread's sixteen words are polled
// together: every pass re-requests all the groups of four that are still incomplete before it looks at any of
// them, so a vector that lands while the thread waits costs one more trip to L2, not one per group.
struct TaggedSource {
    const uint32_t* words;
    uint32_t tag;
    int* status;
    __device__ __forceinline__ void begin() const {}
    __device__ __forceinline__ void load(int g, float (&v)[16]) const {
        uint4 w[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) w[q] = gemvq8::ll_load4(words + 16 * g + 4 * q);
        unsigned long long t0 = 0;
        for (unsigned int n = 0;; ++n) {
            bool ready[4];
            bool all = true;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                ready[q] = gemvq8::ll_ready4(w[q], tag);
                all = all && ready[q];
            }
            if (all) break;
            if ((n & 63u) == 63u) {
                if (*reinterpret_cast<volatile int*>(status) & RCU_DEVFLAG_TIMEOUT) break;
                const unsigned long long t = ringq8::globaltimer();
                if (t0 == 0) t0 = t;
                else if (t - t0 > rcu_wait_limit(status)) { atomicOr(status, RCU_DEVFLAG_TIMEOUT); break; }
            }
#pragma unroll
            for (int q = 0; q < 4; ++q)
                if (!ready[q]) w[q] = gemvq8::ll_load4(words + 16 * g + 4 * q);
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const uint2 h = gemvq8::ll_pack4(w[q]);
            const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&h.x));
            const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&h.y));
            v[4 * q] = f0.x; v[4 * q + 1] = f0.y; v[4 * q + 2] = f1.x; v[4 * q + 3] = f1.y;
        }
    }
};

template <int HD, class ScaleT, int NW>
__global__ void __launch_bounds__((NW + 1) * 32, 1) decode_flow_kernel(const __grid_constant__ Params p, int kmax) {
    constexpr int NT = NW * 32;                      // consumer threads
    extern __shared__ __align__(128) unsigned char smem_raw[];
    uint64_t* full_bars = reinterpret_cast<uint64_t*>(smem_raw);
    uint64_t* empty_bars = full_bars + NW * kMaxDepth;
    float* tab = reinterpret_cast<float*>(smem_raw + bars_bytes(NW));
    float* scratch = tab + kMaxRope;
    Ranges* rgs = reinterpret_cast<Ranges*>(smem_raw + ranges_off(NW));
    LayerPtrs* lp = reinterpret_cast<LayerPtrs*>(smem_raw + layer_ptrs_off(NW));
    unsigned char* planes = smem_raw + union_off(NW, p.n_layers);
    AttnShared<HD, NW>* ash = reinterpret_cast<AttnShared<HD, NW>*>(planes);
    unsigned char* rings = planes + union_bytes<HD, NW>(kmax);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    const int P = (int)*p.d_pos;
    const int n_tiles = (P + 1 + kTileP - 1) / kTileP;
    const unsigned step = *p.d_step;
    const int n_jobs = n_jobs_of(p);
    if (warp < NW && lane == 0) {
        for (int s = 0; s < p.depth; ++s) {
            gemvq8::mbar_init(&full_bars[warp * kMaxDepth + s], 1);
            gemvq8::mbar_init(&empty_bars[warp * kMaxDepth + s], 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        Ranges& mine = rgs[warp];
        for (int k = 0; k < kKinds; ++k) {
            if (k == K_ATTN) mine.r[k] = attn_range<NW>(p.H, n_tiles, warp, &mine.head);
            else mine.r[k] = gemv_range<NW>(p.kd[k], warp);
        }
    }
    for (int i = tid; i < p.n_layers * (int)(sizeof(LayerPtrs) / 8); i += NT + 32)
        reinterpret_cast<unsigned long long*>(lp)[i] = reinterpret_cast<const unsigned long long*>(p.layers)[i];
    for (int i = tid; i < p.rope_dim; i += NT + 32) tab[i] = p.rope_tab[i];
    __syncthreads();

    if (warp == NW) {
        requester<HD, NW>(p, lp, rgs, P, rings, full_bars, empty_bars);
        return;
    }

    const Ranges& rg = rgs[warp];
    unsigned char* ring = rings + (size_t)warp * p.depth * p.slot_bytes;
    uint64_t* full = full_bars + warp * kMaxDepth;
    uint64_t* empty = empty_bars + warp * kMaxDepth;
    WarpState ws;
    ws.cc = Cursor{0, 0, 0, 0};
    seek(p, rg, ws.cc);
    ws.slot = 0;
    ws.parity = 0;
    ws.alive = true;
    const int wph = warps_per_head<NW>(p.H);
    for (int j = 0; j < n_jobs; ++j) {
        int li, kind;
        split_job(p, j, li, kind);
        ringq8::stage_barrier<NT>();                       // the planes and the attention scratch of job j - 1 are free again
        if (p.prof && blockIdx.x == 0 && tid == 0) p.prof[2 * j] = ringq8::globaltimer();
        if (p.prof_cta && tid == 0) {
            if (j == p.prof_job) p.prof_cta[3 * blockIdx.x] = ringq8::globaltimer();
            if (j == p.prof_job + 1) p.prof_cta[3 * blockIdx.x + 2] = ringq8::globaltimer();
        }
        if (kind != K_ATTN) {
            const KindDesc& k = p.kd[kind];
            // the residuals of this warp's units (final since the job before last): lane i, unit i of the warp
            float resv = 0.f;
            if ((kind == K_O || kind == K_DOWN) && ws.cc.job == j) {
                const int u = rg.r[kind].first * k.ri + lane;
                if (u < k.n_units) resv = __half2float(__ushort_as_half((unsigned short)(__ldcg(p.win + k.res_off + u) & 0xFFFFu)));
            }
            // ---- activation vector -> planes (waits for the words still in flight)
            const TaggedSource src{p.win + k.in_off, make_tag(step, k.in_per_step, (uint32_t)(li * k.in_mul + k.in_add)), p.status};
            if (k.rms) {
                const float* gamma = kind == K_HEAD ? p.out_norm : (kind == K_QKV ? lp[li].attn_norm : lp[li].ffn_norm);
                ringq8::RmsPlanes<TaggedSource, NT> pro{src, gamma, p.eps};
                pro.stage(planes, k.K, scratch);
            } else {
                ringq8::PlainPlanes<TaggedSource, NT> pro{src};
                pro.stage(planes, k.K, scratch);
            }
            ringq8::stage_barrier<NT>();
            if (p.prof && blockIdx.x == 0 && tid == 0) p.prof[2 * j + 1] = ringq8::globaltimer();
            if (p.prof_cta && tid == 0 && j == p.prof_job) p.prof_cta[3 * blockIdx.x + 1] = ringq8::globaltimer();
            if (ws.cc.job != j) continue;
            const Out out = make_out(p, k.out_off, k.push != 0, make_tag(step, k.out_per_step, (uint32_t)(li * k.out_mul + k.out_add)), kind);
            switch (k.unit * 8 + k.ri) {
                case 8 + 1: run_gemv_items<1, 1, ScaleT>(p, rg, k, out, ws, ring, full, empty, planes, resv); break;
                case 8 + 2: run_gemv_items<1, 2, ScaleT>(p, rg, k, out, ws, ring, full, empty, planes, resv); break;
                case 8 + 4: run_gemv_items<1, 4, ScaleT>(p, rg, k, out, ws, ring, full, empty, planes, resv); break;
                case 16 + 1: run_gemv_items<2, 1, ScaleT>(p, rg, k, out, ws, ring, full, empty, planes, resv); break;
                default: run_gemv_items<2, 2, ScaleT>(p, rg, k, out, ws, ring, full, empty, planes, resv); break;
            }
            continue;
        }
        // ---- attention: this warp's run of tiles of one head, folded with an online softmax
        const int h = rg.head;
        Running st{-INFINITY, 0.f, 0.f, 0.f, 0.f, 0.f};
        if (rg.r[K_ATTN].count > 0) {
            const uint32_t qtag = make_tag(step, p.q_per_step, (uint32_t)li);
            WarpAttn<HD>& wa = ash->w[warp];
            fetch_row<HD>(p, p.q_off + (uint32_t)h * HD, qtag, wa.raw);
            rope_row<HD>(wa.raw, tab, p.rope_dim, wa.q);
            while (ws.cc.job == j) {
                if (ws.alive && !ringq8::ring_wait(&full[ws.slot], ws.parity, p.status)) ws.alive = false;
                if (ws.alive)
                    attn_tile<HD>(p, lp[li], h, rg.r[K_ATTN].first + ws.cc.idx, P, ring + (size_t)ws.slot * p.slot_bytes, wa, tab, qtag, st);
                release_slot(p, rg, ws, empty);
            }
        }
        if (p.prof && blockIdx.x == 0 && tid == 0) p.prof[2 * j + 1] = ringq8::globaltimer();     // warp 0's tiles are folded
        // ---- the warps of a head inside this CTA merge through shared memory (a CTA holds warps of at most two heads)
        const int h_first = (blockIdx.x * NW) / wph;
        if (h < p.H) write_part<HD>(ash->part[h - h_first][warp], st);
        ringq8::stage_barrier<NT>();
        if (warp < 2) {
            const int hh = h_first + warp;
            const int gw0 = blockIdx.x * NW;
            const int w0 = max(hh * wph, gw0) - gw0, w1 = min((hh + 1) * wph, gw0 + NW) - gw0;
            if (hh < p.H && w1 > w0) {
                constexpr int kStride = (int)(sizeof(Part<HD>) / sizeof(float));
                const uint32_t atag = make_tag(step, p.a_per_step, (uint32_t)li);
                Running r;
                merge_parts<HD, false>(&ash->part[warp][w0].m, w1 - w0, kStride, r);
                const int cta_first = (hh * wph) / NW, cta_last = ((hh + 1) * wph - 1) / NW;
                const int n_ctas = cta_last - cta_first + 1;
                if (n_ctas == 1) {
                    publish_head<HD>(p, hh, r, atag);
                } else {
                    // ---- the CTAs of a head merge through global scratch; the last one to arrive publishes
                    float* mine = p.partial + ((size_t)hh * p.part_stride + (blockIdx.x - cta_first)) * kStride;
                    if (lane == 0) { mine[0] = r.m; mine[1] = r.l; }
                    mine[2 + 2 * lane] = r.o0;
                    mine[2 + 2 * lane + 1] = r.o1;
                    if (HD > 64 && lane < HD / 2 - 32) {
                        mine[2 + 64 + 2 * lane] = r.o2;
                        mine[2 + 64 + 2 * lane + 1] = r.o3;
                    }
                    __threadfence();
                    __syncwarp();
                    unsigned int ticket = 0;
                    if (lane == 0) ticket = atomicAdd(&p.counters[hh], 1u);
                    ticket = __shfl_sync(0xffffffffu, ticket, 0);
                    if (ticket == (unsigned int)n_ctas - 1) {
                        __threadfence();
                        Running all;
                        merge_parts<HD, true>(p.partial + (size_t)hh * p.part_stride * kStride, n_ctas, kStride, all);
                        publish_head<HD>(p, hh, all, atag);
                        if (lane == 0) p.counters[hh] = 0;       // ready for the next layer
                    }
                }
            }
        }
    }
    if (p.prof && blockIdx.x == 0 && tid == 0) p.prof[2 * n_jobs] = ringq8::globaltimer();
}

}  // namespace flow
