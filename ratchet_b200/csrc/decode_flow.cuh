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
//     tensor maps, no multicast).  While a warp waits
//     for the activation vector of one matrix, its slots fill with rows of that matrix and of the next,
//     so HBM keeps streaming across the hand-overs.
// Arithmetic and rounding points are those of the per-kernel step: gemvq8's dp4a inner product on
// 16-bit fixed-point planes, its prologues and epilogues, and split-KV attention with f16-rounded
// scores (phi3/attn.rs:142-157).
//
// Attention: head h belongs to the CTAs [h * stride, h * stride + c) with stride = grid / heads and c = the
// CTAs a head needs so that a warp folds about two 16-position tiles (at most eight, at most stride).
// A warp owns a contiguous run of tiles and folds them with an online softmax, its q in registers; the
// warps of a CTA merge through shared memory; with c = 1 that CTA publishes the head's output as tagged
// words at once, otherwise the head's CTAs merge through a small global scratch and a per-head ticket
// and the last one publishes (every partial result requested before any is used: one trip to L2).
// The CTAs without a head keep requesting the weights of the jobs ahead.
//
// Every wait (mbarrier, tagged word) is bounded by the device's wait limit; a wait that runs out raises
// RCU_DEVFLAG_TIMEOUT, after which every other wait returns at once and the kernel runs to its end
// with meaningless results instead of hanging.
#pragma once
#include "ring.cuh"

namespace flow {

// cached positions per attention item (K rows, then V rows, in one ring slot).  Sixteen measured faster than
// thirty-two (fewer, larger items leave a head's warps with less to overlap).
template <int HD> __host__ __device__ constexpr int tile_positions() { return 16; }
constexpr int kSubP = 16;                // positions folded per pass: two lanes per position
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
    unsigned long long* partial;         // [H][part_stride][HD + 2] tagged 64-bit words: partial results between the CTAs of a head
    int part_stride;                     // CTAs per head the scratch is laid out for
    // ring
    int slot_bytes, depth;
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

// CTAs per head for this step's cached length, and the head (or -1) this CTA works for.
constexpr int kTilesPerWarp = 2;
constexpr int kMaxCtasPerHead = 8;
template <int NW> __device__ __forceinline__ int ctas_per_head(int H, int n_tiles) {
    const int stride = min((int)gridDim.x / H, kMaxCtasPerHead);
    const int want = (n_tiles + NW * kTilesPerWarp - 1) / (NW * kTilesPerWarp);
    return min(stride, max(1, want));
}
__device__ __forceinline__ int head_of_cta(int H, int cph) {
    const int stride = (int)gridDim.x / H;
    const int h = (int)blockIdx.x / stride;
    return (h < H && (int)blockIdx.x - h * stride < cph) ? h : -1;
}

template <int NW>
__device__ __forceinline__ Range attn_range(int H, int n_tiles, int warp, int* head) {
    const int cph = ctas_per_head<NW>(H, n_tiles);
    const int h = head_of_cta(H, cph);
    *head = h;
    if (h < 0) return Range{0, 0};
    const int stride = (int)gridDim.x / H;
    const int s = ((int)blockIdx.x - h * stride) * NW + warp, n = cph * NW;      // this warp among the head's warps
    const int t0 = s * n_tiles / n, t1 = (s + 1) * n_tiles / n;
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

// One thread: request the item at `c` into `slot` (completion on `bar`).
template <int HD>
__device__ __forceinline__ void issue(const Params& p, const LayerPtrs* lp, const Ranges& rg, const Cursor& c, int P, unsigned char* slot, uint64_t* bar) {
    if (c.kind == K_ATTN) {
        const int h = rg.head, kvh = h / (p.H / p.Hkv);
        const int begin = (rg.r[K_ATTN].first + c.idx) * tile_positions<HD>();
        const int n_cached = min(tile_positions<HD>(), P - begin);                     // rows already in the cache (the tile may also hold position P)
        const unsigned bytes = n_cached > 0 ? (unsigned)n_cached * HD * 2u : 0u;
        const __half* kc = lp[c.li].kc + ((size_t)kvh * p.max_cache + begin) * HD;
        const __half* vc = lp[c.li].vc + ((size_t)kvh * p.max_cache + begin) * HD;
        gemvq8::mbar_expect_tx(bar, 2u * bytes);
        if (bytes) {
            gemvq8::bulk_load_1d(slot, kc, bytes, bar);
            gemvq8::bulk_load_1d(slot + tile_positions<HD>() * HD * 2, vc, bytes, bar);
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
    gemvq8::mbar_expect_tx(bar, (unsigned)(k.unit * nr * (k.kc + sc_row)));
    unsigned char* sdst = slot + k.unit * k.ri * k.kc;
    for (int b = 0; b < k.unit; ++b) {
        const size_t row0 = (size_t)u0 + (size_t)b * k.n_units;    // the up rows follow the gate rows
        if (k.nc == 1) {
            gemvq8::bulk_load_1d(slot + b * k.ri * k.kc, w + row0 * k.K, (uint32_t)(nr * k.kc), bar);
            gemvq8::bulk_load_1d(sdst + b * k.ri * sc_row, scales + row0 * sc_pitch, (uint32_t)(nr * sc_row), bar);
        } else {
            for (int r = 0; r < nr; ++r) {
                const int8_t* qsrc = w + (row0 + r) * k.K + (size_t)ch * k.kc;
                const unsigned char* ssrc = scales + (row0 + r) * sc_pitch + (size_t)ch * sc_row;
                gemvq8::bulk_load_1d(slot + (b * k.ri + r) * k.kc, qsrc, (uint32_t)k.kc, bar);
                gemvq8::bulk_load_1d(sdst + (b * k.ri + r) * sc_row, ssrc, (uint32_t)sc_row, bar);
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
    int slot = 0, round = 0;
    unsigned long long t0 = 0;
    unsigned spins = 0;
    while (pc.job < n_jobs) {
        bool is_free = round == 0;
        if (!is_free) is_free = gemvq8::mbar_test_wait(&empty[slot], (unsigned)(round - 1) & 1u);
        if (is_free) {
            issue<HD>(p, lp, rg, pc, P, ring + (size_t)slot * p.slot_bytes, &full[slot]);
            advance(p, rg, pc);
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
// Attention.  Per-warp scratch in shared memory: raw q / k / v rows and the rotated q, HD floats each.
template <int HD> struct WarpAttn {
    float raw[HD];
    float q[HD];
    float raw_k[HD];     // the new position's k and v rows (only the warp whose tiles hold that position fetches them)
    float raw_v[HD];
};
// Partial result of one warp / one CTA for a head: m, l, unnormalised o.
template <int HD> struct Part {
    float m, l;
    float o[HD];
};
template <int HD, int NW> struct AttnShared {
    WarpAttn<HD> w[NW];
    Part<HD> part[NW];                   // one per warp of the CTA
};

// The q row and, if asked, the new k and v rows of a head at once: all words are requested before any is waited for.
template <int HD>
__device__ __forceinline__ void fetch_qkv(const Params& p, uint32_t q_off, uint32_t k_off, uint32_t v_off, bool with_kv, uint32_t tag,
                                          WarpAttn<HD>& wa) {
    const int lane = threadIdx.x & 31;
    if (lane < HD / 4) {
        const uint32_t* qw = p.win + q_off;
        const uint32_t* kw = p.win + k_off;
        const uint32_t* vw = p.win + v_off;
        uint4 a = gemvq8::ll_load4(qw + 4 * lane), b = a, c = a;
        if (with_kv) {
            b = gemvq8::ll_load4(kw + 4 * lane);
            c = gemvq8::ll_load4(vw + 4 * lane);
        }
        unsigned long long t0 = 0;
        for (unsigned int n = 0;; ++n) {
            const bool ra = gemvq8::ll_ready4(a, tag), rb = !with_kv || gemvq8::ll_ready4(b, tag), rc = !with_kv || gemvq8::ll_ready4(c, tag);
            if (ra && rb && rc) break;
            if ((n & 63u) == 63u) {
                if (*reinterpret_cast<volatile int*>(p.status) & RCU_DEVFLAG_TIMEOUT) break;
                const unsigned long long t = ringq8::globaltimer();
                if (t0 == 0) t0 = t;
                else if (t - t0 > rcu_wait_limit(p.status)) { atomicOr(p.status, RCU_DEVFLAG_TIMEOUT); break; }
            }
            if (!ra) a = gemvq8::ll_load4(qw + 4 * lane);
            if (!rb) b = gemvq8::ll_load4(kw + 4 * lane);
            if (!rc) c = gemvq8::ll_load4(vw + 4 * lane);
        }
        auto unpack = [&](const uint4& w, float* dst) {
            const uint2 h = gemvq8::ll_pack4(w);
            const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&h.x));
            const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&h.y));
            dst[4 * lane] = f0.x; dst[4 * lane + 1] = f0.y; dst[4 * lane + 2] = f1.x; dst[4 * lane + 3] = f1.y;
        };
        unpack(a, wa.raw);
        if (with_kv) { unpack(b, wa.raw_k); unpack(c, wa.raw_v); }
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

// Sixteen positions from `begin` of a landed tile (their K rows at Ks, V rows at Vs) folded into the running state.
template <int HD>
__device__ __forceinline__ void attn_tile(const Params& p, const LayerPtrs& lw, int h, int begin, int P, __half* Ks, __half* Vs, WarpAttn<HD>& ws,
                                          const float (&q)[HD / 2], const float* tab, Running& st) {
    const int lane = threadIdx.x & 31;
    const int group = p.H / p.Hkv, kvh = h / group;
    const int T = P + 1;
    if (P >= begin && P < begin + kSubP) {
        // this tile holds the new position: rotate k, append both rows to the cache (ops/cache.rs:73-103) and to the tile
        // (its k and v rows were fetched with q when the job began)
        const int row = P - begin;
        const bool to_cache = h % group == 0;
        rope_row_half<HD>(ws.raw_k, tab, p.rope_dim, Ks + row * HD, to_cache ? lw.kc + ((size_t)kvh * p.max_cache + P) * HD : nullptr);
        for (int i = lane; i < HD; i += 32) {
            const __half vh = __float2half_rn(ws.raw_v[i]);               // exact: the value was an f16
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
        uint4 kw[HD / 16];
#pragma unroll
        for (int v = 0; v < HD / 16; ++v) kw[v] = kp[v];
        float d4[4] = {0.f, 0.f, 0.f, 0.f};            // four chains: the sum's order is fixed, whatever the head it belongs to
#pragma unroll
        for (int v = 0; v < HD / 16; ++v) {
            const __half2* hp = reinterpret_cast<const __half2*>(&kw[v]);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f = __half22float2(hp[j]);
                d4[j] = fmaf(q[v * 8 + 2 * j], f.x, d4[j]);
                d4[j] = fmaf(q[v * 8 + 2 * j + 1], f.y, d4[j]);
            }
        }
        dot = (d4[0] + d4[1]) + (d4[2] + d4[3]);
    }
    dot += __shfl_xor_sync(0xffffffffu, dot, 1);
    const float sc = begin + pos < T ? f16r(dot * p.scale) : -INFINITY;      // `.mul(scale).cast(f16)` (attn.rs:142-146)
    const float m_tile = warp_max(sc);
    const float m_new = fmaxf(st.m, m_tile);                                  // finite: the tile holds at least one position
    const float corr = expf(st.m - m_new);                                    // 0 on the first tile (m = -inf)
    const float pe = begin + pos < T ? expf(sc - m_new) : 0.f;
    st.l = st.l * corr + 0.5f * warp_sum(pe);                                 // every position sits in two lanes
    st.o0 *= corr; st.o1 *= corr; st.o2 *= corr; st.o3 *= corr;
    const int n = min(kSubP, T - begin);
#pragma unroll
    for (int j = 0; j < kSubP; ++j) {
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

// One warp: merge n <= MAXN partial results (m, l, o[HD]; `stride` floats apart) into (M, L, o); every lane ends
// with its features.  All loads are requested before any is used: from global scratch each costs a trip to L2.
template <int HD, bool GLOBAL, int MAXN>
__device__ __forceinline__ void merge_parts(const float* parts, int n, int stride, Running& out) {
    const int lane = threadIdx.x & 31;
    auto ld = [&](const float* q) { return GLOBAL ? __ldcg(q) : *q; };
    constexpr bool kWide = HD > 64;
    const bool wide = kWide && lane < HD / 2 - 32;
    float m[MAXN], l[MAXN], a0[MAXN], a1[MAXN], a2[MAXN], a3[MAXN];
#pragma unroll
    for (int j = 0; j < MAXN; ++j) {
        m[j] = -INFINITY; l[j] = 0.f; a0[j] = a1[j] = a2[j] = a3[j] = 0.f;
        if (j < n) {
            const float* q = parts + (size_t)j * stride;
            m[j] = ld(q);
            l[j] = ld(q + 1);
            a0[j] = ld(q + 2 + 2 * lane);
            a1[j] = ld(q + 2 + 2 * lane + 1);
            if (wide) {
                a2[j] = ld(q + 2 + 64 + 2 * lane);
                a3[j] = ld(q + 2 + 64 + 2 * lane + 1);
            }
        }
    }
    float M = m[0];
#pragma unroll
    for (int j = 1; j < MAXN; ++j) M = fmaxf(M, m[j]);
    Running r{M, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int j = 0; j < MAXN; ++j) {
        const float w = m[j] > -INFINITY ? expf(m[j] - M) : 0.f;
        r.l = fmaf(l[j], w, r.l);
        r.o0 = fmaf(a0[j], w, r.o0);
        r.o1 = fmaf(a1[j], w, r.o1);
        r.o2 = fmaf(a2[j], w, r.o2);
        r.o3 = fmaf(a3[j], w, r.o3);
    }
    out = r;
}

// A partial result as tagged 64-bit words (tag in the high half, the float's bits in the low half): an aligned
// 8-byte store is indivisible, so a reader that finds the tag has the value.
__device__ __forceinline__ void put64(unsigned long long* p, uint32_t tag, float v) {
    *p = ((unsigned long long)tag << 32) | (unsigned long long)__float_as_uint(v);
}
__device__ __forceinline__ unsigned long long ld64(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
template <int HD>
__device__ __forceinline__ void put_part(unsigned long long* dst, uint32_t tag, const Running& r) {
    const int lane = threadIdx.x & 31;
    if (lane == 0) { put64(dst, tag, r.m); put64(dst + 1, tag, r.l); }
    put64(dst + 2 + 2 * lane, tag, r.o0);
    put64(dst + 2 + 2 * lane + 1, tag, r.o1);
    if (HD > 64 && lane < HD / 2 - 32) {
        put64(dst + 2 + 64 + 2 * lane, tag, r.o2);
        put64(dst + 2 + 64 + 2 * lane + 1, tag, r.o3);
    }
}

// The head's first CTA: its own partial `mine` (slot 0) merged with the partials of the head's other CTAs
// (slots 1 .. n - 1 of `parts`), in slot order.  All words are requested together and re-requested together
// until they carry `tag` (bounded by the device's wait limit).
template <int HD, int MAXN>
__device__ __forceinline__ void gather_parts(const unsigned long long* parts, int n, int stride, uint32_t tag, int* status, const Running& mine,
                                             Running& out) {
    const int lane = threadIdx.x & 31;
    constexpr bool kWide = HD > 64;
    const bool wide = kWide && lane < HD / 2 - 32;
    unsigned long long w[MAXN][6];
    const unsigned long long done = (unsigned long long)tag << 32;
#pragma unroll
    for (int j = 1; j < MAXN; ++j) {
#pragma unroll
        for (int e = 0; e < 6; ++e) w[j][e] = done;           // slots beyond n, and the wide features of narrow lanes, count as arrived
    }
    unsigned long long t0 = 0;
    for (unsigned int it = 0;; ++it) {
        // every word that has not arrived is requested again, all of them before any is looked at
#pragma unroll
        for (int j = 1; j < MAXN; ++j) {
            if (j < n) {
                const unsigned long long* q = parts + (size_t)j * stride;
                if (it == 0 || (uint32_t)(w[j][0] >> 32) != tag) w[j][0] = ld64(q);
                if (it == 0 || (uint32_t)(w[j][1] >> 32) != tag) w[j][1] = ld64(q + 1);
                if (it == 0 || (uint32_t)(w[j][2] >> 32) != tag) w[j][2] = ld64(q + 2 + 2 * lane);
                if (it == 0 || (uint32_t)(w[j][3] >> 32) != tag) w[j][3] = ld64(q + 2 + 2 * lane + 1);
                if (wide && (it == 0 || (uint32_t)(w[j][4] >> 32) != tag)) w[j][4] = ld64(q + 2 + 64 + 2 * lane);
                if (wide && (it == 0 || (uint32_t)(w[j][5] >> 32) != tag)) w[j][5] = ld64(q + 2 + 64 + 2 * lane + 1);
            }
        }
        bool all = true;
#pragma unroll
        for (int j = 1; j < MAXN; ++j) {
#pragma unroll
            for (int e = 0; e < 6; ++e) all = all && (uint32_t)(w[j][e] >> 32) == tag;
        }
        if (__all_sync(0xffffffffu, all)) break;
        if ((it & 63u) == 63u) {
            if (*reinterpret_cast<volatile int*>(status) & RCU_DEVFLAG_TIMEOUT) break;
            const unsigned long long t = ringq8::globaltimer();
            if (t0 == 0) t0 = t;
            else if (t - t0 > rcu_wait_limit(status)) { atomicOr(status, RCU_DEVFLAG_TIMEOUT); break; }
        }
    }
    float M = mine.m;
#pragma unroll
    for (int j = 1; j < MAXN; ++j)
        if (j < n) M = fmaxf(M, __uint_as_float((uint32_t)w[j][0]));
    const float w0 = mine.m > -INFINITY ? expf(mine.m - M) : 0.f;
    Running r{M, mine.l * w0, mine.o0 * w0, mine.o1 * w0, mine.o2 * w0, mine.o3 * w0};
#pragma unroll
    for (int j = 1; j < MAXN; ++j) {
        if (j < n) {
            const float mj = __uint_as_float((uint32_t)w[j][0]);
            const float wj = mj > -INFINITY ? expf(mj - M) : 0.f;
            r.l = fmaf(__uint_as_float((uint32_t)w[j][1]), wj, r.l);
            r.o0 = fmaf(__uint_as_float((uint32_t)w[j][2]), wj, r.o0);
            r.o1 = fmaf(__uint_as_float((uint32_t)w[j][3]), wj, r.o1);
            r.o2 = fmaf(__uint_as_float((uint32_t)w[j][4]), wj, r.o2);
            r.o3 = fmaf(__uint_as_float((uint32_t)w[j][5]), wj, r.o3);
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

// Activation vector of a GEMV job -> planes (waits for the words still in flight).
template <int NT>
__device__ __forceinline__ void stage_job(const Params& p, const KindDesc& k, const float* gamma, uint32_t tag, unsigned char* planes, float* scratch) {
    const TaggedSource src{p.win + k.in_off, tag, p.status};
    if (k.rms) {
        ringq8::RmsPlanes<TaggedSource, NT> pro{src, gamma, p.eps};
        pro.stage(planes, k.K, scratch);
    } else {
        ringq8::PlainPlanes<TaggedSource, NT> pro{src};
        pro.stage(planes, k.K, scratch);
    }
}

// The attention job of one consumer warp whose CTA works for head `h`: its run of tiles folded with an online
// softmax, then the merges that end with the head's output published.  Kept out of line: it runs once per
// layer and would otherwise claim registers in the GEMV item loops.
template <int HD, int NW>
__device__ __noinline__ WarpState attention_job(const Params& p, const LayerPtrs& lw, const Ranges& rg, WarpState ws, int li, int j, int P, int n_tiles,
                                                unsigned step, unsigned char* ring, uint64_t* full, uint64_t* empty, AttnShared<HD, NW>* ash,
                                                const float* tab) {
    constexpr int NT = NW * 32;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int h = rg.head;
    Running st{-INFINITY, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (rg.r[K_ATTN].count > 0) {
        const uint32_t qtag = make_tag(step, p.q_per_step, (uint32_t)li);
        WarpAttn<HD>& wa = ash->w[warp];
        const int tile_p = P / tile_positions<HD>(), kvh = h / (p.H / p.Hkv);
        const bool owns_new = rg.r[K_ATTN].first <= tile_p && tile_p < rg.r[K_ATTN].first + rg.r[K_ATTN].count;
        fetch_qkv<HD>(p, p.q_off + (uint32_t)h * HD, p.q_off + (uint32_t)(p.H + kvh) * HD, p.q_off + (uint32_t)(p.H + p.Hkv + kvh) * HD, owns_new, qtag, wa);
        rope_row<HD>(wa.raw, tab, p.rope_dim, wa.q);
        float q[HD / 2];                                // this lane's half of the rotated q
#pragma unroll
        for (int i = 0; i < HD / 2; ++i) q[i] = wa.q[(lane & 1) * (HD / 2) + i];
        while (ws.cc.job == j) {
            if (ws.alive && !ringq8::ring_wait(&full[ws.slot], ws.parity, p.status)) ws.alive = false;
            if (ws.alive) {
                const int begin = (rg.r[K_ATTN].first + ws.cc.idx) * tile_positions<HD>();
                __half* Ks = reinterpret_cast<__half*>(ring + (size_t)ws.slot * p.slot_bytes);
                __half* Vs = Ks + tile_positions<HD>() * HD;
#pragma unroll
                for (int sub = 0; sub < tile_positions<HD>() / kSubP; ++sub)
                    if (begin + sub * kSubP <= P) attn_tile<HD>(p, lw, h, begin + sub * kSubP, P, Ks + sub * kSubP * HD, Vs + sub * kSubP * HD, wa, q, tab, st);
            }
            release_slot(p, rg, ws, empty);
        }
    }
    if (p.prof && blockIdx.x == 0 && tid == 0) p.prof[2 * j + 1] = ringq8::globaltimer();     // warp 0's tiles are folded
    // ---- the warps of the CTA merge through shared memory
    write_part<HD>(ash->part[warp], st);
    ringq8::stage_barrier<NT>();
    if (warp != 0) return ws;
    constexpr int kStride = (int)(sizeof(Part<HD>) / sizeof(float));
    const uint32_t atag = make_tag(step, p.a_per_step, (uint32_t)li);
    Running r;
    merge_parts<HD, false, NW>(&ash->part[0].m, NW, kStride, r);
    const int cph = ctas_per_head<NW>(p.H, n_tiles);
    const int cta_first = h * ((int)gridDim.x / p.H);
    unsigned long long* head_parts = p.partial + (size_t)h * p.part_stride * kStride;
    if (cph == 1) {
        publish_head<HD>(p, h, r, atag);
    } else if ((int)blockIdx.x != cta_first) {
        // ---- the other CTAs of the head hand their partial result to the head's first CTA: every float
        // travels with the exchange's tag in one 64-bit word, so there is no fence and no counter
        put_part<HD>(head_parts + (size_t)(blockIdx.x - cta_first) * kStride, atag, r);
    } else {
        Running all;
        gather_parts<HD, kMaxCtasPerHead>(head_parts, cph, kStride, atag, p.status, r, all);
        publish_head<HD>(p, h, all, atag);
    }
    return ws;
}

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
    const int n_tiles = (P + 1 + tile_positions<HD>() - 1) / tile_positions<HD>();
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
    for (int j = 0; j < n_jobs; ++j) {
        int li, kind;
        split_job(p, j, li, kind);
        ringq8::stage_barrier<NT>();                       // the planes and the attention scratch of job j - 1 are free again
        if (p.prof && blockIdx.x == 0 && tid == 0) p.prof[2 * j] = ringq8::globaltimer();
        if (kind != K_ATTN) {
            const KindDesc& k = p.kd[kind];
            // the residuals of this warp's units (final since the job before last): lane i, unit i of the warp
            float resv = 0.f;
            if ((kind == K_O || kind == K_DOWN) && ws.cc.job == j) {
                const int u = rg.r[kind].first * k.ri + lane;
                if (u < k.n_units) resv = __half2float(__ushort_as_half((unsigned short)(__ldcg(p.win + k.res_off + u) & 0xFFFFu)));
            }
            // ---- activation vector -> planes (waits for the words still in flight)
            const float* gamma = !k.rms ? nullptr : (kind == K_HEAD ? p.out_norm : (kind == K_QKV ? lp[li].attn_norm : lp[li].ffn_norm));
            stage_job<NT>(p, k, gamma, make_tag(step, k.in_per_step, (uint32_t)(li * k.in_mul + k.in_add)), planes, scratch);
            ringq8::stage_barrier<NT>();
            if (p.prof && blockIdx.x == 0 && tid == 0) p.prof[2 * j + 1] = ringq8::globaltimer();
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
        // ---- attention: CTAs that work for a head fold its tiles and merge; the others go on (their requester keeps asking for weights)
        if (rg.head < 0) {
            if (p.prof && blockIdx.x == 0 && tid == 0) p.prof[2 * j + 1] = ringq8::globaltimer();
            continue;
        }
        ws = attention_job<HD, NW>(p, lp[li], rg, ws, li, j, P, n_tiles, step, ring, full, empty, ash, tab);
    }
    if (p.prof && blockIdx.x == 0 && tid == 0) p.prof[2 * n_jobs] = ringq8::globaltimer();
}

}  // namespace flow
