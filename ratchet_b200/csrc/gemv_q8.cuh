// Q8_0 GEMV kernel template shared by the Matmul entry point (plain prologue / epilogue) and the
// decode engine (fused RMSNorm prologue, residual and SiLU-gate epilogues).
//
// y[N] = W[N,K] . x[K], W = ratchet Q8_0 segments (int8 qs row-major, one scale per 32 along K).
// Takes the place of ratchet-core's subgroup_gemv / workgroup_gemv WGSL kernels
// (ops/matmul/subgroup_gemv.rs:89-309, ops/matmul/workgroup_gemv.rs:221-371).
//
// The kernel is HBM-bound: every weight byte is read exactly once.  Layout of the work:
//   * persistent CTAs (a multiple of the SM count), 8 warps each; the Prologue stages the activation
//     vector once per CTA in shared memory (optionally normalising it on the way);
//   * output units (a row, or a gate/up row pair) are dealt to warps as contiguous ranges balanced
//     to one unit, so there is no tail wave;
//   * a warp walks K in 512-element chunks, each lane owning 16 consecutive int8 (one 16-byte
//     streaming load per row per chunk), ROWS rows at a time so that ROWS x UNROLL loads are in
//     flight per lane and the activation registers are reused ROWS times;
//   * int8 -> float conversion is exact, products are accumulated in f32, one f32 multiply by the
//     block scale per 16 elements, warp-shuffle reduction at the end;
//   * small N: KSPLIT warps share a unit range and split K, combined through shared memory.
#pragma once
#include <type_traits>

#include "common.cuh"

namespace gemvq8 {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}

// four packed int8 -> four exact floats: byte ^ 0x80 in the mantissa of 2^23, minus (2^23 + 128)
__device__ __forceinline__ void i8x4_to_f32x4(uint32_t w, float q[4]) {
    const uint32_t t = w ^ 0x80808080u;
    q[0] = __uint_as_float(prmt(t, 0x4B000000u, 0x7440u)) - 8388736.f;
    q[1] = __uint_as_float(prmt(t, 0x4B000000u, 0x7441u)) - 8388736.f;
    q[2] = __uint_as_float(prmt(t, 0x4B000000u, 0x7442u)) - 8388736.f;
    q[3] = __uint_as_float(prmt(t, 0x4B000000u, 0x7443u)) - 8388736.f;
}

// Dot of 16 int8 (one uint4) with 16 activations held in registers.
// MODE 1: activations widened to f32 once per chunk (shared by all ROWS rows), int8 -> f32 through the
// mantissa trick, FFMA: the path for f32 activations (bar 1e-4).  MODE 2 (f16 activations) is Dot16Local below.
template <class ActT, int MODE> struct Dot16;

template <class ActT> struct Dot16<ActT, 1> {
    float x[16];
    __device__ __forceinline__ void load(const ActT* xs, int k) {
        if constexpr (sizeof(ActT) == 4) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float4 v = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(xs) + k + 4 * i);
                x[4 * i] = v.x; x[4 * i + 1] = v.y; x[4 * i + 2] = v.z; x[4 * i + 3] = v.w;
            }
        } else {
            const uint4 a = *reinterpret_cast<const uint4*>(xs + k);
            const uint4 b = *reinterpret_cast<const uint4*>(xs + k + 8);
            const uint32_t h[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h[i]));
                x[2 * i] = f.x; x[2 * i + 1] = f.y;
            }
        }
    }
    __device__ __forceinline__ float dot(const uint4& w) const {
        const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
        float p0 = 0.f, p1 = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float q[4];
            i8x4_to_f32x4(ws[i], q);
            p0 = fmaf(q[0], x[4 * i], p0);
            p1 = fmaf(q[1], x[4 * i + 1], p1);
            p0 = fmaf(q[2], x[4 * i + 2], p0);
            p1 = fmaf(q[3], x[4 * i + 3], p1);
        }
        return p0 + p1;
    }
};

// MODE 2 (f16 activations): the staged vector is re-expressed once per CTA as 16-bit fixed point in
// groups of 16 elements, x = s_g * X with s_g = max|x_g| / 32767, kept as a signed high-byte plane and an
// unsigned low-byte plane (2^-15 of the group's largest element, below f16's own 2^-11 per element; a
// group-local scale keeps that true when the vector holds outliers, as transformer residual streams
// do).  Sixteen int8 codes then meet the planes in eight dp4a and one int -> float conversion.
// A group that holds a NaN or an infinity gets a NaN scale, so every output that depends on it is NaN
// (the f16 arithmetic of the reference gives NaN or an infinity there).
__device__ __forceinline__ int dp4a_ss(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ int dp4a_su(uint32_t a, uint32_t b, int c) {   // signed bytes of a x unsigned bytes of b
    int d;
    asm("dp4a.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// Every 16 activations carry a scale of their own, so building the planes needs no reduction over the
// CTA, only the barrier after it.
struct Dot16Local {
    uint4 h, l;
    float s;
    __device__ __forceinline__ void load(const unsigned char* planes, int K, int k) {
        h = *reinterpret_cast<const uint4*>(planes + k);
        l = *reinterpret_cast<const uint4*>(planes + K + k);
        s = reinterpret_cast<const float*>(planes + 2 * (size_t)K)[k >> 4];
    }
    __device__ __forceinline__ float dot(const uint4& w) const {
        // four chains of two instead of two chains of four: the sums are exact integers, and a warp that has
        // few others to hide behind gets its result two dp4a latencies sooner
        const int h0 = dp4a_ss(w.y, h.y, dp4a_ss(w.x, h.x, 0)), h1 = dp4a_ss(w.w, h.w, dp4a_ss(w.z, h.z, 0));
        const int l0 = dp4a_su(w.y, l.y, dp4a_su(w.x, l.x, 0)), l1 = dp4a_su(w.w, l.w, dp4a_su(w.z, l.z, 0));
        return (float)((h0 + h1) * 256 + (l0 + l1)) * s;
    }
};

// planes: [K signed high bytes][K unsigned low bytes][K / 16 f32 scales]; all kThreads threads; ends with a CTA barrier
__device__ __forceinline__ void stage_fixed_planes_local(const __half* xs, unsigned char* planes, int K) {
    for (int i = threadIdx.x; i < K / 16; i += kThreads) {
        const uint4 u0 = reinterpret_cast<const uint4*>(xs)[2 * i], u1 = reinterpret_cast<const uint4*>(xs)[2 * i + 1];
        const uint32_t hw[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
        float v[16];
        float amax = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&hw[e]));
            v[2 * e] = f.x; v[2 * e + 1] = f.y;
            amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
        }
        bool finite = true;                    // fmaxf drops a NaN operand: look for NaN / infinity separately
#pragma unroll
        for (int e = 0; e < 16; ++e) finite = finite && fabsf(v[e]) <= 65504.f;
        const float inv = (amax > 0.f && finite) ? 32767.f / amax : 0.f;
        uint32_t hi[4] = {0, 0, 0, 0}, lo[4] = {0, 0, 0, 0};
#pragma unroll
        for (int e = 0; e < 16; ++e) {
            const int X = __float2int_rn(finite ? v[e] * inv : 0.f);
            hi[e >> 2] |= (uint32_t)((X >> 8) & 0xFF) << (8 * (e & 3));
            lo[e >> 2] |= (uint32_t)(X & 0xFF) << (8 * (e & 3));
        }
        reinterpret_cast<uint4*>(planes)[i] = make_uint4(hi[0], hi[1], hi[2], hi[3]);
        reinterpret_cast<uint4*>(planes + K)[i] = make_uint4(lo[0], lo[1], lo[2], lo[3]);
        reinterpret_cast<float*>(planes + 2 * (size_t)K)[i] = finite ? amax / 32767.f : __int_as_float(0x7fc00000);
    }
    __syncthreads();
}
template <class ScaleT> __device__ __forceinline__ float ld_scale(const ScaleT* p);
template <> __device__ __forceinline__ float ld_scale<float>(const float* p) { return __ldg(p); }
template <> __device__ __forceinline__ float ld_scale<__half>(const __half* p) {
    return __half2float(__ushort_as_half(__ldg(reinterpret_cast<const unsigned short*>(p))));
}

// ------------------------------------------------------------------------------------------------
// Prologues: stage x[K] into shared memory (all kThreads threads call; caller syncs afterwards).
// `scratch` is kWarps floats of shared memory.
// ------------------------------------------------------------------------------------------------
template <class ActT> struct PlainPrologue {
    const ActT* x;
    __device__ __forceinline__ void stage(ActT* xs, int K, float* /*scratch*/) const {
        const int vec = 16 / (int)sizeof(ActT);
        const uint4* src = reinterpret_cast<const uint4*>(x);
        uint4* dst = reinterpret_cast<uint4*>(xs);
        for (int i = threadIdx.x; i < K / vec; i += kThreads) dst[i] = __ldcg(src + i);   // produced by the previous kernel: read at L2
    }
};

// RMSNorm as ratchet-nn schedules it (ratchet-nn/src/norm.rs:63-69): upcast to f32,
// y = x * (1/sqrt(mean(x^2) + eps)) * gamma (cpu/norm.rs:185-213), cast back to the input dtype.
struct RmsNormPrologueH {
    const __half* x;
    const float* gamma;
    float eps;
    __device__ __forceinline__ void stage(__half* xs, int K, float* scratch) const {
        // one trip to L2: raw values are parked in shared memory while the sum of squares is reduced
        float s2 = 0.f;
        for (int i = threadIdx.x; i < K; i += kThreads) {
            const __half h = __ldcg(x + i);
            xs[i] = h;
            const float v = __half2float(h);
            s2 = fmaf(v, v, s2);
        }
        s2 = warp_sum(s2);
        if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = s2;
        // the kThreads staging threads only (a kernel may run extra warps that do not stage)
        asm volatile("bar.sync 15, %0;" ::"n"(kThreads) : "memory");
        float tot = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) tot += scratch[w];
        const float rstd = 1.0f / sqrtf(tot / (float)K + eps);
        for (int i = threadIdx.x; i < K; i += kThreads) xs[i] = __float2half_rn(__half2float(xs[i]) * rstd * __ldg(gamma + i));
    }
};

// ------------------------------------------------------------------------------------------------
// Epilogues: called by lane 0 (or the combining lanes) with the finished f32 sums of one unit.
// UNIT = rows per unit; row j of unit u is u + j * unit_stride.
// ------------------------------------------------------------------------------------------------
template <class ActT> struct PlainEpilogue {
    static constexpr int UNIT = 1;
    const ActT* bias;
    ActT* y;
    __device__ __forceinline__ void store(int u, const float* acc) const {
        float s = acc[0];
        if (bias) s += to_f32<ActT>(bias[u]);
        y[u] = from_f32<ActT>(s);
    }
    __device__ __forceinline__ void warp_done(int, int) const {}
    __device__ __forceinline__ void finish() const {}
};

// y = residual + Linear(x): the Linear output is rounded to f16 first, then added in f16
// (phi3/model.rs:110-116: `residual.add(attn_output)` on f16 tensors).
struct ResidualEpilogueH {
    static constexpr int UNIT = 1;
    const __half* residual;
    __half* y;
    __device__ __forceinline__ void store(int u, const float* acc) const {
        const float lin = __half2float(__float2half_rn(acc[0]));
        y[u] = __float2half_rn(lin + __half2float(__ldcg(residual + u)));
    }
    __device__ __forceinline__ void warp_done(int, int) const {}
    __device__ __forceinline__ void finish() const {}
};

// Fused gate_up projection of phi3/mlp.rs:31-39: unit u pairs row u (gate) with row u + N/2 (up);
// out[u] = up * f16(silu(f32(gate))), silu(x) = x / (1 + exp(-x)) (cpu/unary.rs:64).
struct SiluGateEpilogueH {
    static constexpr int UNIT = 2;
    __half* y;
    __device__ __forceinline__ void store(int u, const float* acc) const {
        const float gate = __half2float(__float2half_rn(acc[0]));
        const float up = __half2float(__float2half_rn(acc[1]));
        const float act = __half2float(__float2half_rn(gate / (1.0f + expf(-gate))));
        y[u] = __float2half_rn(up * act);
    }
    __device__ __forceinline__ void warp_done(int, int) const {}
    __device__ __forceinline__ void finish() const {}
};

// Output shard of a row-sharded Linear, all-gathered by the kernel itself.  Units are stored into this
// GPU's slice of its own full-size output buffer; a warp that has finished its range of rows copies that
// range into the same place of every peer's buffer with plain stores over NVLink (peer-mapped memory, no
// multicast, no collective library), so the gather proceeds while other warps are still streaming weights.
// A CTA whose warps have all pushed adds one to its arrival counter on every peer (system-scope release);
// the last CTA of the grid then waits (bounded) until every peer's CTAs have arrived here, so the kernel ends
// with the gathered vector complete and no wait launch follows.  The counters only ever grow: what a step
// waits for derives from a device-resident use count of the slot, so a captured launch replays correctly.
constexpr int kMaxPeers = 8;
struct GatherEpilogueH {
    static constexpr int UNIT = 1;
    const __half* bias;                    // local slice of the bias or nullptr
    __half* y_local;                       // this rank's slice inside its own full buffer
    __half* peer_dst[kMaxPeers];           // where the slice goes in each peer's full buffer
    unsigned int* peer_count[kMaxPeers];   // this rank's arrival counter for the slot, on each peer
    int n_peers;
    const unsigned int* my_counts;         // the slot's arrival counters on this rank, one per source rank [world]
    unsigned int* uses;                    // times the slot has been used so far (device memory)
    unsigned int* ticket;                  // zero between launches
    int world, self;
    int* status;
    __device__ __forceinline__ void store(int u, const float* acc) const {
        float s = acc[0];
        if (bias) s += __half2float(bias[u]);
        y_local[u] = __float2half_rn(s);
    }
    // all lanes of a warp, once, after its last unit: rows [u_begin, u_end) are this warp's and final
    __device__ __forceinline__ void warp_done(int u_begin, int u_end) const {
        __syncwarp();                       // the lanes' stores to y_local are ordered before the loads below
        const int lane = threadIdx.x & 31;
#pragma unroll
        for (int p = 0; p < kMaxPeers; ++p) {
            if (p < n_peers) {
                __half* dst = peer_dst[p];
                for (int i = u_begin + lane; i < u_end; i += 32) dst[i] = y_local[i];
            }
        }
        __threadfence_system();
    }
    __device__ __forceinline__ void finish() const {
        __shared__ int is_last;
        __syncthreads();                    // every warp of the CTA has pushed (and fenced) its rows
        if ((int)threadIdx.x < n_peers)
            asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(peer_count[threadIdx.x]) : "memory");
        if (threadIdx.x == 0) {
            const unsigned int t = atomicAdd(ticket, 1u);
            is_last = (t == gridDim.x - 1);
        }
        __syncthreads();
        if (!is_last) return;
        // Thread p polls source rank p's counter (bounded by the device's wait limit, then RCU_DEVFLAG_TIMEOUT).
        const unsigned int target = (*reinterpret_cast<volatile unsigned int*>(uses) + 1u) * gridDim.x;
        const int p = threadIdx.x;
        if (p < world && p != self) {
            unsigned long long t0;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
            for (;;) {
                unsigned int v;
                asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(my_counts + p) : "memory");
                if ((int)(v - target) >= 0) break;
                unsigned long long t;
                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
                if (t - t0 > rcu_wait_limit(status)) {
                    atomicOr(status, RCU_DEVFLAG_TIMEOUT);
                    break;
                }
            }
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            *uses += 1u;
            *ticket = 0;
        }
    }
};

// ------------------------------------------------------------------------------------------------
// Low-latency exchange of short f16 vectors between the GPUs of a node (the all-gathers of a sharded
// decode step).  Every element travels as one 32-bit word: the exchange's sequence number in the
// high half, the f16 bits in the low half.  The producer of an element stores that word straight
// into its own and every peer's window (an aligned 4-byte store is indivisible); a consumer polls a
// word until its high half is the number it expects.  No separate flag, no fence, no ticket: the
// latency of an exchange is one NVLink store, and each producing CTA sends as soon as it has a result.
// Sequence numbers are (step * per_step + idx + 1) mod 65536 with `step` read from device memory, so a
// CUDA graph replays with fresh numbers; a word is rewritten by every exchange that uses its place,
// so the value it held before is always a different number.
// ------------------------------------------------------------------------------------------------
struct LLSeq {
    const unsigned int* step;
    unsigned int per_step, idx;
    __device__ __forceinline__ uint32_t tag() const { return ((__ldg(step) * per_step + idx + 1u) & 0xFFFFu) << 16; }
};

struct LLPush {
    uint32_t* local;               // this rank's window; element u lives at word u (nullptr: not in use)
    uint32_t* peer[kMaxPeers];     // the same place in each peer's window
    int n_peers;
    LLSeq seq;
    __device__ __forceinline__ void put(int u, __half v) const {
        const uint32_t word = seq.tag() | (uint32_t)__half_as_ushort(v);
        local[u] = word;
#pragma unroll
        for (int p = 0; p < kMaxPeers; ++p)      // unrolled with a predicate: the pointers stay in the parameter bank
            if (p < n_peers) peer[p][u] = word;
    }
};

// Four consecutive words at once (16-byte aligned): each word is still written by one indivisible
// 4-byte store, so the vector load may see any mix of old and new words but never a torn one.
__device__ __forceinline__ uint4 ll_load4(const uint32_t* p) {
    uint4 v;
    asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ bool ll_ready4(const uint4& v, uint32_t tag) {
    return (((v.x ^ tag) | (v.y ^ tag) | (v.z ^ tag) | (v.w ^ tag)) & 0xFFFF0000u) == 0u;
}
// Re-polls `v` (words 4 i .. 4 i + 3) until all four carry `tag`.  The wait is bounded in time (the device's
// wait limit, two seconds by default); a wait that runs out, or finds that another one already did, records RCU_DEVFLAG_TIMEOUT and
// goes on with what is there.
__device__ __forceinline__ void ll_wait4(const uint32_t* words, int i, uint32_t tag, int* status, uint4& v) {
    unsigned long long t0 = 0;
    for (unsigned int n = 0; !ll_ready4(v, tag); ++n) {
        if ((n & 63u) == 63u) {
            if (*reinterpret_cast<volatile int*>(status) & RCU_DEVFLAG_TIMEOUT) break;
            unsigned long long t;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
            if (t0 == 0) t0 = t;
            else if (t - t0 > rcu_wait_limit(status)) { atomicOr(status, RCU_DEVFLAG_TIMEOUT); break; }
        }
        v = ll_load4(words + 4 * i);
    }
}
// the four f16 values of four words, packed
__device__ __forceinline__ uint2 ll_pack4(const uint4& v) {
    return make_uint2((v.x & 0xFFFFu) | (v.y << 16), (v.z & 0xFFFFu) | (v.w << 16));
}

struct LLSource {
    const uint32_t* words;         // this rank's window
    LLSeq seq;
    int* status;
};

// Prologues reading x from an exchange (the plain ones above read an ordinary f16 vector).  A thread
// requests two groups of four words before it checks the first: a trip to L2 costs most of a
// microsecond, and the words that are already there (usually all of them) need no second look.
struct LLPlainPrologueH {
    LLSource src;
    __device__ __forceinline__ void stage(__half* xs, int K, float* /*scratch*/) const {
        const uint32_t tag = src.seq.tag();
        const int nvec = K >> 2;
        uint2* dst = reinterpret_cast<uint2*>(xs);
        for (int i = threadIdx.x; i < nvec; i += 2 * kThreads) {
            const bool second = i + kThreads < nvec;
            uint4 a = ll_load4(src.words + 4 * i);
            uint4 b = a;
            if (second) b = ll_load4(src.words + 4 * (i + kThreads));
            ll_wait4(src.words, i, tag, src.status, a);
            dst[i] = ll_pack4(a);
            if (second) {
                ll_wait4(src.words, i + kThreads, tag, src.status, b);
                dst[i + kThreads] = ll_pack4(b);
            }
        }
    }
};

struct LLRmsNormPrologueH {
    LLSource src;
    const float* gamma;
    float eps;
    __device__ __forceinline__ void stage(__half* xs, int K, float* scratch) const {
        const uint32_t tag = src.seq.tag();
        const int nvec = K >> 2;
        uint2* dst = reinterpret_cast<uint2*>(xs);
        for (int i = threadIdx.x; i < nvec; i += 2 * kThreads) {
            const bool second = i + kThreads < nvec;
            uint4 a = ll_load4(src.words + 4 * i);
            uint4 b = a;
            if (second) b = ll_load4(src.words + 4 * (i + kThreads));
            ll_wait4(src.words, i, tag, src.status, a);
            dst[i] = ll_pack4(a);
            if (second) {
                ll_wait4(src.words, i + kThreads, tag, src.status, b);
                dst[i + kThreads] = ll_pack4(b);
            }
        }
        asm volatile("bar.sync 15, %0;" ::"n"(kThreads) : "memory");
        // the sum of squares runs over shared memory in the element order of RmsNormPrologueH, so that a
        // sharded step normalises with exactly the factor of the single-GPU step
        float s2 = 0.f;
        for (int i = threadIdx.x; i < K; i += kThreads) {
            const float v = __half2float(xs[i]);
            s2 = fmaf(v, v, s2);
        }
        s2 = warp_sum(s2);
        if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = s2;
        asm volatile("bar.sync 15, %0;" ::"n"(kThreads) : "memory");
        float tot = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) tot += scratch[w];
        const float rstd = 1.0f / sqrtf(tot / (float)K + eps);
        for (int i = threadIdx.x; i < K; i += kThreads) xs[i] = __float2half_rn(__half2float(xs[i]) * rstd * __ldg(gamma + i));
    }
};

// Epilogues sending their slice of the output to every rank (u = row within this rank's shard; the
// window pointers of LLPush already point at the shard's first element).
struct LLPlainEpilogueH {
    static constexpr int UNIT = 1;
    LLPush out;
    __device__ __forceinline__ void store(int u, const float* acc) const { out.put(u, __float2half_rn(acc[0])); }
    __device__ __forceinline__ void warp_done(int, int) const {}
    __device__ __forceinline__ void finish() const {}
};

// y = residual + Linear(x) on this rank's rows of x.  The residual is the rank's own rows of the
// current x: an ordinary f16 vector (`res_plain`, the embedding) or words of the window this epilogue
// then overwrites in place (`res_words`; they were written by this rank itself in an earlier kernel).
struct LLResidualEpilogueH {
    static constexpr int UNIT = 1;
    const __half* res_plain;
    const uint32_t* res_words;
    LLPush out;
    __device__ __forceinline__ void store(int u, const float* acc) const {
        const float lin = __half2float(__float2half_rn(acc[0]));
        const float r = res_plain ? __half2float(__ldcg(res_plain + u))
                                  : __half2float(__ushort_as_half((unsigned short)(__ldcg(res_words + u) & 0xFFFFu)));
        out.put(u, __float2half_rn(lin + r));
    }
    __device__ __forceinline__ void warp_done(int, int) const {}
    __device__ __forceinline__ void finish() const {}
};

struct LLSiluGateEpilogueH {
    static constexpr int UNIT = 2;
    LLPush out;
    __device__ __forceinline__ void store(int u, const float* acc) const {
        const float gate = __half2float(__float2half_rn(acc[0]));
        const float up = __half2float(__float2half_rn(acc[1]));
        const float act = __half2float(__float2half_rn(gate / (1.0f + expf(-gate))));
        out.put(u, __float2half_rn(up * act));
    }
    __device__ __forceinline__ void warp_done(int, int) const {}
    __device__ __forceinline__ void finish() const {}
};

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <class ScaleT, class ActT, int KSPLIT, int UNROLL, int MODE, class Prologue, class Epilogue>
__global__ void __launch_bounds__(kThreads)
gemv_q8_kernel(const int8_t* __restrict__ qs, const ScaleT* __restrict__ scales, Prologue pro, Epilogue epi, int n_units,
               int unit_stride, int K) {
    constexpr int UNIT = Epilogue::UNIT;
    constexpr int ROWS = 4;                     // weight rows in flight per warp iteration
    constexpr int UPI = ROWS / UNIT;            // units per iteration
    extern __shared__ __align__(16) unsigned char smem_raw[];
    ActT* xs = reinterpret_cast<ActT*>(smem_raw);
    float* red = reinterpret_cast<float*>(smem_raw + (size_t)K * sizeof(ActT));  // [kWarps][ROWS]

    // nothing before this point touches data written by the previous kernel in the stream
    pdl_launch_dependents();
    pdl_wait();
    pro.stage(xs, K, red);
    __syncthreads();
    // MODE 2: fixed-point byte planes of x (with 16-element scales) behind the reduction scratch
    unsigned char* planes = smem_raw + (size_t)K * sizeof(ActT) + kWarps * 4 * sizeof(float);
    if constexpr (MODE == 2) stage_fixed_planes_local(reinterpret_cast<const __half*>(xs), planes, K);

    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    constexpr int RG = kWarps / KSPLIT;          // independent unit ranges per CTA
    const int rg = warp / KSPLIT, ks = warp % KSPLIT;
    const long long gw = (long long)blockIdx.x * RG + rg;
    const long long W = (long long)gridDim.x * RG;
    // whole groups of UPI units are dealt (balanced to one group), so only the last group of the matrix
    // can be partial: a warp never spends an iteration on duplicated rows
    const long long n_groups_all = (n_units + UPI - 1) / UPI;
    const int u_begin = (int)((gw * n_groups_all) / W) * UPI;
    const int u_end = min(n_units, (int)(((gw + 1) * n_groups_all) / W) * UPI);
    const int kblocks = K >> 5;
    const int nchunks = (K + 511) >> 9;
    const int kl = lane << 4;

    for (int u0 = u_begin; u0 < u_end; u0 += UPI) {
        float acc[ROWS];
        const int8_t* wrow[ROWS];
        const ScaleT* srow[ROWS];
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            acc[r] = 0.f;
            const int u = min(u0 + r / UNIT, u_end - 1);     // duplicate the last unit; its result is dropped
            const int row = u + (r % UNIT) * unit_stride;
            wrow[r] = qs + (size_t)row * K;
            srow[r] = scales + (size_t)row * kblocks;
        }
        for (int c0 = ks; c0 < nchunks; c0 += KSPLIT * UNROLL) {
            uint4 w[UNROLL][ROWS];
            float sc[UNROLL][ROWS];
            bool live[UNROLL];
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                const int k = ((c0 + u * KSPLIT) << 9) + kl;
                live[u] = k < K;
#pragma unroll
                for (int r = 0; r < ROWS; ++r) {
                    if (live[u]) {
                        w[u][r] = ld_stream_v4(wrow[r] + k);
                        sc[u][r] = ld_scale<ScaleT>(srow[r] + (k >> 5));
                    } else {
                        w[u][r] = make_uint4(0x0, 0x0, 0x0, 0x0);
                        sc[u][r] = 0.f;
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                if (!live[u]) continue;
                const int k = ((c0 + u * KSPLIT) << 9) + kl;
                typename std::conditional<MODE == 2, Dot16Local, Dot16<ActT, 1>>::type d16;
                if constexpr (MODE == 2) d16.load(planes, K, k);
                else d16.load(xs, k);
#pragma unroll
                for (int r = 0; r < ROWS; ++r) acc[r] = fmaf(d16.dot(w[u][r]), sc[u][r], acc[r]);
            }
        }
#pragma unroll
        for (int r = 0; r < ROWS; ++r) acc[r] = warp_sum(acc[r]);

        if (KSPLIT > 1) {
            if (lane == 0) {
#pragma unroll
                for (int r = 0; r < ROWS; ++r) red[warp * ROWS + r] = acc[r];
            }
            asm volatile("bar.sync %0, %1;" ::"r"(1 + rg), "r"(KSPLIT * 32) : "memory");
            if (ks == 0 && lane < UPI) {
                float s[UNIT];
#pragma unroll
                for (int j = 0; j < UNIT; ++j) {
                    s[j] = 0.f;
#pragma unroll
                    for (int q = 0; q < KSPLIT; ++q) s[j] += red[(rg * KSPLIT + q) * ROWS + lane * UNIT + j];
                }
                if (u0 + lane < u_end) epi.store(u0 + lane, s);
            }
            asm volatile("bar.sync %0, %1;" ::"r"(1 + rg), "r"(KSPLIT * 32) : "memory");
        } else if (lane == 0) {
#pragma unroll
            for (int i = 0; i < UPI; ++i)
                if (u0 + i < u_end) epi.store(u0 + i, &acc[i * UNIT]);
        }
    }
    if (ks == 0) epi.warp_done(u_begin, u_end);
    epi.finish();
}

// Variant for short kernels (the GEMVs of a decode step): two register slots of loads are put in
// flight BEFORE the kernel waits for its predecessor and stages x, and refilled as they are consumed.
// It needs 128 registers (two CTAs per SM); on long, cold streams the plain kernel above, with three
// CTAs per SM, measures faster, on 10-60 MB weights this one does.

// One pipeline slot: the weight vectors and block scales of UNROLL chunks x ROWS rows, in registers.
template <int UNROLL, int ROWS> struct Slot {
    uint4 w[UNROLL][ROWS];
    float sc[UNROLL][ROWS];
};

template <class ScaleT, class ActT, int KSPLIT, int UNROLL, int MODE, class Prologue, class Epilogue>
__global__ void __launch_bounds__(kThreads)
gemv_q8_pipe_kernel(const int8_t* __restrict__ qs, const ScaleT* __restrict__ scales, Prologue pro, Epilogue epi, int n_units,
               int unit_stride, int K) {
    constexpr int UNIT = Epilogue::UNIT;
    constexpr int ROWS = 4;                     // weight rows in flight per warp iteration
    constexpr int UPI = ROWS / UNIT;            // units per iteration
    extern __shared__ __align__(16) unsigned char smem_raw[];
    ActT* xs = reinterpret_cast<ActT*>(smem_raw);
    float* red = reinterpret_cast<float*>(smem_raw + (size_t)K * sizeof(ActT));  // [kWarps][ROWS]
    // MODE 2: fixed-point byte planes of x (with 16-element scales) behind the reduction scratch
    unsigned char* planes = smem_raw + (size_t)K * sizeof(ActT) + kWarps * 4 * sizeof(float);

    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    constexpr int RG = kWarps / KSPLIT;          // independent unit ranges per CTA
    const int rg = warp / KSPLIT, ks = warp % KSPLIT;
    const long long gw = (long long)blockIdx.x * RG + rg;
    const long long W = (long long)gridDim.x * RG;
    // whole groups of UPI units are dealt (balanced to one group), so only the last group of the matrix
    // can be partial: a warp never spends an iteration on duplicated rows
    const long long n_groups_all = (n_units + UPI - 1) / UPI;
    const int u_begin = (int)((gw * n_groups_all) / W) * UPI;
    const int u_end = min(n_units, (int)(((gw + 1) * n_groups_all) / W) * UPI);
    const int kblocks = K >> 5;
    const int nchunks = (K + 511) >> 9;
    const int kl = lane << 4;
    // work items of this warp: (unit group, chunk group), chunk groups innermost
    const int n_groups = (u_end - u_begin + UPI - 1) / UPI;
    const int ncg = (nchunks - ks + KSPLIT * UNROLL - 1) / (KSPLIT * UNROLL);
    const int n_items = n_groups * ncg;

    auto load_item = [&](int it, Slot<UNROLL, ROWS>& s) {
        const int u0 = u_begin + (it / ncg) * UPI;
        const int c0 = ks + (it % ncg) * (KSPLIT * UNROLL);
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int k = ((c0 + u * KSPLIT) << 9) + kl;
            const bool live = k < K;
#pragma unroll
            for (int r = 0; r < ROWS; ++r) {
                const int un = min(u0 + r / UNIT, u_end - 1);     // duplicate the last unit; its result is dropped
                const size_t row = (size_t)(un + (r % UNIT) * unit_stride);
                if (live) {
                    s.w[u][r] = ld_stream_v4(qs + row * K + k);
                    s.sc[u][r] = ld_scale<ScaleT>(scales + row * kblocks + (k >> 5));
                } else {
                    s.w[u][r] = make_uint4(0x0, 0x0, 0x0, 0x0);
                    s.sc[u][r] = 0.f;
                }
            }
        }
    };

    float acc[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) acc[r] = 0.f;

    auto compute_item = [&](int it, const Slot<UNROLL, ROWS>& s) {
        const int c0 = ks + (it % ncg) * (KSPLIT * UNROLL);
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int k = ((c0 + u * KSPLIT) << 9) + kl;
            if (k < K) {
                typename std::conditional<MODE == 2, Dot16Local, Dot16<ActT, 1>>::type d16;
                if constexpr (MODE == 2) d16.load(planes, K, k);
                else d16.load(xs, k);
#pragma unroll
                for (int r = 0; r < ROWS; ++r) acc[r] = fmaf(d16.dot(s.w[u][r]), s.sc[u][r], acc[r]);
            }
        }
        if (it % ncg != ncg - 1) return;
        // last chunk group of this unit group: reduce and store
        const int u0 = u_begin + (it / ncg) * UPI;
#pragma unroll
        for (int r = 0; r < ROWS; ++r) acc[r] = warp_sum(acc[r]);
        if (KSPLIT > 1) {
            if (lane == 0) {
#pragma unroll
                for (int r = 0; r < ROWS; ++r) red[warp * ROWS + r] = acc[r];
            }
            asm volatile("bar.sync %0, %1;" ::"r"(1 + rg), "r"(KSPLIT * 32) : "memory");
            if (ks == 0 && lane < UPI) {
                float sum[UNIT];
#pragma unroll
                for (int j = 0; j < UNIT; ++j) {
                    sum[j] = 0.f;
#pragma unroll
                    for (int q = 0; q < KSPLIT; ++q) sum[j] += red[(rg * KSPLIT + q) * ROWS + lane * UNIT + j];
                }
                if (u0 + lane < u_end) epi.store(u0 + lane, sum);
            }
            asm volatile("bar.sync %0, %1;" ::"r"(1 + rg), "r"(KSPLIT * 32) : "memory");
        } else if (lane == 0) {
#pragma unroll
            for (int i = 0; i < UPI; ++i)
                if (u0 + i < u_end) epi.store(u0 + i, &acc[i * UNIT]);
        }
#pragma unroll
        for (int r = 0; r < ROWS; ++r) acc[r] = 0.f;
    };

    // The weights do not depend on the kernel before this one: put the first loads in flight, let
    // the next kernel start launching, and only then wait for the producer of x and stage x.
    Slot<UNROLL, ROWS> s0, s1;
    pdl_launch_dependents();
    if (n_items > 0) load_item(0, s0);
    if (n_items > 1) load_item(1, s1);
    pdl_wait();
    pro.stage(xs, K, red);
    __syncthreads();
    if constexpr (MODE == 2) stage_fixed_planes_local(reinterpret_cast<const __half*>(xs), planes, K);

    for (int it = 0; it < n_items; it += 2) {
        compute_item(it, s0);
        if (it + 2 < n_items) load_item(it + 2, s0);
        if (it + 1 < n_items) {
            compute_item(it + 1, s1);
            if (it + 3 < n_items) load_item(it + 3, s1);
        }
    }
    if (ks == 0) epi.warp_done(u_begin, u_end);
    epi.finish();
}

struct Plan { int ksplit; int grid; };

// Pick the K split and grid: enough warps in flight to cover HBM latency even when N is small.
inline Plan plan(const rcu_device* dev, int n_units, int unit, int K, int ctas_per_sm = 3) {
    Plan p;
    const long long max_ctas = (long long)dev->sm_count * ctas_per_sm;
    const int upi = 4 / unit;
    const long long groups = (n_units + upi - 1) / upi;
    const long long warps_wanted = max_ctas * kWarps;
    int ksplit = 1;
    while (ksplit < 8 && groups * ksplit * 2 <= warps_wanted && (K / (ksplit * 2)) >= 1024) ksplit *= 2;
    // Groups are dealt whole to the warp teams (kWarps / ksplit per CTA).  With only a few groups per team
    // the team that gets one more sets the kernel's time: when that imbalance (rounds of the busiest team
    // over the average) exceeds 6 %, take the K split that minimises it while every warp keeps two chunks.
    auto imbalance = [&](int ks) {
        const double teams = (double)max_ctas * (kWarps / ks);
        const double avg = (double)groups / teams;
        return avg <= 0.0 ? 1.0 : (double)((groups + (long long)teams - 1) / (long long)teams) / avg;
    };
    if (groups * ksplit > warps_wanted / 2 && imbalance(ksplit) > 1.06) {
        int best = ksplit;
        for (int ks = ksplit * 2; ks <= 8 && (K / (ks * 2)) >= 1024; ks *= 2)
            if (imbalance(ks) < imbalance(best) - 0.01) best = ks;
        ksplit = best;
    }
    p.ksplit = ksplit;
    const long long ctas_needed = (groups * ksplit + kWarps - 1) / kWarps;
    p.grid = (int)(ctas_needed < max_ctas ? (ctas_needed < 1 ? 1 : ctas_needed) : max_ctas);
    return p;
}

template <class ScaleT, class ActT, int MODE, class Prologue, class Epilogue>
// overlap = launch with programmatic stream serialization: the kernel may start while its predecessor
// in the stream is still draining; it touches nothing but weights until griddepcontrol.wait returns.
rcu_status launch(rcu_device* dev, const int8_t* qs, const void* scales, const Prologue& pro, const Epilogue& epi, int N, int K,
                  bool overlap = false, int ctas_per_sm = 3, bool pipelined = false) {
    constexpr int UNROLL = 2;
    if (pipelined && ctas_per_sm > 2) ctas_per_sm = 2;
    constexpr int UNIT = Epilogue::UNIT;
    const int n_units = N / UNIT;
    const Plan p = plan(dev, n_units, UNIT, K, ctas_per_sm);
    const size_t smem = (size_t)K * sizeof(ActT) + kWarps * 4 * sizeof(float) + (MODE == 2 ? 2 * (size_t)K + (size_t)K / 4 : 0);
    if (smem > (size_t)dev->smem_optin) return rcu_fail(dev, RCU_ERR_UNSUPPORTED, "gemv: K=%d does not fit the activation stage", K);
#define RCU_GEMV_Q8_CASE(KS)                                                                                  \
    case KS: {                                                                                                \
        auto kern = pipelined ? gemv_q8_pipe_kernel<ScaleT, ActT, KS, UNROLL, MODE, Prologue, Epilogue>       \
                              : gemv_q8_kernel<ScaleT, ActT, KS, UNROLL, MODE, Prologue, Epilogue>;            \
        if (smem > 48 * 1024) RCU_CUDA(dev, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        cudaLaunchConfig_t cfg = {};                                                                          \
        cfg.gridDim = dim3(p.grid); cfg.blockDim = dim3(kThreads); cfg.dynamicSmemBytes = smem; cfg.stream = dev->stream; \
        cudaLaunchAttribute attr[1];                                                                          \
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;                                      \
        attr[0].val.programmaticStreamSerializationAllowed = 1;                                               \
        cfg.attrs = attr; cfg.numAttrs = overlap ? 1 : 0;                                                     \
        RCU_CUDA(dev, cudaLaunchKernelEx(&cfg, kern, qs, (const ScaleT*)scales, pro, epi, n_units, N / UNIT, K)); \
        break;                                                                                                \
    }
    switch (p.ksplit) {
        RCU_GEMV_Q8_CASE(1)
        RCU_GEMV_Q8_CASE(2)
        RCU_GEMV_Q8_CASE(4)
        RCU_GEMV_Q8_CASE(8)
    }
#undef RCU_GEMV_Q8_CASE
    RCU_LAUNCH_CHECK(dev);
    return RCU_OK;
}

}  // namespace gemvq8
