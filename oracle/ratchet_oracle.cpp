// TEST INFRASTRUCTURE, NOT PRODUCT CODE.
//
// CPU restatement of ratchet-core's CPU device (crates/ratchet-core/src/cpu/*.rs,
// crates/ratchet-core/src/quant.rs) plus the shader arithmetic of the ops that have no CPU
// implementation in the reference (Conv1d, Cache, IndexWrite, GGUF-style Q4_K decode).
// Only the tests, the smoke check and the CPU-baseline leg of the benchmark may link or call
// this file; the CUDA library never does.
//
// Parity status
//   * Integer / byte / index work (Q8_0 quantise + dequantise, segment offsets, gather, concat,
//     permute, slice, broadcast, cache, index_write) is bit-defined by quant.rs and cpu/*.rs and
//     restated exactly.
//   * Floating-point results: PARITY UNPINNED at the bit level.  The reference keeps no golden
//     vectors for this path, it cannot be compiled here (Rust, no toolchain), and the exact
//     rounding of matmul / f16 arithmetic lives in un-vendored crates (`gemm` 0.18.0 and
//     `half` 2.3.1).  Their published behaviour is restated: f16/bf16 operations are computed in
//     f32 and rounded to nearest-even after every operation; matmul accumulates in f32.  The
//     reference's own tests pin these ops against torch only within tolerances, and the tests in
//     this repository check this file the same way.
//
// Every function cites the reference file:line it follows.

#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <vector>
#include <algorithm>

#ifdef _OPENMP
#include <omp.h>
#endif

extern "C" {

// dtype codes shared with the tests (same numbering as the C ABI header)
enum { ORC_F32 = 0, ORC_F16 = 1, ORC_BF16 = 2, ORC_I32 = 3, ORC_U32 = 4 };

int orc_num_threads() {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
void orc_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

}  // extern "C"

namespace {

// ---------------------------------------------------------------------------------------------
// f16 / bf16 as storage types; arithmetic = f32 op then round-to-nearest-even (the `half` crate's
// documented semantics for software arithmetic, Cargo.toml:33).
// ---------------------------------------------------------------------------------------------
struct f16_t { uint16_t bits; };
struct bf16_t { uint16_t bits; };

inline float h2f(uint16_t h) { _Float16 v; std::memcpy(&v, &h, 2); return (float)v; }
inline uint16_t f2h(float f) { _Float16 v = (_Float16)f; uint16_t h; std::memcpy(&h, &v, 2); return h; }
inline float bf2f(uint16_t b) { uint32_t u = (uint32_t)b << 16; float f; std::memcpy(&f, &u, 4); return f; }
inline uint16_t f2bf(float f) {
    uint32_t u; std::memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u);  // quiet NaN
    uint32_t round = 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)((u + round) >> 16);
}

template <class T> struct Num;
template <> struct Num<float> {
    static float ld(const float* p, size_t i) { return p[i]; }
    static void st(float* p, size_t i, float v) { p[i] = v; }
    static float r(float v) { return v; }
};
template <> struct Num<f16_t> {
    static float ld(const f16_t* p, size_t i) { return h2f(p[i].bits); }
    static void st(f16_t* p, size_t i, float v) { p[i].bits = f2h(v); }
    static float r(float v) { return h2f(f2h(v)); }
};
template <> struct Num<bf16_t> {
    static float ld(const bf16_t* p, size_t i) { return bf2f(p[i].bits); }
    static void st(bf16_t* p, size_t i, float v) { p[i].bits = f2bf(v); }
    static float r(float v) { return bf2f(f2bf(v)); }
};

inline size_t align256(size_t n) { return (n + 255) / 256 * 256; }  // gpu/align.rs:24-40

inline size_t numel(const int64_t* shape, int rank) {
    size_t n = 1;
    for (int i = 0; i < rank; ++i) n *= (size_t)shape[i];
    return n;
}

// Rust `f32 as i32`: saturating, NaN -> 0.
inline int32_t rust_as_i32(float v) {
    if (std::isnan(v)) return 0;
    if (v >= 2147483648.0f) return INT32_MAX;
    if (v <= -2147483648.0f) return INT32_MIN;
    return (int32_t)v;
}

// ---------------------------------------------------------------------------------------------
// quant.rs:19-49  quantize_inner<Q>.  PACK = values per u32, GROUP = 32, SF = 127 (Q8_0) or 7
// (ratchet's absmax 4-bit scheme, dtype/blocks.rs:200-219).  All arithmetic in Q::FP.
// ---------------------------------------------------------------------------------------------
template <class T>
size_t quantize_absmax(const T* x, size_t n, int pack, float sf, uint8_t* out) {
    const int group = 32;
    const int lshift = group / pack;            // dtype/blocks.rs:174
    const int32_t mask = (1 << lshift) - 1;     // dtype/blocks.rs:175
    size_t q_bytes = align256(n / pack * 4);
    size_t d_bytes = align256(n / group * sizeof(T));
    std::memset(out, 0, q_bytes + d_bytes);
    uint32_t* q = reinterpret_cast<uint32_t*>(out);
    T* dm = reinterpret_cast<T*>(out + q_bytes);
#pragma omp parallel for schedule(static)
    for (int64_t g = 0; g < (int64_t)(n / group); ++g) {
        size_t base = (size_t)g * group;
        float amax = 0.f;
        for (int j = 0; j < group; ++j) amax = std::fmax(amax, std::fabs(Num<T>::ld(x, base + j)));
        float d = Num<T>::r(amax / sf);
        Num<T>::st(dm, g, d);
        for (int p = 0; p < group / pack; ++p) {
            int32_t packed = 0;
            for (int j = 0; j < pack; ++j) {
                float v = Num<T>::r(Num<T>::ld(x, base + p * pack + j) / d);
                v = Num<T>::r(std::round(v));  // Rust round(): half away from zero (quant.rs:41)
                packed |= (rust_as_i32(v) & mask) << (j * lshift);
            }
            q[(base + p * pack) / pack] = (uint32_t)packed;
        }
    }
    return q_bytes + d_bytes;
}

// quant.rs:101-130  dequantize_inner<Q>
template <class T>
void dequantize_absmax(const uint8_t* buf, size_t n, int pack, T* out) {
    const int group = 32;
    const int lshift = group / pack;
    const int rshift = group - lshift;
    size_t q_bytes = align256(n / pack * 4);
    const uint32_t* q = reinterpret_cast<const uint32_t*>(buf);
    const T* dm = reinterpret_cast<const T*>(buf + q_bytes);
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < (int64_t)n; i += pack) {
        float d = Num<T>::ld(dm, i / group);
        uint32_t packed = q[i / pack];
        for (int j = 0; j < pack; ++j) {
            // ((packed << (LSHIFT*(PACK-j-1))) >> RSHIFT) with arithmetic shift on i32
            int32_t v = (int32_t)(packed << (lshift * (pack - j - 1))) >> rshift;
            Num<T>::st(out, i + j, Num<T>::r((float)v) * d);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// GGUF-style Q4_K in ratchet's 4-segment layout: dtype/blocks.rs:124-148 (segment sizes) and
// ratchet-loader/src/gguf/dtype.rs:39-125 (order qs | scales | dmin | d, each padded to 256 B).
// Decode follows ops/matmul/quantized.rs:158-266.
// ---------------------------------------------------------------------------------------------
struct Q4KSeg { size_t qs, scales, dmin, d, total; };
inline Q4KSeg q4k_segments(size_t n, size_t fp) {
    size_t nb = n / 256;
    Q4KSeg s;
    s.qs = 0;
    s.scales = align256(n / 2);
    s.dmin = s.scales + align256(nb * 12);
    s.d = s.dmin + align256(nb * fp);
    s.total = s.d + align256(nb * fp);
    return s;
}

// quantized.rs:158-204: 6-bit (scale, min) of sub-block j in the 12-byte pack
inline void q4k_scale_min(const uint8_t* sc, int j, uint32_t* s, uint32_t* m) {
    if (j < 4) {
        *s = sc[j] & 63u;
        *m = sc[j + 4] & 63u;
    } else {
        *s = (sc[j + 4] & 0xFu) | ((uint32_t)(sc[j - 4] >> 6) << 4);
        *m = (uint32_t)(sc[j + 4] >> 4) | ((uint32_t)(sc[j] >> 6) << 4);
    }
}

template <class T>
void dequantize_q4k(const uint8_t* buf, size_t n, T* out) {
    Q4KSeg seg = q4k_segments(n, sizeof(T));
    const uint8_t* qs = buf + seg.qs;
    const uint8_t* scales = buf + seg.scales;
    const T* dmin = reinterpret_cast<const T*>(buf + seg.dmin);
    const T* dd = reinterpret_cast<const T*>(buf + seg.d);
#pragma omp parallel for schedule(static)
    for (int64_t b = 0; b < (int64_t)(n / 256); ++b) {
        float d = Num<T>::ld(dd, b), mn = Num<T>::ld(dmin, b);
        const uint8_t* sc = scales + b * 12;
        const uint8_t* q = qs + b * 128;
        for (int c = 0; c < 4; ++c) {        // 32-byte chunk = sub-blocks 2c (low nibbles), 2c+1 (high)
            for (int hi = 0; hi < 2; ++hi) {
                uint32_t s, m;
                q4k_scale_min(sc, 2 * c + hi, &s, &m);
                float delta = Num<T>::r((float)s * d);      // quantized.rs:207-208
                float mind = Num<T>::r((float)m * mn);
                for (int l = 0; l < 32; ++l) {
                    uint32_t v = hi ? (q[c * 32 + l] >> 4) : (q[c * 32 + l] & 0xF);
                    // fma(q, delta, -min), single rounding (quantized.rs:230)
                    Num<T>::st(out, (size_t)b * 256 + (2 * c + hi) * 32 + l,
                               std::fmaf((float)v, delta, -mind));
                }
            }
        }
    }
}

// A simple GGUF-style Q4_K quantiser of this repository's own design (the reference has none):
// per 32-weight sub-block min/max -> scale=(max-min)/15, min offset=-min (clamped at >= 0);
// per 256 super-block d = max scale/63, dmin = max offset/63 stored as T; 6-bit codes; 4-bit q.
template <class T>
size_t quantize_q4k(const float* x, size_t n, uint8_t* out) {
    Q4KSeg seg = q4k_segments(n, sizeof(T));
    std::memset(out, 0, seg.total);
    uint8_t* qs = out + seg.qs;
    uint8_t* scales = out + seg.scales;
    T* dmin = reinterpret_cast<T*>(out + seg.dmin);
    T* dd = reinterpret_cast<T*>(out + seg.d);
#pragma omp parallel for schedule(static)
    for (int64_t b = 0; b < (int64_t)(n / 256); ++b) {
        const float* xb = x + b * 256;
        float sc[8], mn[8];
        float max_sc = 0.f, max_mn = 0.f;
        for (int j = 0; j < 8; ++j) {
            float lo = xb[j * 32], hi = xb[j * 32];
            for (int l = 1; l < 32; ++l) { lo = std::fmin(lo, xb[j * 32 + l]); hi = std::fmax(hi, xb[j * 32 + l]); }
            if (lo > 0.f) lo = 0.f;
            sc[j] = (hi - lo) / 15.f;
            mn[j] = -lo;
            max_sc = std::fmax(max_sc, sc[j]);
            max_mn = std::fmax(max_mn, mn[j]);
        }
        float d = Num<T>::r(max_sc / 63.f), dm = Num<T>::r(max_mn / 63.f);
        Num<T>::st(dd, b, d);
        Num<T>::st(dmin, b, dm);
        uint8_t ls[8], lm[8];
        for (int j = 0; j < 8; ++j) {
            int a = d > 0.f ? (int)std::lround(sc[j] / d) : 0;
            int c = dm > 0.f ? (int)std::lround(mn[j] / dm) : 0;
            ls[j] = (uint8_t)std::min(63, std::max(0, a));
            lm[j] = (uint8_t)std::min(63, std::max(0, c));
        }
        uint8_t* s = scales + b * 12;
        for (int j = 0; j < 4; ++j) {
            s[j] = (ls[j] & 63) | ((ls[j + 4] >> 4) << 6);
            s[j + 4] = (lm[j] & 63) | ((lm[j + 4] >> 4) << 6);
            s[j + 8] = (ls[j + 4] & 0xF) | ((lm[j + 4] & 0xF) << 4);
        }
        uint8_t* q = qs + b * 128;
        for (int j = 0; j < 8; ++j) {
            float delta = Num<T>::r((float)ls[j] * d);
            float mind = Num<T>::r((float)lm[j] * dm);
            for (int l = 0; l < 32; ++l) {
                int v = delta > 0.f ? (int)std::lround((xb[j * 32 + l] + mind) / delta) : 0;
                v = std::min(15, std::max(0, v));
                uint8_t& byte = q[(j / 2) * 32 + l];
                if (j & 1) byte |= (uint8_t)(v << 4); else byte |= (uint8_t)v;
            }
        }
    }
    return seg.total;
}

// ---------------------------------------------------------------------------------------------
// Matmul.  Shape rules: ops/matmul/mod.rs:392-466 (compute_dst_shape) and 74-157 (MatmulSpec);
// arithmetic: cpu/gemm.rs:59-127 calls the `gemm` crate with alpha=0, beta=1, f32 accumulation.
// A quantised lhs is dequantised first (quant.rs:132-164) and the bias, which the reference CPU
// matmul drops (cpu/gemm.rs:149-188), is added here in f32 before the single final rounding.
// Generic strided inner kernel: C[b,i,j] = sum_k A[b,i,k] * B[b,k,j].
// ---------------------------------------------------------------------------------------------
template <class T>
void gemm_strided(const T* A, const T* B, const T* bias, T* C, size_t stacks, size_t a_skip, size_t b_skip,
                  size_t M, size_t N, size_t K, int64_t a_rs, int64_t a_cs, int64_t b_rs, int64_t b_cs,
                  int64_t c_rs, int64_t c_cs, bool bias_on_rows) {
    // Pack operands into f32 row-major A[M,K] and Bt[N,K] per stack so the dot loops vectorise.
    for (size_t s = 0; s < stacks; ++s) {
        const T* a = A + s * a_skip;
        const T* b = B + s * b_skip;
        T* c = C + s * M * N;
        std::vector<float> Ap(M * K), Bp(N * K);
#pragma omp parallel for schedule(static)
        for (int64_t i = 0; i < (int64_t)M; ++i)
            for (size_t k = 0; k < K; ++k) Ap[i * K + k] = Num<T>::ld(a, i * a_rs + k * a_cs);
#pragma omp parallel for schedule(static)
        for (int64_t j = 0; j < (int64_t)N; ++j)
            for (size_t k = 0; k < K; ++k) Bp[j * K + k] = Num<T>::ld(b, k * b_rs + j * b_cs);
        const size_t JB = 64;
#pragma omp parallel for schedule(dynamic) collapse(2)
        for (int64_t jb = 0; jb < (int64_t)((N + JB - 1) / JB); ++jb) {
            for (int64_t i = 0; i < (int64_t)M; ++i) {
                const float* ar = &Ap[i * K];
                size_t j1 = std::min(N, (size_t)(jb + 1) * JB);
                for (size_t j = jb * JB; j < j1; ++j) {
                    const float* br = &Bp[j * K];
                    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
                    size_t k = 0;
                    for (; k + 8 <= K; k += 8)
                        for (int u = 0; u < 8; ++u) acc[u] += ar[k + u] * br[k + u];
                    float t = 0.f;
                    for (; k < K; ++k) t += ar[k] * br[k];
                    float sum = ((acc[0] + acc[4]) + (acc[1] + acc[5])) + ((acc[2] + acc[6]) + (acc[3] + acc[7])) + t;
                    if (bias) sum += Num<T>::ld(bias, bias_on_rows ? (size_t)i : j);
                    Num<T>::st(c, i * c_rs + j * c_cs, sum);
                }
            }
        }
    }
}

template <class T>
int matmul_t(const T* lhs, const int64_t* ls_in, int lrank, const T* rhs, const int64_t* rs_in, int rrank,
             const T* bias, int tl, int tr, int td, T* dst, int64_t* dst_shape, int* dst_rank) {
    // Rank equalisation by left-padding with 1 (ops/matmul/mod.rs:94-102, 413-419)
    if (lrank < 2 || rrank < 2) return 1;
    int rank = std::max(lrank, rrank);
    if (rank > 8) return 1;
    int64_t ls[8], rs[8];
    for (int i = 0; i < rank; ++i) {
        ls[i] = i < rank - lrank ? 1 : ls_in[i - (rank - lrank)];
        rs[i] = i < rank - rrank ? 1 : rs_in[i - (rank - rrank)];
    }
    size_t lstack = 1, rstack = 1, dstack = 1;
    int64_t pre[8];
    for (int i = 0; i < rank - 2; ++i) {
        if (ls[i] != rs[i] && ls[i] != 1 && rs[i] != 1) return 2;
        pre[i] = std::max(ls[i], rs[i]);
        lstack *= ls[i]; rstack *= rs[i]; dstack *= pre[i];
    }
    if (lstack != 1 && rstack != 1 && !(lstack == rstack && rstack == dstack)) return 2;  // mod.rs:117-121
    int64_t lr = ls[rank - 2], lc = ls[rank - 1], rr = rs[rank - 2], rc = rs[rank - 1];
    int64_t m = tl ? lc : lr, kl = tl ? lr : lc;
    int64_t kr = tr ? rc : rr, n = tr ? rr : rc;
    if (kl != kr) return 3;
    for (int i = 0; i < rank - 2; ++i) dst_shape[i] = pre[i];
    dst_shape[rank - 2] = td ? n : m;
    dst_shape[rank - 1] = td ? m : n;
    *dst_rank = rank;
    // op(A)[i,k]: strides in the stored [lr,lc] matrix
    int64_t a_rs = tl ? 1 : lc, a_cs = tl ? lc : 1;
    int64_t b_rs = tr ? 1 : rc, b_cs = tr ? rc : 1;
    int64_t c_rs = td ? 1 : n, c_cs = td ? m : 1;
    // The bias is a vector over the last dimension of dst (broadcast add, gemm.rs bias handling).
    bool bias_on_rows = td != 0;
    gemm_strided<T>(lhs, rhs, bias, dst, dstack, lstack == 1 ? 0 : (size_t)(lr * lc),
                    rstack == 1 ? 0 : (size_t)(rr * rc), (size_t)m, (size_t)n, (size_t)kl, a_rs, a_cs, b_rs,
                    b_cs, c_rs, c_cs, bias_on_rows);
    return 0;
}

// ---------------------------------------------------------------------------------------------
// cpu/binary.rs:78-119 and cpu/unary.rs:46-66
// ---------------------------------------------------------------------------------------------
template <class T>
void binary_t(int op, const T* a, const T* b, T* out, size_t n) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < (int64_t)n; ++i) {
        float x = Num<T>::ld(a, i), y = Num<T>::ld(b, i), r;
        switch (op) {
            case 0: r = x + y; break;
            case 1: r = x - y; break;
            case 2: r = x * y; break;
            default: r = x / y; break;
        }
        Num<T>::st(out, i, r);
    }
}

template <class T>
float unary_scalar(int op, float x) {
    auto R = [](float v) { return Num<T>::r(v); };
    switch (op) {
        case 0: {  // gelu, cpu/unary.rs:46-51: 0.5*x*(1+tanh(0.7978846*x*(1+0.044715*x*x)))
            float c05 = R(0.5f), c1 = R(1.0f), ck = R(0.7978846f), cc = R(0.044715f);
            float inner = R(c1 + R(R(cc * x) * x));
            float arg = R(R(ck * x) * inner);
            return R(R(c05 * x) * R(c1 + R(std::tanh(arg))));
        }
        case 1: return R(std::tanh(x));
        case 2: return R(std::exp(x));
        case 3: return R(std::log(x));
        case 4: return R(std::sin(x));
        case 5: return R(std::cos(x));
        case 6: return std::fabs(x);
        case 7: return R(std::sqrt(x));
        case 8: return std::fmax(x, 0.f);  // relu: x.max(0)
        case 9: return std::floor(x);
        case 10: return std::ceil(x);
        case 11: return -x;
        case 12: return R(x / R(R(1.0f) + R(std::exp(-x))));        // silu, unary.rs:64
        default: return R(R(1.0f) / R(R(1.0f) + R(std::exp(-x))));  // sigmoid, unary.rs:65
    }
}

template <class T>
void unary_t(int op, const T* x, T* out, size_t n) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < (int64_t)n; ++i) Num<T>::st(out, i, unary_scalar<T>(op, Num<T>::ld(x, i)));
}

// ---------------------------------------------------------------------------------------------
// cpu/norm.rs:91-147 (layer_norm) and 185-213 (rms_norm); mean = sequential sum / n (72-89).
// For f16/bf16 the row sums are accumulated in f32 and rounded once (the `half` crate's Sum).
// ---------------------------------------------------------------------------------------------
template <class T>
void layer_norm_t(const T* x, const T* scale, const T* bias, float eps, T* out, size_t rows, size_t N) {
    auto R = [](float v) { return Num<T>::r(v); };
    float nf = R((float)N);
    float e = R(eps);
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < (int64_t)rows; ++r) {
        const size_t o = (size_t)r * N;
        float s = 0.f, s2 = 0.f;
        for (size_t j = 0; j < N; ++j) s += Num<T>::ld(x, o + j);
        for (size_t j = 0; j < N; ++j) { float v = Num<T>::ld(x, o + j); s2 += R(v * v); }
        float mu = R(R(s) / nf);
        float ex2 = R(R(s2) / nf);
        float var = R(ex2 - R(mu * mu));                 // E[x^2] - E[x]^2  (norm.rs:113-121)
        float rstd = R(R(1.0f) / R(std::sqrt(R(var + e))));  // norm.rs:128-130
        for (size_t j = 0; j < N; ++j) {
            float v = R(Num<T>::ld(x, o + j) - mu);
            v = R(v * rstd);
            v = R(v * Num<T>::ld(scale, j));
            if (bias) v = R(v + Num<T>::ld(bias, j));
            Num<T>::st(out, o + j, v);
        }
    }
}

template <class T>
void rms_norm_t(const T* x, const T* scale, float eps, T* out, size_t rows, size_t N) {
    auto R = [](float v) { return Num<T>::r(v); };
    float nf = R((float)N);
    float e = R(eps);
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < (int64_t)rows; ++r) {
        const size_t o = (size_t)r * N;
        float s2 = 0.f;
        for (size_t j = 0; j < N; ++j) { float v = Num<T>::ld(x, o + j); s2 += R(v * v); }
        float ms = R(R(s2) / nf);
        float rstd = R(R(1.0f) / R(std::sqrt(R(ms + e))));
        for (size_t j = 0; j < N; ++j) {
            float v = R(Num<T>::ld(x, o + j) * rstd);
            Num<T>::st(out, o + j, R(v * Num<T>::ld(scale, j)));
        }
    }
}

// cpu/softmax.rs:21-42: exp then divide by the running sum; no max subtraction; chunks of
// shape[dim] over the flat buffer.
template <class T>
void softmax_t(const T* x, T* out, size_t total, size_t N) {
    auto R = [](float v) { return Num<T>::r(v); };
#pragma omp parallel for schedule(static)
    for (int64_t c = 0; c < (int64_t)(total / N); ++c) {
        size_t o = (size_t)c * N;
        float sum = 0.f;
        for (size_t j = 0; j < N; ++j) {
            float e = R(std::exp(Num<T>::ld(x, o + j)));
            Num<T>::st(out, o + j, e);
            sum = R(sum + e);
        }
        for (size_t j = 0; j < N; ++j) Num<T>::st(out, o + j, R(Num<T>::ld(out, o + j) / sum));
    }
}

// cpu/reindex.rs:42-251 — 4-D promoted index remaps
template <class T>
void permute_t(const T* src, const int64_t* sshape, int rank, const int* perm_in, T* dst) {
    int64_t s4[4], d4[4]; int p4[4];
    int pad = 4 - rank;
    for (int i = 0; i < 4; ++i) s4[i] = i < pad ? 1 : sshape[i - pad];
    // Permute::promote: leading identity dims, then the user's perm shifted
    for (int i = 0; i < 4; ++i) p4[i] = i < pad ? i : perm_in[i - pad] + pad;
    for (int i = 0; i < 4; ++i) d4[i] = s4[p4[i]];
    int64_t ss[4] = {s4[1] * s4[2] * s4[3], s4[2] * s4[3], s4[3], 1};
    size_t n = (size_t)(s4[0] * s4[1] * s4[2] * s4[3]);
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < (int64_t)n; ++i) {
        int64_t rem = i, di[4];
        di[0] = rem / (d4[1] * d4[2] * d4[3]); rem -= di[0] * (d4[1] * d4[2] * d4[3]);
        di[1] = rem / (d4[2] * d4[3]); rem -= di[1] * (d4[2] * d4[3]);
        di[2] = rem / d4[3]; di[3] = rem - di[2] * d4[3];
        int64_t si[4];
        for (int k = 0; k < 4; ++k) si[p4[k]] = di[k];   // reindex.rs:72-76
        dst[i] = src[si[0] * ss[0] + si[1] * ss[1] + si[2] * ss[2] + si[3] * ss[3]];
    }
}

template <class T>
void slice_t(const T* src, const int64_t* sshape, int rank, const int64_t* start, const int64_t* stop, T* dst) {
    int64_t sstr[8], dsh[8], ddot[8];
    int64_t acc = 1;
    for (int i = rank - 1; i >= 0; --i) { sstr[i] = acc; acc *= sshape[i]; }
    size_t n = 1;
    for (int i = 0; i < rank; ++i) { dsh[i] = stop[i] - start[i]; n *= (size_t)dsh[i]; }
    acc = 1;
    for (int i = rank - 1; i >= 0; --i) { ddot[i] = acc; acc *= dsh[i]; }
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < (int64_t)n; ++i) {
        int64_t tmp = i, si = 0;
        for (int d = 0; d < rank; ++d) { int64_t c = tmp / ddot[d]; tmp %= ddot[d]; si += (c + start[d]) * sstr[d]; }
        dst[i] = src[si];
    }
}

// numpy-style broadcast (cpu/reindex.rs:189-222 generic_broadcast).  The reference's special
// case for vectors whose length equals dst_shape[0] (reindex.rs:165-173) repeats each element
// instead; it is selectable with `vector_fast_path` so both behaviours can be tested.
template <class T>
void broadcast_t(const T* src, const int64_t* sshape, int srank, const int64_t* dshape, int drank, T* dst,
                 int vector_fast_path) {
    size_t n = numel(dshape, drank);
    size_t sn = numel(sshape, srank);
    int nontrivial = 0; for (int i = 0; i < srank; ++i) nontrivial += sshape[i] != 1;
    if (vector_fast_path && nontrivial == 1 && sshape[0] > 1 && sshape[0] == dshape[0] && srank >= 1) {
        size_t chunk = n / sn;
        for (size_t i = 0; i < sn; ++i) for (size_t j = 0; j < chunk; ++j) dst[i * chunk + j] = src[i];
        return;
    }
    int64_t s4[4], d4[4];
    for (int i = 0; i < 4; ++i) { s4[i] = i < 4 - srank ? 1 : sshape[i - (4 - srank)]; d4[i] = i < 4 - drank ? 1 : dshape[i - (4 - drank)]; }
    int64_t ss[4] = {s4[1] * s4[2] * s4[3], s4[2] * s4[3], s4[3], 1};
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < (int64_t)n; ++i) {
        int64_t rem = i, di[4];
        di[0] = rem / (d4[1] * d4[2] * d4[3]); rem -= di[0] * (d4[1] * d4[2] * d4[3]);
        di[1] = rem / (d4[2] * d4[3]); rem -= di[1] * (d4[2] * d4[3]);
        di[2] = rem / d4[3]; di[3] = rem - di[2] * d4[3];
        int64_t so = 0;
        for (int k = 0; k < 4; ++k) so += (s4[k] != 1 ? di[k] : 0) * ss[k];
        dst[i] = src[so];
    }
}

size_t dt_size(int dt) { return (dt == ORC_F16 || dt == ORC_BF16) ? 2 : 4; }

}  // namespace

// =============================================================================================
// C entry points
// =============================================================================================
extern "C" {

// dtype/blocks.rs:69-82: Q8_0 buffer = [qs: numel B -> 256] [d: numel/32 * fp -> 256]
uint64_t orc_q8_nbytes(uint64_t n, int half_scales) { return align256(n) + align256(n / 32 * (half_scales ? 2 : 4)); }
uint64_t orc_q8_scale_offset(uint64_t n) { return align256(n); }
// ratchet's absmax 4-bit scheme (quant.rs with PACK 8): [q: numel/2 B -> 256] [d -> 256]
uint64_t orc_q4abs_nbytes(uint64_t n, int half_scales) { return align256(n / 2) + align256(n / 32 * (half_scales ? 2 : 4)); }
// dtype/blocks.rs:124-148
uint64_t orc_q4k_nbytes(uint64_t n, int half_scales) { return q4k_segments(n, half_scales ? 2 : 4).total; }
void orc_q4k_offsets(uint64_t n, int half_scales, uint64_t* off4) {
    Q4KSeg s = q4k_segments(n, half_scales ? 2 : 4);
    off4[0] = s.qs; off4[1] = s.scales; off4[2] = s.dmin; off4[3] = s.d;
}

// quant.rs:51-99 — x holds f32 (half_scales=0) or f16 (half_scales=1) values
uint64_t orc_quantize_q8(const void* x, uint64_t n, int half_scales, void* out) {
    return half_scales ? quantize_absmax<f16_t>((const f16_t*)x, n, 4, 127.f, (uint8_t*)out)
                       : quantize_absmax<float>((const float*)x, n, 4, 127.f, (uint8_t*)out);
}
void orc_dequantize_q8(const void* buf, uint64_t n, int half_scales, void* out) {
    if (half_scales) dequantize_absmax<f16_t>((const uint8_t*)buf, n, 4, (f16_t*)out);
    else dequantize_absmax<float>((const uint8_t*)buf, n, 4, (float*)out);
}
uint64_t orc_quantize_q4abs(const void* x, uint64_t n, int half_scales, void* out) {
    return half_scales ? quantize_absmax<f16_t>((const f16_t*)x, n, 8, 7.f, (uint8_t*)out)
                       : quantize_absmax<float>((const float*)x, n, 8, 7.f, (uint8_t*)out);
}
void orc_dequantize_q4abs(const void* buf, uint64_t n, int half_scales, void* out) {
    if (half_scales) dequantize_absmax<f16_t>((const uint8_t*)buf, n, 8, (f16_t*)out);
    else dequantize_absmax<float>((const uint8_t*)buf, n, 8, (float*)out);
}
uint64_t orc_quantize_q4k(const float* x, uint64_t n, int half_scales, void* out) {
    return half_scales ? quantize_q4k<f16_t>(x, n, (uint8_t*)out) : quantize_q4k<float>(x, n, (uint8_t*)out);
}
void orc_dequantize_q4k(const void* buf, uint64_t n, int half_scales, void* out) {
    if (half_scales) dequantize_q4k<f16_t>((const uint8_t*)buf, n, (f16_t*)out);
    else dequantize_q4k<float>((const uint8_t*)buf, n, (float*)out);
}

// Matmul on float tensors. Returns 0 on success; dst_shape/dst_rank receive the result shape.
int orc_matmul(int dt, const void* lhs, const int64_t* lshape, int lrank, const void* rhs, const int64_t* rshape,
               int rrank, const void* bias, int tl, int tr, int td, void* dst, int64_t* dst_shape, int* dst_rank) {
    switch (dt) {
        case ORC_F32: return matmul_t<float>((const float*)lhs, lshape, lrank, (const float*)rhs, rshape, rrank, (const float*)bias, tl, tr, td, (float*)dst, dst_shape, dst_rank);
        case ORC_F16: return matmul_t<f16_t>((const f16_t*)lhs, lshape, lrank, (const f16_t*)rhs, rshape, rrank, (const f16_t*)bias, tl, tr, td, (f16_t*)dst, dst_shape, dst_rank);
        case ORC_BF16: return matmul_t<bf16_t>((const bf16_t*)lhs, lshape, lrank, (const bf16_t*)rhs, rshape, rrank, (const bf16_t*)bias, tl, tr, td, (bf16_t*)dst, dst_shape, dst_rank);
    }
    return 9;
}

// Quantised-weight GEMV without materialising the dequantised matrix (same arithmetic as
// dequantise -> matmul for a [N,K] weight and a [K] activation): used to time the CPU baseline on
// shapes whose f32 copy would not fit comfortably in host memory.
// w_is_half: Q8_0H (scales and dequantised weights in f16) else Q8_0F. act_dt: ORC_F32 / ORC_F16.
void orc_gemv_q8(const void* wbuf, uint64_t N, uint64_t K, int half_scales, const void* x, int act_dt,
                 const void* bias, void* y, uint64_t row_begin, uint64_t row_end) {
    const uint8_t* buf = (const uint8_t*)wbuf;
    const int8_t* qs = (const int8_t*)buf;
    const uint8_t* dseg = buf + align256(N * K);
    std::vector<float> xf(K);
    for (size_t k = 0; k < K; ++k) xf[k] = act_dt == ORC_F16 ? h2f(((const uint16_t*)x)[k]) : ((const float*)x)[k];
#pragma omp parallel for schedule(static)
    for (int64_t r = (int64_t)row_begin; r < (int64_t)row_end; ++r) {
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (size_t kb = 0; kb < K / 32; ++kb) {
            size_t blk = (size_t)r * (K / 32) + kb;
            float d = half_scales ? h2f(((const uint16_t*)dseg)[blk]) : ((const float*)dseg)[blk];
            const int8_t* q = qs + (size_t)r * K + kb * 32;
            const float* xx = &xf[kb * 32];
            for (int j = 0; j < 32; ++j) {
                float w = (float)q[j] * d;
                if (half_scales) w = h2f(f2h(w));
                acc[j & 7] += w * xx[j];
            }
        }
        float sum = ((acc[0] + acc[4]) + (acc[1] + acc[5])) + ((acc[2] + acc[6]) + (acc[3] + acc[7]));
        if (bias) sum += act_dt == ORC_F16 ? h2f(((const uint16_t*)bias)[r]) : ((const float*)bias)[r];
        if (act_dt == ORC_F16) ((uint16_t*)y)[r] = f2h(sum); else ((float*)y)[r] = sum;
    }
}

int orc_binary(int dt, int op, const void* a, const void* b, void* out, uint64_t n) {
    switch (dt) {
        case ORC_F32: binary_t<float>(op, (const float*)a, (const float*)b, (float*)out, n); return 0;
        case ORC_F16: binary_t<f16_t>(op, (const f16_t*)a, (const f16_t*)b, (f16_t*)out, n); return 0;
        case ORC_BF16: binary_t<bf16_t>(op, (const bf16_t*)a, (const bf16_t*)b, (bf16_t*)out, n); return 0;
    }
    return 9;
}

int orc_unary(int dt, int op, const void* x, void* out, uint64_t n) {
    switch (dt) {
        case ORC_F32: unary_t<float>(op, (const float*)x, (float*)out, n); return 0;
        case ORC_F16: unary_t<f16_t>(op, (const f16_t*)x, (f16_t*)out, n); return 0;
        case ORC_BF16: unary_t<bf16_t>(op, (const bf16_t*)x, (bf16_t*)out, n); return 0;
    }
    return 9;
}

// cpu/mod.rs:127-156: f32<->f16, f32<->bf16 convert; f32<->i32/u32 are bit reinterpretations.
int orc_cast(int src_dt, int dst_dt, const void* x, void* out, uint64_t n) {
    if (src_dt == dst_dt) { std::memcpy(out, x, n * dt_size(src_dt)); return 0; }
    if (src_dt == ORC_F32 && dst_dt == ORC_F16) { for (size_t i = 0; i < n; ++i) ((uint16_t*)out)[i] = f2h(((const float*)x)[i]); return 0; }
    if (src_dt == ORC_F32 && dst_dt == ORC_BF16) { for (size_t i = 0; i < n; ++i) ((uint16_t*)out)[i] = f2bf(((const float*)x)[i]); return 0; }
    if (src_dt == ORC_F16 && dst_dt == ORC_F32) { for (size_t i = 0; i < n; ++i) ((float*)out)[i] = h2f(((const uint16_t*)x)[i]); return 0; }
    if (src_dt == ORC_BF16 && dst_dt == ORC_F32) { for (size_t i = 0; i < n; ++i) ((float*)out)[i] = bf2f(((const uint16_t*)x)[i]); return 0; }
    if ((src_dt == ORC_F32 && (dst_dt == ORC_I32 || dst_dt == ORC_U32)) ||
        ((src_dt == ORC_I32 || src_dt == ORC_U32) && dst_dt == ORC_F32)) { std::memcpy(out, x, n * 4); return 0; }
    return 9;
}

int orc_layer_norm(int dt, const void* x, const void* scale, const void* bias, float eps, void* out, uint64_t rows, uint64_t N) {
    switch (dt) {
        case ORC_F32: layer_norm_t<float>((const float*)x, (const float*)scale, (const float*)bias, eps, (float*)out, rows, N); return 0;
        case ORC_F16: layer_norm_t<f16_t>((const f16_t*)x, (const f16_t*)scale, (const f16_t*)bias, eps, (f16_t*)out, rows, N); return 0;
        case ORC_BF16: layer_norm_t<bf16_t>((const bf16_t*)x, (const bf16_t*)scale, (const bf16_t*)bias, eps, (bf16_t*)out, rows, N); return 0;
    }
    return 9;
}
int orc_rms_norm(int dt, const void* x, const void* scale, float eps, void* out, uint64_t rows, uint64_t N) {
    switch (dt) {
        case ORC_F32: rms_norm_t<float>((const float*)x, (const float*)scale, eps, (float*)out, rows, N); return 0;
        case ORC_F16: rms_norm_t<f16_t>((const f16_t*)x, (const f16_t*)scale, eps, (f16_t*)out, rows, N); return 0;
        case ORC_BF16: rms_norm_t<bf16_t>((const bf16_t*)x, (const bf16_t*)scale, eps, (bf16_t*)out, rows, N); return 0;
    }
    return 9;
}
int orc_softmax(int dt, const void* x, void* out, uint64_t total, uint64_t N) {
    switch (dt) {
        case ORC_F32: softmax_t<float>((const float*)x, (float*)out, total, N); return 0;
        case ORC_F16: softmax_t<f16_t>((const f16_t*)x, (f16_t*)out, total, N); return 0;
        case ORC_BF16: softmax_t<bf16_t>((const bf16_t*)x, (bf16_t*)out, total, N); return 0;
    }
    return 9;
}

// cpu/rope.rs:23-143, f32 only: inv_f[i] = exp(-i*ln(base)/half); theta = pos*inv_f;
// out[..half] = x1*cos - x2*sin; out[half..dim] = x1*sin + x2*cos; tail copied.
void orc_rope(const float* x, float* out, uint64_t B, uint64_t H, uint64_t S, uint64_t D, uint64_t dim, float base, uint64_t offset) {
    size_t half = dim / 2;
    std::vector<float> sn(S * half), cs(S * half);
    float lb = std::log(base);
    for (size_t s = 0; s < S; ++s)
        for (size_t i = 0; i < half; ++i) {
            float inv = std::exp(-(float)i * lb / (float)half);
            float th = (float)(s + offset) * inv;
            sn[s * half + i] = std::sin(th);
            cs[s * half + i] = std::cos(th);
        }
#pragma omp parallel for schedule(static)
    for (int64_t bh = 0; bh < (int64_t)(B * H); ++bh)
        for (size_t s = 0; s < S; ++s) {
            const float* xi = x + ((size_t)bh * S + s) * D;
            float* oi = out + ((size_t)bh * S + s) * D;
            for (size_t i = 0; i < half; ++i) {
                float x1 = xi[i], x2 = xi[half + i], c = cs[s * half + i], sv = sn[s * half + i];
                oi[i] = x1 * c - x2 * sv;
                oi[half + i] = x1 * sv + x2 * c;
            }
            for (size_t i = dim; i < D; ++i) oi[i] = xi[i];
        }
}

// cpu/mod.rs:158-211 concat of n inputs along dim; shapes are [n][rank]; esize = bytes/element.
void orc_concat(const void* const* inputs, const int64_t* shapes, int n_inputs, int rank, int dim, void* dst, int esize) {
    int64_t dshape[8];
    for (int i = 0; i < rank; ++i) dshape[i] = shapes[i];
    dshape[dim] = 0;
    for (int k = 0; k < n_inputs; ++k) dshape[dim] += shapes[k * rank + dim];
    size_t block = 1; for (int i = dim + 1; i < rank; ++i) block *= dshape[i];
    size_t dst_s = block * dshape[dim];
    size_t dst_o = 0;
    for (int k = 0; k < n_inputs; ++k) {
        const int64_t* ss = shapes + k * rank;
        size_t a_dim = 1; for (int i = 0; i < dim; ++i) a_dim *= ss[i];
        size_t b_dim = block * ss[dim];
        for (size_t idx = 0; idx < a_dim; ++idx)
            std::memcpy((char*)dst + (idx * dst_s + dst_o) * esize, (const char*)inputs[k] + idx * b_dim * esize, b_dim * esize);
        dst_o += b_dim;
    }
}

// cpu/mod.rs:44-88 index_select on float tables (esize bytes per element).
void orc_index_select(const void* src, const int64_t* sshape, int rank, const int32_t* ids, uint64_t n_ids, int dim, void* dst, int esize) {
    size_t left = 1, right = 1;
    for (int i = 0; i < dim; ++i) left *= sshape[i];
    for (int i = dim + 1; i < rank; ++i) right *= sshape[i];
    size_t src_dim = sshape[dim];
    for (size_t l = 0; l < left; ++l)
        for (size_t i = 0; i < n_ids; ++i)
            std::memcpy((char*)dst + (l * right * n_ids + i * right) * esize,
                        (const char*)src + (l * right * src_dim + (size_t)ids[i] * right) * esize, right * esize);
}

// cpu/mod.rs:90-104 qindex_select: dequantise the whole table, then gather.  Output dtype is the
// table's activation dtype (ops/select.rs:48-60).
void orc_index_select_q8(const void* wbuf, const int64_t* sshape, int half_scales, const int32_t* ids, uint64_t n_ids, int dim, void* dst) {
    size_t n = (size_t)sshape[0] * sshape[1];
    size_t es = half_scales ? 2 : 4;
    std::vector<uint8_t> full(n * es);
    orc_dequantize_q8(wbuf, n, half_scales, full.data());
    orc_index_select(full.data(), sshape, 2, ids, n_ids, dim, dst, (int)es);
}

int orc_permute(int esize, const void* src, const int64_t* sshape, int rank, const int* perm, void* dst) {
    if (esize == 4) permute_t<uint32_t>((const uint32_t*)src, sshape, rank, perm, (uint32_t*)dst);
    else if (esize == 2) permute_t<uint16_t>((const uint16_t*)src, sshape, rank, perm, (uint16_t*)dst);
    else return 9;
    return 0;
}
int orc_slice(int esize, const void* src, const int64_t* sshape, int rank, const int64_t* start, const int64_t* stop, void* dst) {
    if (esize == 4) slice_t<uint32_t>((const uint32_t*)src, sshape, rank, start, stop, (uint32_t*)dst);
    else if (esize == 2) slice_t<uint16_t>((const uint16_t*)src, sshape, rank, start, stop, (uint16_t*)dst);
    else return 9;
    return 0;
}
int orc_broadcast(int esize, const void* src, const int64_t* sshape, int srank, const int64_t* dshape, int drank, void* dst, int vector_fast_path) {
    if (esize == 4) broadcast_t<uint32_t>((const uint32_t*)src, sshape, srank, dshape, drank, (uint32_t*)dst, vector_fast_path);
    else if (esize == 2) broadcast_t<uint16_t>((const uint16_t*)src, sshape, srank, dshape, drank, (uint16_t*)dst, vector_fast_path);
    else return 9;
    return 0;
}

// ops/cache.rs:73-103 (WGSL; no CPU code in the reference): dst = concat(cache[:offset], src)
// along dim and cache[offset:offset+s] = src.  4-D promoted shapes; cache is updated in place.
void orc_cache(void* cache, const int64_t* cshape, const void* src, const int64_t* sshape, int rank, int dim, uint64_t offset, void* dst, int esize) {
    int64_t dshape[4];
    for (int i = 0; i < rank; ++i) dshape[i] = cshape[i];
    dshape[dim] = (int64_t)offset + sshape[dim];
    size_t inner = 1; for (int i = dim + 1; i < rank; ++i) inner *= cshape[i];
    size_t outer = 1; for (int i = 0; i < dim; ++i) outer *= cshape[i];
    size_t cdim = cshape[dim], sdim = sshape[dim], ddim = dshape[dim];
    for (size_t o = 0; o < outer; ++o) {
        char* c = (char*)cache + o * cdim * inner * esize;
        const char* s = (const char*)src + o * sdim * inner * esize;
        char* d = (char*)dst + o * ddim * inner * esize;
        std::memcpy(c + offset * inner * esize, s, sdim * inner * esize);
        std::memcpy(d, c, ddim * inner * esize);
    }
}

// ops/index_write.rs:100-108: write the contiguous src block into dst at an N-D start index.
void orc_index_write(void* dst, const int64_t* dshape, const void* src, const int64_t* sshape, int rank, const int64_t* start, int esize) {
    int64_t dstr[8]; int64_t acc = 1;
    for (int i = rank - 1; i >= 0; --i) { dstr[i] = acc; acc *= dshape[i]; }
    size_t n = numel(sshape, rank);
    for (size_t i = 0; i < n; ++i) {
        size_t rem = i; int64_t off = 0;
        for (int d = rank - 1; d >= 0; --d) { int64_t c = rem % sshape[d]; rem /= sshape[d]; off += (c + start[d]) * dstr[d]; }
        std::memcpy((char*)dst + off * esize, (const char*)src + i * esize, esize);
    }
}

// ops/conv.rs:65-120 (WGSL; no CPU code in the reference): conv1d, kernel size 3, f32.
// x [B,Cin,Lin], w [Cout,Cin,3], b [Cout] -> y [B,Cout,Lout], Lout = (Lin + 2p - 3)/s + 1.
// Per input channel the three taps are accumulated into three separate sums with fma and the
// sums are added at the end with the bias, as the shader does (conv.rs:73-89).
void orc_conv1d_k3(const float* x, const float* w, const float* b, float* y, uint64_t B, uint64_t Cin, uint64_t Lin, uint64_t Cout, uint64_t stride, uint64_t pad) {
    size_t Lout = (Lin + 2 * pad - 3) / stride + 1;
#pragma omp parallel for schedule(static) collapse(2)
    for (int64_t n = 0; n < (int64_t)B; ++n)
        for (int64_t co = 0; co < (int64_t)Cout; ++co) {
            std::vector<float> a0(Lout, 0.f), a1(Lout, 0.f), a2(Lout, 0.f);
            for (size_t ci = 0; ci < Cin; ++ci) {
                const float* xr = x + ((size_t)n * Cin + ci) * Lin;
                const float* wk = w + ((size_t)co * Cin + ci) * 3;
                for (size_t lo = 0; lo < Lout; ++lo) {
                    int64_t i0 = (int64_t)(lo * stride) - (int64_t)pad;
                    if (i0 >= 0 && i0 < (int64_t)Lin) a0[lo] = std::fmaf(xr[i0], wk[0], a0[lo]);
                    if (i0 + 1 >= 0 && i0 + 1 < (int64_t)Lin) a1[lo] = std::fmaf(xr[i0 + 1], wk[1], a1[lo]);
                    if (i0 + 2 >= 0 && i0 + 2 < (int64_t)Lin) a2[lo] = std::fmaf(xr[i0 + 2], wk[2], a2[lo]);
                }
            }
            float* yr = y + ((size_t)n * Cout + co) * Lout;
            for (size_t lo = 0; lo < Lout; ++lo) yr[lo] = a0[lo] + a1[lo] + a2[lo] + (b ? b[co] : 0.f);
        }
}

}  // extern "C"
