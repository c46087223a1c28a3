// Matmul entry point: shape rules, kernel selection, and the general SIMT GEMM.
//
// Shape rules follow Matmul::compute_dst_shape and MatmulSpec::new
// (ratchet-core/src/ops/matmul/mod.rs:74-157,392-466); kernel selection follows
// Matmul::select_kernel (mod.rs:716-748): a vector rhs with an untransposed lhs goes to the GEMV
// family, large half-precision / quantised problems go to the tcgen05 GEMM, everything else to the
// SIMT GEMM below (the stand-in for the reference's 32x32-tile WGSL `gemm`, ops/matmul/gemm.rs).
#include "common.cuh"

rcu_status rcu_gemv_dispatch(rcu_device* dev, int lhs_dt, const void* w, int act_dt, const void* x, const void* bias,
                             void* y, uint64_t N, uint64_t K);
// returns RCU_ERR_UNSUPPORTED when the problem does not fit the tensor-core kernel's constraints
rcu_status rcu_gemm_tc_dispatch(rcu_device* dev, int lhs_dt, const void* w, int act_dt, const void* x, const void* bias,
                                void* y, uint64_t M, uint64_t N, uint64_t K);
bool rcu_gemm_tc_eligible(int lhs_dt, int act_dt, uint64_t M, uint64_t N, uint64_t K);
// f32 Linear on the tensor cores (split-TF32, f32-level accuracy)
rcu_status rcu_gemm_tc_f32_dispatch(rcu_device* dev, const void* w, const void* x, const void* bias, void* y, uint64_t M, uint64_t N,
                                    uint64_t K, uint64_t batches, const void* bias_rows = nullptr);
bool rcu_gemm_tc_f32_eligible(int lhs_dt, int act_dt, uint64_t M, uint64_t N, uint64_t K);
rcu_status rcu_gemm_tc_batched_f16(rcu_device* dev, const void* w, const void* x, void* y, uint64_t M, uint64_t N, uint64_t K, uint64_t batch,
                                   uint64_t pitch_w, uint64_t pitch_x);
rcu_status rcu_copy2d_pitched(rcu_device* dev, const void* src, void* dst, size_t rows, size_t row_bytes, size_t spitch, size_t dpitch);
rcu_status rcu_gemv_q4k_dispatch(rcu_device* dev, int lhs_dt, const void* w, int act_dt, const void* x, const void* bias, void* y,
                                 uint64_t N, uint64_t K);

namespace {

struct MatmulDims {
    uint32_t rank;
    uint64_t dst_shape[RCU_MAX_RANK];
    uint64_t lstack, rstack, dstack;
    uint64_t lr, lc, rr, rc;  // stored matrix dims of lhs and rhs
    uint64_t m, n, k;         // op(lhs) is m x k, op(rhs) is k x n
};

rcu_status matmul_dims(rcu_device* dev, const rcu_tensor* lhs, const rcu_tensor* rhs, int tl, int tr, int td, MatmulDims* d) {
    RCU_REQUIRE(dev, lhs && rhs, "matmul: null tensor");
    RCU_REQUIRE(dev, lhs->rank >= 2 && rhs->rank >= 2 && lhs->rank <= RCU_MAX_RANK && rhs->rank <= RCU_MAX_RANK,
                "MatMul: inputs must be at least 2D (got ranks %u, %u)", lhs->rank, rhs->rank);
    uint32_t rank = lhs->rank > rhs->rank ? lhs->rank : rhs->rank;
    uint64_t ls[RCU_MAX_RANK], rs[RCU_MAX_RANK];
    for (uint32_t i = 0; i < rank; ++i) {
        ls[i] = i < rank - lhs->rank ? 1 : lhs->shape[i - (rank - lhs->rank)];
        rs[i] = i < rank - rhs->rank ? 1 : rhs->shape[i - (rank - rhs->rank)];
    }
    d->rank = rank;
    d->lstack = d->rstack = d->dstack = 1;
    for (uint32_t i = 0; i + 2 < rank; ++i) {
        RCU_REQUIRE(dev, ls[i] == rs[i] || ls[i] == 1 || rs[i] == 1, "Matmul broadcasting: stack dims %llu vs %llu",
                    (unsigned long long)ls[i], (unsigned long long)rs[i]);
        d->dst_shape[i] = ls[i] > rs[i] ? ls[i] : rs[i];
        d->lstack *= ls[i];
        d->rstack *= rs[i];
        d->dstack *= d->dst_shape[i];
    }
    RCU_REQUIRE(dev, d->lstack == 1 || d->rstack == 1 || (d->lstack == d->rstack && d->rstack == d->dstack),
                "Matmul: stacks must be equal or one of them 1");
    d->lr = ls[rank - 2]; d->lc = ls[rank - 1];
    d->rr = rs[rank - 2]; d->rc = rs[rank - 1];
    d->m = tl ? d->lc : d->lr;
    uint64_t kl = tl ? d->lr : d->lc;
    uint64_t kr = tr ? d->rc : d->rr;
    d->n = tr ? d->rr : d->rc;
    RCU_REQUIRE(dev, kl == kr, "Matmul broadcasting: ka != kb: %llu != %llu", (unsigned long long)kl, (unsigned long long)kr);
    d->k = kl;
    d->dst_shape[rank - 2] = td ? d->n : d->m;
    d->dst_shape[rank - 1] = td ? d->m : d->n;
    return RCU_OK;
}

// ------------------------------------------------------------------------------------------------
// Operand loaders for the SIMT GEMM: element (flat index) -> f32, rounded the way the CPU
// dequantiser rounds (quant.rs:118-127: product rounded once in the scale type).
// ------------------------------------------------------------------------------------------------
template <class T> struct LoadPlain {
    const T* p;
    __device__ __forceinline__ float operator()(size_t i) const { return to_f32<T>(p[i]); }
};
template <class ScaleT> struct LoadQ8 {
    const int8_t* q;
    const ScaleT* d;
    __device__ __forceinline__ float operator()(size_t i) const {
        return rnd<ScaleT>((float)q[i] * to_f32<ScaleT>(d[i >> 5]));
    }
};
// GGUF Q4_K in ratchet's segment layout (ops/matmul/quantized.rs:158-266)
template <class FP> struct LoadQ4K {
    const uint8_t* qs;
    const uint8_t* scales;
    const FP* dmin;
    const FP* d;
    __device__ __forceinline__ float operator()(size_t i) const {
        const size_t b = i >> 8;
        const int within = (int)(i & 255);
        const int j = within >> 5, l = within & 31;
        const uint8_t* sc = scales + b * 12;
        uint32_t s, m;
        if (j < 4) {
            s = sc[j] & 63u;
            m = sc[j + 4] & 63u;
        } else {
            s = (sc[j + 4] & 0xFu) | ((uint32_t)(sc[j - 4] >> 6) << 4);
            m = (uint32_t)(sc[j + 4] >> 4) | ((uint32_t)(sc[j] >> 6) << 4);
        }
        const uint8_t byte = qs[b * 128 + (j >> 1) * 32 + l];
        const float qv = (float)((j & 1) ? (byte >> 4) : (byte & 0xF));
        const float delta = rnd<FP>((float)s * to_f32<FP>(d[b]));
        const float mn = rnd<FP>((float)m * to_f32<FP>(dmin[b]));
        return rnd<FP>(fmaf(qv, delta, -mn));
    }
};

constexpr int BM = 64, BN = 64, BK = 16;

template <class ALoad, class BT>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(ALoad A, const BT* __restrict__ B, const BT* __restrict__ bias, BT* __restrict__ C, int M, int N, int K,
                 long long a_rs, long long a_cs, long long a_ss, long long b_rs, long long b_cs, long long b_ss,
                 long long c_rs, long long c_cs, long long c_ss, int bias_on_rows) {
    rcu_kernel_entry();
    __shared__ float As[BK][BM + 4];
    __shared__ float Bs[BK][BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int s = blockIdx.z;
    const size_t a_base = (size_t)s * a_ss;
    const BT* Bp = B + (size_t)s * b_ss;
    BT* Cp = C + (size_t)s * c_ss;
    // choose the load order so that consecutive threads walk the contiguous direction
    const bool a_kfast = a_cs == 1;
    const bool b_kfast = b_rs == 1;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int idx = tid + e * 256;
            int i, k;
            if (a_kfast) { k = idx % BK; i = idx / BK; } else { i = idx % BM; k = idx / BM; }
            const int gm = m0 + i, gk = k0 + k;
            As[k][i] = (gm < M && gk < K) ? A(a_base + (size_t)gm * a_rs + (size_t)gk * a_cs) : 0.f;
            int j, kk;
            if (b_kfast) { kk = idx % BK; j = idx / BK; } else { j = idx % BN; kk = idx / BN; }
            const int gn = n0 + j, gk2 = k0 + kk;
            Bs[kk][j] = (gn < N && gk2 < K) ? to_f32<BT>(Bp[(size_t)gk2 * b_rs + (size_t)gn * b_cs]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            const float4 a = *reinterpret_cast<const float4*>(&As[k][ty * 4]);
            const float4 b = *reinterpret_cast<const float4*>(&Bs[k][tx * 4]);
            const float av[4] = {a.x, a.y, a.z, a.w};
            const float bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gm = m0 + ty * 4 + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx * 4 + j;
            if (gn >= N) continue;
            float v = acc[i][j];
            if (bias) v += to_f32<BT>(bias[bias_on_rows ? gm : gn]);
            Cp[(size_t)gm * c_rs + (size_t)gn * c_cs] = from_f32<BT>(v);
        }
    }
}

template <class ALoad, class BT>
rcu_status launch_simt(rcu_device* dev, ALoad A, const void* B, const void* bias, void* C, const MatmulDims& d, int tl, int tr,
                       int td) {
    const long long a_rs = tl ? 1 : (long long)d.lc, a_cs = tl ? (long long)d.lc : 1;
    const long long b_rs = tr ? 1 : (long long)d.rc, b_cs = tr ? (long long)d.rc : 1;
    const long long c_rs = td ? 1 : (long long)d.n, c_cs = td ? (long long)d.m : 1;
    const long long a_ss = d.lstack == 1 ? 0 : (long long)(d.lr * d.lc);
    const long long b_ss = d.rstack == 1 ? 0 : (long long)(d.rr * d.rc);
    const long long c_ss = (long long)(d.m * d.n);
    RCU_REQUIRE(dev, d.dstack <= 65535, "matmul: more than 65535 stacks");
    dim3 grid((unsigned)((d.n + BN - 1) / BN), (unsigned)((d.m + BM - 1) / BM), (unsigned)d.dstack);
    RCU_REQUIRE(dev, grid.y <= 65535, "matmul: M too large for the SIMT kernel");
    rcu_launch(dev, gemm_simt_kernel<ALoad, BT>, grid, 256, 0, A, (const BT*)B, (const BT*)bias, (BT*)C, (int)d.m, (int)d.n,
                                                               (int)d.k, a_rs, a_cs, a_ss, b_rs, b_cs, b_ss, c_rs, c_cs,
                                                               c_ss, td ? 1 : 0);
    RCU_LAUNCH_CHECK(dev);
    return RCU_OK;
}

bool dtype_pair_ok(int l, int r) {
    return (l == RCU_F32 && r == RCU_F32) || (l == RCU_F16 && r == RCU_F16) || (l == RCU_BF16 && r == RCU_BF16) ||
           (l == RCU_Q8_0F && r == RCU_F32) || (l == RCU_Q8_0H && r == RCU_F16) || (l == RCU_Q8_0F && r == RCU_F16) ||
           (l == RCU_Q4_KF && r == RCU_F32) || (l == RCU_Q4_KH && r == RCU_F16);
}

}  // namespace

extern "C" {

rcu_status rcu_matmul_dst_shape(const rcu_tensor* lhs, const rcu_tensor* rhs, int tl, int tr, int td, rcu_tensor* dst) {
    if (!dst) return RCU_ERR_INVALID_ARG;
    MatmulDims d;
    rcu_status st = matmul_dims(nullptr, lhs, rhs, tl, tr, td, &d);
    if (st != RCU_OK) return st;
    dst->rank = d.rank;
    for (uint32_t i = 0; i < d.rank; ++i) dst->shape[i] = d.dst_shape[i];
    dst->dt = rhs->dt;  // compute_view: dst dtype = rhs dtype (mod.rs:484-495)
    return RCU_OK;
}

rcu_status rcu_matmul(rcu_device* dev, const rcu_tensor* lhs, const rcu_tensor* rhs, const rcu_tensor* bias, int tl, int tr,
                      int td, rcu_tensor* dst) {
    if (!dev) return RCU_ERR_INVALID_ARG;
    RCU_REQUIRE(dev, t_valid(lhs) && t_valid(rhs) && t_valid(dst), "matmul: invalid tensor descriptor");
    if (!dtype_pair_ok(lhs->dt, rhs->dt)) return rcu_fail(dev, RCU_ERR_INVALID_ARG, "DType mismatch: lhs: %d, rhs: %d", lhs->dt, rhs->dt);
    RCU_REQUIRE(dev, !bias || bias->dt == rhs->dt, "DType mismatch: bias: %d, rhs: %d", bias ? bias->dt : -1, rhs->dt);
    RCU_REQUIRE(dev, dst->dt == rhs->dt, "matmul: dst dtype must equal rhs dtype");
    MatmulDims d;
    rcu_status st = matmul_dims(dev, lhs, rhs, tl, tr, td, &d);
    if (st != RCU_OK) return st;
    RCU_REQUIRE(dev, t_numel(dst) == d.dstack * d.m * d.n, "matmul: dst holds %llu elements, expected %llu",
                (unsigned long long)t_numel(dst), (unsigned long long)(d.dstack * d.m * d.n));
    const uint64_t bias_len = td ? d.m : d.n;
    RCU_REQUIRE(dev, !bias || t_numel(bias) == bias_len, "matmul: bias must be a vector over dst's last dimension");
    DevGuard g(dev->ordinal);
    const void* bptr = bias ? bias->data : nullptr;

    // GEMV: rhs squeezes to a vector and lhs is not transposed (mod.rs:717-718)
    const bool rhs_vector = d.rstack == 1 && d.n == 1;
    if (rhs_vector && !tl && d.lstack == 1 && d.dstack == 1 && lhs->dt != RCU_BF16) {
        if (dt_is_q4k(lhs->dt)) return rcu_gemv_q4k_dispatch(dev, lhs->dt, lhs->data, rhs->dt, rhs->data, bptr, dst->data, d.m, d.k);
        return rcu_gemv_dispatch(dev, lhs->dt, lhs->data, rhs->dt, rhs->data, bptr, dst->data, d.m, d.k);
    }
    // Linear convention W[N,K] . x[M,K]^T -> [M,N]: tensor-core path when the shape qualifies
    if (!tl && tr && td && d.lstack == 1 && rcu_gemm_tc_eligible(lhs->dt, rhs->dt, d.rstack * d.n, d.m, d.k)) {
        st = rcu_gemm_tc_dispatch(dev, lhs->dt, lhs->data, rhs->dt, rhs->data, bptr, dst->data, d.rstack * d.n, d.m, d.k);
        if (st != RCU_ERR_UNSUPPORTED) return st;
    }
    if (!tl && tr && td && d.lstack == 1 && rcu_gemm_tc_f32_eligible(lhs->dt, rhs->dt, d.rstack * d.n, d.m, d.k)) {
        st = rcu_gemm_tc_f32_dispatch(dev, lhs->data, rhs->data, bptr, dst->data, d.rstack * d.n, d.m, d.k, 1);
        if (st != RCU_ERR_UNSUPPORTED) return st;
    }
    // Quantised weights with f32 activations (Q8_0F / Q4_KF Linear, the quantised Whisper graphs): the
    // weights are dequantised once into pooled scratch (bit-exact, as the CPU path does for every
    // quantised op) and the product runs on the f32 tensor-core kernel.
    if (!tl && tr && td && d.lstack == 1 && (lhs->dt == RCU_Q8_0F || lhs->dt == RCU_Q4_KF) && rhs->dt == RCU_F32 &&
        rcu_gemm_tc_f32_eligible(RCU_F32, RCU_F32, d.rstack * d.n, d.m, d.k)) {
        void* wf = nullptr;
        st = rcu_alloc(dev, d.m * d.k * 4, &wf);
        if (st != RCU_OK) return st;
        rcu_tensor wsrc{lhs->dt, 2, {d.m, d.k, 1, 1}, lhs->data};
        rcu_tensor wdst{RCU_F32, 2, {d.m, d.k, 1, 1}, wf};
        st = rcu_dequantize(dev, &wsrc, &wdst);
        if (st == RCU_OK) st = rcu_gemm_tc_f32_dispatch(dev, wf, rhs->data, bptr, dst->data, d.rstack * d.n, d.m, d.k, 1);
        rcu_free(dev, wf);      // the pool reuses blocks in stream order
        if (st != RCU_ERR_UNSUPPORTED) return st;
    }
    // Batched f32 products of the attention kind, A[b, M, K] . B[b, K, N] (or B given as [b, N, K] with
    // trans_rhs): the tensor-core kernel wants both operands K-major, so an untransposed B is transposed
    // into pooled scratch first (it is the small operand of these products).
    if (!tl && !td && !bias && d.lstack == d.rstack && d.dstack == d.lstack && rcu_gemm_tc_f32_eligible(lhs->dt, rhs->dt, d.m, d.n, d.k)) {
        const void* wptr = rhs->data;
        void* scratch = nullptr;
        st = RCU_OK;
        if (!tr) {
            st = rcu_alloc(dev, d.rstack * d.k * d.n * 4, &scratch);
            if (st != RCU_OK) return st;
            rcu_tensor src{RCU_F32, 3, {d.rstack, d.k, d.n, 1}, rhs->data};
            rcu_tensor tdst{RCU_F32, 3, {d.rstack, d.n, d.k, 1}, scratch};
            const uint32_t perm[3] = {0, 2, 1};
            st = rcu_permute(dev, &src, perm, &tdst);
            wptr = scratch;
        }
        if (st == RCU_OK) st = rcu_gemm_tc_f32_dispatch(dev, wptr, lhs->data, nullptr, dst->data, d.m, d.n, d.k, d.lstack);
        if (scratch) rcu_free(dev, scratch);     // the pool reuses blocks in stream order
        if (st != RCU_ERR_UNSUPPORTED) return st;
    }
    // The same products in f16 (the attention of an f16 model): A[b, M, K] . B[b, K, N] on the f16 tensor-core
    // kernel, one problem per blockIdx.z.  Tensor maps need row pitches of whole 16 bytes: an operand whose K
    // is not a multiple of 8 (Whisper's 1500 positions) is copied into pooled scratch with padded rows (the
    // kernel never reads the padding: the maps give the true K and fill beyond it with zeros), and an
    // untransposed B is transposed first.
    if (!tl && !td && !bias && lhs->dt == RCU_F16 && rhs->dt == RCU_F16 && d.lstack == d.rstack && d.dstack == d.lstack &&
        d.m >= 128 && d.n >= 64 && d.k >= 64 && d.n % 4 == 0 && d.m * d.n * d.k * d.lstack >= (1ull << 24)) {
        const uint64_t b = d.lstack, kp = (d.k + 7) & ~7ull;
        void* scratch[3] = {nullptr, nullptr, nullptr};
        const void* aptr = lhs->data;
        const void* wptr = rhs->data;
        st = RCU_OK;
        if (!tr) {          // B [b, K, N] -> [b, N, K]
            st = rcu_alloc(dev, b * d.k * d.n * 2, &scratch[0]);
            if (st == RCU_OK) {
                rcu_tensor src{RCU_F16, 3, {b, d.k, d.n, 1}, rhs->data};
                rcu_tensor tdst{RCU_F16, 3, {b, d.n, d.k, 1}, scratch[0]};
                const uint32_t perm[3] = {0, 2, 1};
                st = rcu_permute(dev, &src, perm, &tdst);
                wptr = scratch[0];
            }
        }
        if (st == RCU_OK && kp != d.k) {
            st = rcu_alloc(dev, b * d.n * kp * 2, &scratch[1]);
            if (st == RCU_OK) st = rcu_copy2d_pitched(dev, wptr, scratch[1], b * d.n, d.k * 2, d.k * 2, kp * 2);
            wptr = scratch[1];
            if (st == RCU_OK) st = rcu_alloc(dev, b * d.m * kp * 2, &scratch[2]);
            if (st == RCU_OK) st = rcu_copy2d_pitched(dev, aptr, scratch[2], b * d.m, d.k * 2, d.k * 2, kp * 2);
            aptr = scratch[2];
        }
        if (st == RCU_OK) st = rcu_gemm_tc_batched_f16(dev, wptr, aptr, dst->data, d.m, d.n, d.k, b, kp, kp);
        for (void* s : scratch)
            if (s) rcu_free(dev, s);     // the pool reuses blocks in stream order
        if (st != RCU_ERR_UNSUPPORTED) return st;
    }
    const uint64_t numel = t_numel(lhs);
    uint64_t off[4];
    rcu_dtype_segments(lhs->dt, numel, off);
    const char* base = (const char*)lhs->data;
    switch (lhs->dt) {
        case RCU_F32: return launch_simt<LoadPlain<float>, float>(dev, LoadPlain<float>{(const float*)base}, rhs->data, bptr, dst->data, d, tl, tr, td);
        case RCU_F16: return launch_simt<LoadPlain<__half>, __half>(dev, LoadPlain<__half>{(const __half*)base}, rhs->data, bptr, dst->data, d, tl, tr, td);
        case RCU_BF16: return launch_simt<LoadPlain<__nv_bfloat16>, __nv_bfloat16>(dev, LoadPlain<__nv_bfloat16>{(const __nv_bfloat16*)base}, rhs->data, bptr, dst->data, d, tl, tr, td);
        case RCU_Q8_0F:
            if (rhs->dt == RCU_F32)
                return launch_simt<LoadQ8<float>, float>(dev, LoadQ8<float>{(const int8_t*)base, (const float*)(base + off[1])}, rhs->data, bptr, dst->data, d, tl, tr, td);
            return launch_simt<LoadQ8<float>, __half>(dev, LoadQ8<float>{(const int8_t*)base, (const float*)(base + off[1])}, rhs->data, bptr, dst->data, d, tl, tr, td);
        case RCU_Q8_0H: return launch_simt<LoadQ8<__half>, __half>(dev, LoadQ8<__half>{(const int8_t*)base, (const __half*)(base + off[1])}, rhs->data, bptr, dst->data, d, tl, tr, td);
        case RCU_Q4_KF:
            return launch_simt<LoadQ4K<float>, float>(dev, LoadQ4K<float>{(const uint8_t*)base, (const uint8_t*)base + off[1], (const float*)(base + off[2]), (const float*)(base + off[3])}, rhs->data, bptr, dst->data, d, tl, tr, td);
        case RCU_Q4_KH:
            return launch_simt<LoadQ4K<__half>, __half>(dev, LoadQ4K<__half>{(const uint8_t*)base, (const uint8_t*)base + off[1], (const __half*)(base + off[2]), (const __half*)(base + off[3])}, rhs->data, bptr, dst->data, d, tl, tr, td);
    }
    return rcu_fail(dev, RCU_ERR_UNSUPPORTED, "matmul: no kernel for lhs dtype %d", lhs->dt);
}

}  // extern "C"
