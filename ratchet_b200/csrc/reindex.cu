// Data-movement ops: Permute / Slice / Broadcast, Concat, IndexSelect (plain and Q8_0 dequantising),
// Cache (KV append) and IndexWrite.  All are exact copies (bit-identical with the CPU device).
//
// Stand in for ratchet-core's reindex WGSL kernels (ops/reindex/mod.rs:48-124), concat
// (ops/concat.rs:49-108), index_select (ops/select.rs:122-184), cache (ops/cache.rs:51-105) and
// index_write (ops/index_write.rs:79-111); semantics follow cpu/reindex.rs:42-251 and
// cpu/mod.rs:44-211.
//
// Slab-shaped moves (concat inputs, cache rows, single-axis slices, index_write blocks, row
// gathers) go through one pitched-copy kernel that moves 16 bytes per thread whenever pitches and
// pointers allow it; the generic 4-D remap handles everything else one element per thread.
#include "common.cuh"

namespace {

inline int copy_grid(const rcu_device* dev, size_t work) {
    const size_t blocks = (work + 255) / 256;
    const size_t cap = (size_t)dev->sm_count * 8;
    return (int)(blocks < 1 ? 1 : (blocks < cap ? blocks : cap));
}

// rows x row_bytes, source/destination row pitches in bytes. U = bytes per thread step.
// I is the index type of the flat unit counter: 32-bit division whenever the unit count allows it.
template <class U, class I>
__global__ void __launch_bounds__(256)
copy2d_kernel(const char* __restrict__ src, char* __restrict__ dst, size_t rows, size_t row_units, size_t spitch, size_t dpitch) {
    rcu_kernel_entry();
    const size_t total = rows * row_units;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    const I ru = (I)row_units;
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (; i + stride < total; i += 2 * stride) {      // two units in flight per thread
        const I r0 = (I)i / ru, c0 = (I)i - r0 * ru;
        const I r1 = (I)(i + stride) / ru, c1 = (I)(i + stride) - r1 * ru;
        const U u0 = *reinterpret_cast<const U*>(src + (size_t)r0 * spitch + (size_t)c0 * sizeof(U));
        const U u1 = *reinterpret_cast<const U*>(src + (size_t)r1 * spitch + (size_t)c1 * sizeof(U));
        *reinterpret_cast<U*>(dst + (size_t)r0 * dpitch + (size_t)c0 * sizeof(U)) = u0;
        *reinterpret_cast<U*>(dst + (size_t)r1 * dpitch + (size_t)c1 * sizeof(U)) = u1;
    }
    if (i < total) {
        const I r = (I)i / ru, c = (I)i - r * ru;
        *reinterpret_cast<U*>(dst + (size_t)r * dpitch + (size_t)c * sizeof(U)) = *reinterpret_cast<const U*>(src + (size_t)r * spitch + (size_t)c * sizeof(U));
    }
}

template <class U>
void launch_copy2d(rcu_device* dev, const char* s, char* d, size_t rows, size_t row_units, size_t spitch, size_t dpitch) {
    const size_t total = rows * row_units;
    const int grid = copy_grid(dev, total / 2 + 1);
    if (total <= 0xffffffffull) rcu_launch(dev, copy2d_kernel<U, uint32_t>, grid, 256, 0, s, d, rows, row_units, spitch, dpitch);
    else rcu_launch(dev, copy2d_kernel<U, uint64_t>, grid, 256, 0, s, d, rows, row_units, spitch, dpitch);
}

rcu_status copy2d(rcu_device* dev, const void* src, void* dst, size_t rows, size_t row_bytes, size_t spitch, size_t dpitch) {
    if (rows == 0 || row_bytes == 0) return RCU_OK;
    const uintptr_t bits = reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst) | row_bytes | spitch | dpitch;
    const char* s = (const char*)src;
    char* d = (char*)dst;
    if ((bits & 15) == 0) launch_copy2d<uint4>(dev, s, d, rows, row_bytes / 16, spitch, dpitch);
    else if ((bits & 7) == 0) launch_copy2d<uint2>(dev, s, d, rows, row_bytes / 8, spitch, dpitch);
    else if ((bits & 3) == 0) launch_copy2d<uint32_t>(dev, s, d, rows, row_bytes / 4, spitch, dpitch);
    else if ((bits & 1) == 0) launch_copy2d<uint16_t>(dev, s, d, rows, row_bytes / 2, spitch, dpitch);
    else launch_copy2d<uint8_t>(dev, s, d, rows, row_bytes, spitch, dpitch);
    RCU_LAUNCH_CHECK(dev);
    return RCU_OK;
}

// dst[i0,i1,i2,i3] = src[off + i0*s0 + i1*s1 + i2*s2 + i3*s3]  (element strides; 0 = broadcast)
struct Remap4 {
    uint32_t d[4];
    long long s[4];
    long long off;
};

// U is the unit a thread moves (strides, extents and the offset are in units); I the index type.
template <class U, class I>
__global__ void __launch_bounds__(256) remap4_kernel(const U* __restrict__ src, U* __restrict__ dst, size_t n, Remap4 p) {
    rcu_kernel_entry();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        I r = (I)i;
        const uint32_t i3 = (uint32_t)(r % p.d[3]); r /= p.d[3];
        const uint32_t i2 = (uint32_t)(r % p.d[2]); r /= p.d[2];
        const uint32_t i1 = (uint32_t)(r % p.d[1]); r /= p.d[1];
        const uint32_t i0 = (uint32_t)r;
        dst[i] = src[p.off + i0 * p.s[0] + i1 * p.s[1] + i2 * p.s[2] + i3 * p.s[3]];
    }
}

// Innermost axis broadcast (source stride 0): one element read, V copies stored as one vector.
template <class E, int V, class I>
__global__ void __launch_bounds__(256) remap4_fill_kernel(const E* __restrict__ src, E* __restrict__ dst, size_t nvec, Remap4 p) {
    rcu_kernel_entry();
    struct alignas(sizeof(E) * V) VT { E v[V]; };
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    const uint32_t row_units = p.d[3] / V;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
        I r = (I)i;
        r /= row_units;
        const uint32_t i2 = (uint32_t)(r % p.d[2]); r /= p.d[2];
        const uint32_t i1 = (uint32_t)(r % p.d[1]); r /= p.d[1];
        const uint32_t i0 = (uint32_t)r;
        const E e = src[p.off + i0 * p.s[0] + i1 * p.s[1] + i2 * p.s[2]];
        VT o;
#pragma unroll
        for (int j = 0; j < V; ++j) o.v[j] = e;
        reinterpret_cast<VT*>(dst)[i] = o;
    }
}

// 32x32 shared-memory tile transpose of the two innermost axes of a [batch, R, C] view:
// dst[b, c, r] = src[b, r, c].  Used when a permutation swaps the last two (collapsed) axes.
template <class E>
__global__ void __launch_bounds__(256) transpose_kernel(const E* __restrict__ src, E* __restrict__ dst, int R, int C) {
    rcu_kernel_entry();
    __shared__ E tile[32][33];
    const size_t b = blockIdx.z;
    const E* s = src + b * (size_t)R * C;
    E* d = dst + b * (size_t)R * C;
    const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    for (int j = ty; j < 32; j += 8)
        if (r0 + j < R && c0 + tx < C) tile[j][tx] = s[(size_t)(r0 + j) * C + c0 + tx];
    __syncthreads();
    for (int j = ty; j < 32; j += 8)
        if (c0 + j < C && r0 + tx < R) d[(size_t)(c0 + j) * R + r0 + tx] = tile[tx][j];
}

// 64x64 tile transpose moving element pairs: global loads take two elements of a source row, global
// stores two elements of a destination row; eight pair loads are in flight per thread.  R and C even,
// both pointers aligned to a pair.
template <class E, class P>
__global__ void __launch_bounds__(256) transpose_pair_kernel(const E* __restrict__ src, E* __restrict__ dst, int R, int C) {
    rcu_kernel_entry();
    constexpr int PITCH = sizeof(E) == 2 ? 66 : 65;
    __shared__ E tile[64 * PITCH];
    const size_t b = blockIdx.z;
    const E* s = src + b * (size_t)R * C;
    E* d = dst + b * (size_t)R * C;
    const int c0 = blockIdx.x * 64, r0 = blockIdx.y * 64;
    P in[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const int q = threadIdx.x + k * 256, row = q >> 5, pc = q & 31;
        if (r0 + row < R && c0 + 2 * pc < C) in[k] = *reinterpret_cast<const P*>(s + (size_t)(r0 + row) * C + c0 + 2 * pc);
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const int q = threadIdx.x + k * 256, row = q >> 5, pc = q & 31;
        const E* e = reinterpret_cast<const E*>(&in[k]);
        tile[row * PITCH + 2 * pc] = e[0];
        tile[row * PITCH + 2 * pc + 1] = e[1];
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const int q = threadIdx.x + k * 256, oc = q >> 5, pr = q & 31;
        if (c0 + oc < C && r0 + 2 * pr < R) {
            P o;
            E* e = reinterpret_cast<E*>(&o);
            e[0] = tile[(2 * pr) * PITCH + oc];
            e[1] = tile[(2 * pr + 1) * PITCH + oc];
            *reinterpret_cast<P*>(d + (size_t)(c0 + oc) * R + r0 + 2 * pr) = o;
        }
    }
}

template <class U>
void launch_remap(rcu_device* dev, const void* src, void* dst, size_t n, const Remap4& p) {
    if (n <= 0xffffffffull) rcu_launch(dev, remap4_kernel<U, uint32_t>, copy_grid(dev, n), 256, 0, (const U*)src, (U*)dst, n, p);
    else rcu_launch(dev, remap4_kernel<U, uint64_t>, copy_grid(dev, n), 256, 0, (const U*)src, (U*)dst, n, p);
}

template <class E>
void launch_fill(rcu_device* dev, const void* src, void* dst, size_t nvec, const Remap4& p) {
    constexpr int V = 16 / sizeof(E);
    if (nvec <= 0xffffffffull) rcu_launch(dev, remap4_fill_kernel<E, V, uint32_t>, copy_grid(dev, nvec), 256, 0, (const E*)src, (E*)dst, nvec, p);
    else rcu_launch(dev, remap4_fill_kernel<E, V, uint64_t>, copy_grid(dev, nvec), 256, 0, (const E*)src, (E*)dst, nvec, p);
}

// `p` is in elements of `es` bytes.  When the innermost destination axis is contiguous in the source
// the move is re-expressed in the widest unit (16, 8 or 4 bytes) that divides the innermost extent,
// every outer stride, the offset and both pointers; a broadcast innermost axis stores whole vectors
// of one repeated element; anything else moves one element per thread.
rcu_status remap(rcu_device* dev, int dt, const void* src, void* dst, size_t n, const Remap4& p) {
    if (n == 0) return RCU_OK;
    const size_t es = dt_esize(dt);
    const uintptr_t ptrs = reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst);
    if (p.s[3] == 1 || p.d[3] == 1) {
        for (size_t ub = 16; ub > es; ub >>= 1) {
            const size_t v = ub / es;
            bool ok = (ptrs & (ub - 1)) == 0 && p.d[3] % v == 0 && p.off % (long long)v == 0 && p.d[3] > 1;
            for (int i = 0; i < 3 && ok; ++i) ok = p.s[i] % (long long)v == 0;
            if (!ok) continue;
            Remap4 q = p;
            q.d[3] = (uint32_t)(p.d[3] / v);
            q.off = p.off / (long long)v;
            for (int i = 0; i < 3; ++i) q.s[i] = p.s[i] / (long long)v;
            q.s[3] = 1;
            const size_t nu = n / v;
            if (ub == 16) launch_remap<uint4>(dev, src, dst, nu, q);
            else if (ub == 8) launch_remap<uint2>(dev, src, dst, nu, q);
            else launch_remap<uint32_t>(dev, src, dst, nu, q);
            RCU_LAUNCH_CHECK(dev);
            return RCU_OK;
        }
    } else if (p.s[3] == 0 && p.d[3] % (16 / es) == 0 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
        const size_t nvec = n / (16 / es);
        if (es == 2) launch_fill<uint16_t>(dev, src, dst, nvec, p);
        else launch_fill<uint32_t>(dev, src, dst, nvec, p);
        RCU_LAUNCH_CHECK(dev);
        return RCU_OK;
    }
    if (es == 2) launch_remap<uint16_t>(dev, src, dst, n, p);
    else launch_remap<uint32_t>(dev, src, dst, n, p);
    RCU_LAUNCH_CHECK(dev);
    return RCU_OK;
}

inline bool movable_dtype(int dt) { return dt == RCU_F32 || dt == RCU_F16 || dt == RCU_BF16 || dt == RCU_I32 || dt == RCU_U32; }

// ---------------------------------------------------------------------------------- gather
template <class E>
__global__ void __launch_bounds__(256)
gather_kernel(const E* __restrict__ src, const int32_t* __restrict__ ids, E* __restrict__ dst, size_t left, size_t n_ids,
              size_t right, size_t src_dim, int* status) {
    rcu_kernel_entry();
    const size_t total = left * n_ids * right;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const size_t r = i % right;
        const size_t t = i / right;
        const size_t k = t % n_ids, l = t / n_ids;
        long long id = ids[k];
        if (id < 0 || (size_t)id >= src_dim) {   // the WGSL clamps (ops/select.rs:157); also report it
            atomicOr(status, RCU_DEVFLAG_BOUNDS);
            id = id < 0 ? 0 : (long long)src_dim - 1;
        }
        dst[i] = src[(l * src_dim + (size_t)id) * right + r];
    }
}

// Q8_0 table [V, D]: out[..] = fp(q * d), four values per thread (one packed u32), ops/select.rs:144-164
template <class ScaleT>
__global__ void __launch_bounds__(256)
gather_q8_kernel(const uint32_t* __restrict__ q, const ScaleT* __restrict__ d, const int32_t* __restrict__ ids,
                 ScaleT* __restrict__ dst, size_t left, size_t n_ids, size_t right, size_t src_dim, int* status) {
    rcu_kernel_entry();
    // element (l, id, r) of the table has flat index (l*src_dim + id)*right + r; right % 4 == 0 is required
    const size_t right4 = right >> 2;
    const size_t total = left * n_ids * right4;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const size_t r4 = i % right4;
        const size_t t = i / right4;
        const size_t k = t % n_ids, l = t / n_ids;
        long long id = ids[k];
        if (id < 0 || (size_t)id >= src_dim) {
            atomicOr(status, RCU_DEVFLAG_BOUNDS);
            id = id < 0 ? 0 : (long long)src_dim - 1;
        }
        const size_t flat = (l * src_dim + (size_t)id) * right + r4 * 4;
        const uint32_t packed = q[flat >> 2];
        const float sc = to_f32<ScaleT>(d[flat >> 5]);
        ScaleT* o = dst + (l * n_ids + k) * right + r4 * 4;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int v = (int)(packed << (8 * (3 - j))) >> 24;   // quant.rs:121-125
            o[j] = from_f32<ScaleT>((float)v * sc);
        }
    }
}

// Row gather (dim 0 of a 2-D table): dst row k = src row ids[k], moved in units of U.
template <class U, class I>
__global__ void __launch_bounds__(256)
gather_rows_kernel(const U* __restrict__ src, const int32_t* __restrict__ ids, U* __restrict__ dst, size_t n_ids, size_t row_units,
                   size_t src_dim, int* status) {
    rcu_kernel_entry();
    const size_t total = n_ids * row_units;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    const I ru = (I)row_units;
    auto row_of = [&](I k) -> size_t {
        long long id = ids[k];
        if (id < 0 || (size_t)id >= src_dim) {   // the WGSL clamps (ops/select.rs:157); also report it
            atomicOr(status, RCU_DEVFLAG_BOUNDS);
            id = id < 0 ? 0 : (long long)src_dim - 1;
        }
        return (size_t)id;
    };
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (; i + stride < total; i += 2 * stride) {
        const I k0 = (I)i / ru, c0 = (I)i - k0 * ru;
        const I k1 = (I)(i + stride) / ru, c1 = (I)(i + stride) - k1 * ru;
        const U u0 = src[row_of(k0) * row_units + c0];
        const U u1 = src[row_of(k1) * row_units + c1];
        dst[i] = u0;
        dst[i + stride] = u1;
    }
    if (i < total) {
        const I k = (I)i / ru, c = (I)i - k * ru;
        dst[i] = src[row_of(k) * row_units + c];
    }
}

template <class ScaleT> struct Q8Out;
template <> struct Q8Out<__half> {
    __device__ static __forceinline__ void store8(__half* dst, const float* v) {
        __align__(16) __half h[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) h[i] = __float2half_rn(v[i]);
        *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(h);
    }
};
template <> struct Q8Out<float> {
    __device__ static __forceinline__ void store8(float* dst, const float* v) {
        reinterpret_cast<float4*>(dst)[0] = make_float4(v[0], v[1], v[2], v[3]);
        reinterpret_cast<float4*>(dst)[1] = make_float4(v[4], v[5], v[6], v[7]);
    }
};

// Q8_0 row gather, 16 values per thread: one 16-byte load of packed int8 (half a 32-block, one
// scale), 16-byte stores.  Row length % 16 == 0.
template <class ScaleT>
__global__ void __launch_bounds__(256)
gather_q8_rows16_kernel(const uint4* __restrict__ q, const ScaleT* __restrict__ d, const int32_t* __restrict__ ids,
                        ScaleT* __restrict__ dst, size_t n_ids, uint32_t row16, size_t src_dim, int* status) {
    rcu_kernel_entry();
    const size_t total = n_ids * row16;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const size_t k = i / row16;
        const uint32_t c = (uint32_t)(i - k * row16);
        long long id = ids[k];
        if (id < 0 || (size_t)id >= src_dim) {
            atomicOr(status, RCU_DEVFLAG_BOUNDS);
            id = id < 0 ? 0 : (long long)src_dim - 1;
        }
        const size_t unit = (size_t)id * row16 + c;           // 16-value unit in the table
        const uint4 w = q[unit];
        const float sc = to_f32<ScaleT>(d[unit >> 1]);
        const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
        float v[16];
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
            for (int j = 0; j < 4; ++j) v[a * 4 + j] = rnd<ScaleT>((float)((int)(ws[a] << (8 * (3 - j))) >> 24) * sc);   // quant.rs:121-125
        Q8Out<ScaleT>::store8(dst + i * 16, v);
        Q8Out<ScaleT>::store8(dst + i * 16 + 8, v + 8);
    }
}

}  // namespace

// rows of row_bytes each, source and destination pitches in bytes (used by the batched f16 matmul to give
// rows a pitch the tensor maps accept)
rcu_status rcu_copy2d_pitched(rcu_device* dev, const void* src, void* dst, size_t rows, size_t row_bytes, size_t spitch, size_t dpitch) {
    return copy2d(dev, src, dst, rows, row_bytes, spitch, dpitch);
}


extern "C" {

rcu_status rcu_permute(rcu_device* dev, const rcu_tensor* src, const uint32_t* perm, rcu_tensor* dst) {
    if (!dev) return RCU_ERR_INVALID_ARG;
    RCU_REQUIRE(dev, t_valid(src) && t_valid(dst) && perm, "permute: invalid argument");
    RCU_REQUIRE(dev, movable_dtype(src->dt) && dst->dt == src->dt, "permute: unsupported dtype %d", src->dt);
    RCU_REQUIRE(dev, t_numel(src) == t_numel(dst), "permute: element counts differ");
    const uint32_t rank = src->rank, pad = 4 - rank;
    uint32_t seen = 0;
    for (uint32_t i = 0; i < rank; ++i) {
        RCU_REQUIRE(dev, perm[i] < rank, "permute: axis %u out of range", perm[i]);
        seen |= 1u << perm[i];
    }
    RCU_REQUIRE(dev, seen == (1u << rank) - 1, "permute: dims must be a permutation");
    DevGuard g(dev->ordinal);
    uint64_t s4[4];
    t_promote4(src, s4);
    uint32_t p4[4];
    for (uint32_t i = 0; i < 4; ++i) p4[i] = i < pad ? i : perm[i - pad] + pad;   // Permute::promote
    long long sstr[4] = {(long long)(s4[1] * s4[2] * s4[3]), (long long)(s4[2] * s4[3]), (long long)s4[3], 1};
    Remap4 p;
    p.off = 0;
    bool identity = true;
    for (int i = 0; i < 4; ++i) {
        RCU_REQUIRE(dev, s4[p4[i]] <= 0xffffffffull, "permute: dimension too large");
        p.d[i] = (uint32_t)s4[p4[i]];
        p.s[i] = sstr[p4[i]];
        // axes of size 1 can sit anywhere without moving data
        if (p.d[i] != 1) {
            // identity iff the non-unit axes keep their relative order
            for (int j = 0; j < i; ++j)
                if (p.d[j] != 1 && p4[j] > p4[i]) identity = false;
        }
    }
    const size_t n = t_numel(src);
    if (identity) {
        if (src->data != dst->data) RCU_CUDA(dev, cudaMemcpyAsync(dst->data, src->data, n * dt_esize(src->dt), cudaMemcpyDeviceToDevice, dev->stream));
        return RCU_OK;
    }
    // [.., R, C] -> [.., C, R] with leading axes untouched: tiled transpose
    if (p4[0] == 0 && p4[1] == 1 && p4[2] == 3 && p4[3] == 2 && s4[0] * s4[1] <= 65535 && s4[2] > 1 && s4[3] > 1) {
        const int R = (int)s4[2], C = (int)s4[3];
        const size_t pair = 2 * dt_esize(src->dt);
        const bool pairs_ok = R % 2 == 0 && C % 2 == 0 &&
                              ((reinterpret_cast<uintptr_t>(src->data) | reinterpret_cast<uintptr_t>(dst->data)) & (pair - 1)) == 0;
        if (pairs_ok && (R + 63) / 64 <= 65535) {
            dim3 g64((C + 63) / 64, (R + 63) / 64, (unsigned)(s4[0] * s4[1]));
            if (pair == 4) rcu_launch(dev, transpose_pair_kernel<uint16_t, uint32_t>, g64, 256, 0, (const uint16_t*)src->data, (uint16_t*)dst->data, R, C);
            else rcu_launch(dev, transpose_pair_kernel<uint32_t, uint2>, g64, 256, 0, (const uint32_t*)src->data, (uint32_t*)dst->data, R, C);
            RCU_LAUNCH_CHECK(dev);
            return RCU_OK;
        }
        dim3 grid((C + 31) / 32, (R + 31) / 32, (unsigned)(s4[0] * s4[1]));
        if (grid.y <= 65535) {
            if (dt_esize(src->dt) == 2) rcu_launch(dev, transpose_kernel<uint16_t>, grid, 256, 0, (const uint16_t*)src->data, (uint16_t*)dst->data, R, C);
            else rcu_launch(dev, transpose_kernel<uint32_t>, grid, 256, 0, (const uint32_t*)src->data, (uint32_t*)dst->data, R, C);
            RCU_LAUNCH_CHECK(dev);
            return RCU_OK;
        }
    }
    // [B, X, Y, D] -> [B, Y, X, D] (head split/merge): rows of D elements move as slabs
    if (p4[0] == 0 && p4[1] == 2 && p4[2] == 1 && p4[3] == 3) {
        // handled well enough by the generic kernel: the innermost axis stays contiguous on both sides
    }
    return remap(dev, src->dt, src->data, dst->data, n, p);
}

rcu_status rcu_slice(rcu_device* dev, const rcu_tensor* src, const uint64_t* start, const uint64_t* stop, rcu_tensor* dst) {
    if (!dev) return RCU_ERR_INVALID_ARG;
    RCU_REQUIRE(dev, t_valid(src) && t_valid(dst) && start && stop, "slice: invalid argument");
    RCU_REQUIRE(dev, movable_dtype(src->dt) && dst->dt == src->dt, "slice: unsupported dtype %d", src->dt);
    const uint32_t rank = src->rank, pad = 4 - rank;
    size_t n = 1;
    for (uint32_t i = 0; i < rank; ++i) {
        RCU_REQUIRE(dev, start[i] < stop[i] && stop[i] <= src->shape[i], "slice: bad range on axis %u", i);  // cpu/reindex.rs:111-113
        n *= stop[i] - start[i];
    }
    RCU_REQUIRE(dev, t_numel(dst) == n, "slice: dst holds %llu elements, expected %llu", (unsigned long long)t_numel(dst), (unsigned long long)n);
    DevGuard g(dev->ordinal);
    uint64_t s4[4], b4[4], e4[4];
    t_promote4(src, s4);
    for (uint32_t i = 0; i < 4; ++i) { b4[i] = i < pad ? 0 : start[i - pad]; e4[i] = i < pad ? 1 : stop[i - pad]; }
    long long sstr[4] = {(long long)(s4[1] * s4[2] * s4[3]), (long long)(s4[2] * s4[3]), (long long)s4[3], 1};
    // slab fast path: only one axis is actually cut -> pitched copy
    int cut = -1, ncut = 0;
    for (int i = 0; i < 4; ++i)
        if (e4[i] - b4[i] != s4[i]) { cut = i; ++ncut; }
    const size_t es = dt_esize(src->dt);
    if (ncut == 0) {
        if (src->data != dst->data) RCU_CUDA(dev, cudaMemcpyAsync(dst->data, src->data, n * es, cudaMemcpyDeviceToDevice, dev->stream));
        return RCU_OK;
    }
    if (ncut == 1) {
        size_t outer = 1, inner = 1;
        for (int i = 0; i < cut; ++i) outer *= s4[i];
        for (int i = cut + 1; i < 4; ++i) inner *= s4[i];
        const size_t len = e4[cut] - b4[cut];
        return copy2d(dev, (const char*)src->data + b4[cut] * inner * es, dst->data, outer, len * inner * es, s4[cut] * inner * es, len * inner * es);
    }
    Remap4 p;
    p.off = 0;
    for (int i = 0; i < 4; ++i) {
        p.d[i] = (uint32_t)(e4[i] - b4[i]);
        p.s[i] = sstr[i];
        p.off += (long long)b4[i] * sstr[i];
    }
    return remap(dev, src->dt, src->data, dst->data, n, p);
}

rcu_status rcu_broadcast(rcu_device* dev, const rcu_tensor* src, rcu_tensor* dst) {
    if (!dev) return RCU_ERR_INVALID_ARG;
    RCU_REQUIRE(dev, t_valid(src) && t_valid(dst), "broadcast: invalid tensor descriptor");
    RCU_REQUIRE(dev, movable_dtype(src->dt) && dst->dt == src->dt, "broadcast: unsupported dtype %d", src->dt);
    RCU_REQUIRE(dev, src->rank <= dst->rank, "broadcast: source rank exceeds destination rank");
    DevGuard g(dev->ordinal);
    uint64_t s4[4], d4[4];
    t_promote4(src, s4);
    t_promote4(dst, d4);
    Remap4 p;
    p.off = 0;
    long long acc = 1;
    for (int i = 3; i >= 0; --i) {
        RCU_REQUIRE(dev, s4[i] == d4[i] || s4[i] == 1, "broadcast: axis %d: %llu does not broadcast to %llu", i, (unsigned long long)s4[i], (unsigned long long)d4[i]);
        p.d[i] = (uint32_t)d4[i];
        p.s[i] = s4[i] == 1 ? 0 : acc;   // cpu/reindex.rs:204-216
        acc *= (long long)s4[i];
    }
    return remap(dev, src->dt, src->data, dst->data, t_numel(dst), p);
}

rcu_status rcu_concat(rcu_device* dev, const rcu_tensor* const* inputs, uint32_t n, uint32_t dim, rcu_tensor* dst) {
    if (!dev) return RCU_ERR_INVALID_ARG;
    RCU_REQUIRE(dev, inputs && n >= 1 && n <= RCU_MAX_CONCAT && t_valid(dst), "concat: 1..8 inputs required");  // ops/concat.rs:120-124
    const uint32_t rank = dst->rank;
    RCU_REQUIRE(dev, dim < rank, "concat: dim out of range");
    uint64_t along = 0;
    for (uint32_t k = 0; k < n; ++k) {
        const rcu_tensor* t = inputs[k];
        RCU_REQUIRE(dev, t_valid(t) && t->rank == rank && t->dt == dst->dt, "concat: input %u rank/dtype mismatch", k);
        RCU_REQUIRE(dev, t->data != dst->data, "concat cannot run in place");
        for (uint32_t i = 0; i < rank; ++i)
            RCU_REQUIRE(dev, i == dim || t->shape[i] == dst->shape[i], "concat: input %u differs from dst on axis %u", k, i);
        along += t->shape[dim];
    }
    RCU_REQUIRE(dev, along == dst->shape[dim], "concat: sizes along dim sum to %llu, dst has %llu", (unsigned long long)along, (unsigned long long)dst->shape[dim]);
    RCU_REQUIRE(dev, movable_dtype(dst->dt), "concat: unsupported dtype %d", dst->dt);
    DevGuard g(dev->ordinal);
    const size_t es = dt_esize(dst->dt);
    size_t outer = 1, inner = 1;
    for (uint32_t i = 0; i < dim; ++i) outer *= dst->shape[i];
    for (uint32_t i = dim + 1; i < rank; ++i) inner *= dst->shape[i];
    const size_t dpitch = dst->shape[dim] * inner * es;
    size_t off = 0;
    for (uint32_t k = 0; k < n; ++k) {
        const size_t row = inputs[k]->shape[dim] * inner * es;
        rcu_status st = copy2d(dev, inputs[k]->data, (char*)dst->data + off, outer, row, row, dpitch);
        if (st != RCU_OK) return st;
        off += row;
    }
    return RCU_OK;
}

rcu_status rcu_index_select(rcu_device* dev, const rcu_tensor* src, const rcu_tensor* ids, uint32_t dim, rcu_tensor* dst) {
    if (!dev) return RCU_ERR_INVALID_ARG;
    RCU_REQUIRE(dev, t_valid(src) && t_valid(ids) && t_valid(dst), "index_select: invalid tensor descriptor");
    RCU_REQUIRE(dev, src->rank == 2 && ids->rank == 1, "index_select: src must be 2-D and indices 1-D");   // ops/select.rs:64-69
    RCU_REQUIRE(dev, ids->dt == RCU_I32, "index_select: indices must be I32");
    RCU_REQUIRE(dev, dim < 2, "index_select: dim out of range");
    RCU_REQUIRE(dev, dst->dt == rcu_activation_dtype(src->dt), "index_select: dst dtype must be the source's activation dtype");
    const size_t n_ids = ids->shape[0];
    const size_t left = dim == 0 ? 1 : src->shape[0];
    const size_t right = dim == 0 ? src->shape[1] : 1;
    const size_t src_dim = src->shape[dim];
    RCU_REQUIRE(dev, t_numel(dst) == left * n_ids * right, "index_select: dst has the wrong size");
    DevGuard g(dev->ordinal);
    const size_t total = left * n_ids * right;
    if (total == 0) return RCU_OK;
    if (dt_is_q8(src->dt)) {
        RCU_REQUIRE(dev, right % 4 == 0 && right >= 4, "index_select: Q8_0 gather needs dim 0 and a row length divisible by 4");
        const uint32_t* q = (const uint32_t*)src->data;
        const char* d = (const char*)src->data + align256(t_numel(src));
        if (left == 1 && right % 16 == 0 && (reinterpret_cast<uintptr_t>(dst->data) & 15) == 0 && right / 16 <= 0xffffffffull) {
            const uint32_t row16 = (uint32_t)(right / 16);
            const int g16 = copy_grid(dev, n_ids * row16);
            if (src->dt == RCU_Q8_0F) rcu_launch(dev, gather_q8_rows16_kernel<float>, g16, 256, 0, (const uint4*)q, (const float*)d, (const int32_t*)ids->data, (float*)dst->data, n_ids, row16, src_dim, dev->d_status);
            else rcu_launch(dev, gather_q8_rows16_kernel<__half>, g16, 256, 0, (const uint4*)q, (const __half*)d, (const int32_t*)ids->data, (__half*)dst->data, n_ids, row16, src_dim, dev->d_status);
            RCU_LAUNCH_CHECK(dev);
            return RCU_OK;
        }
        const int grid = copy_grid(dev, total / 4);
        if (src->dt == RCU_Q8_0F) rcu_launch(dev, gather_q8_kernel<float>, grid, 256, 0, q, (const float*)d, (const int32_t*)ids->data, (float*)dst->data, left, n_ids, right, src_dim, dev->d_status);
        else rcu_launch(dev, gather_q8_kernel<__half>, grid, 256, 0, q, (const __half*)d, (const int32_t*)ids->data, (__half*)dst->data, left, n_ids, right, src_dim, dev->d_status);
        RCU_LAUNCH_CHECK(dev);
        return RCU_OK;
    }
    RCU_REQUIRE(dev, dt_is_float(src->dt), "index_select: unsupported dtype %d", src->dt);
    if (left == 1) {   // whole rows move: widest unit the row length and the pointers allow
        const size_t row_bytes = right * dt_esize(src->dt);
        const uintptr_t bits = reinterpret_cast<uintptr_t>(src->data) | reinterpret_cast<uintptr_t>(dst->data) | row_bytes;
#define RCU_GATHER_ROWS(U)                                                                                                                \
        {                                                                                                                                     \
            const size_t ru = row_bytes / sizeof(U);                                                                                          \
            const int gr = copy_grid(dev, n_ids * ru / 2 + 1);                                                                                \
            if (n_ids * ru <= 0xffffffffull) rcu_launch(dev, gather_rows_kernel<U, uint32_t>, gr, 256, 0, (const U*)src->data, (const int32_t*)ids->data, (U*)dst->data, n_ids, ru, src_dim, dev->d_status); \
            else rcu_launch(dev, gather_rows_kernel<U, uint64_t>, gr, 256, 0, (const U*)src->data, (const int32_t*)ids->data, (U*)dst->data, n_ids, ru, src_dim, dev->d_status); \
        }
        if ((bits & 15) == 0) RCU_GATHER_ROWS(uint4)
        else if ((bits & 3) == 0) RCU_GATHER_ROWS(uint32_t)
        else RCU_GATHER_ROWS(uint16_t)
#undef RCU_GATHER_ROWS
        RCU_LAUNCH_CHECK(dev);
        return RCU_OK;
    }
    const int grid = copy_grid(dev, total);
    if (dt_esize(src->dt) == 2) rcu_launch(dev, gather_kernel<uint16_t>, grid, 256, 0, (const uint16_t*)src->data, (const int32_t*)ids->data, (uint16_t*)dst->data, left, n_ids, right, src_dim, dev->d_status);
    else rcu_launch(dev, gather_kernel<uint32_t>, grid, 256, 0, (const uint32_t*)src->data, (const int32_t*)ids->data, (uint32_t*)dst->data, left, n_ids, right, src_dim, dev->d_status);
    RCU_LAUNCH_CHECK(dev);
    return RCU_OK;
}

rcu_status rcu_cache(rcu_device* dev, rcu_tensor* cache, const rcu_tensor* src, uint32_t dim, uint32_t offset, rcu_tensor* dst) {
    if (!dev) return RCU_ERR_INVALID_ARG;
    RCU_REQUIRE(dev, t_valid(cache) && t_valid(src), "cache: invalid tensor descriptor");
    RCU_REQUIRE(dev, cache->rank == src->rank && cache->dt == src->dt && movable_dtype(cache->dt), "cache: rank/dtype mismatch");
    const uint32_t rank = cache->rank;
    RCU_REQUIRE(dev, dim < rank, "cache: dim out of range");
    for (uint32_t i = 0; i < rank; ++i)
        RCU_REQUIRE(dev, i == dim || cache->shape[i] == src->shape[i], "cache: source differs from cache on axis %u", i);
    const uint64_t s = src->shape[dim];
    RCU_REQUIRE(dev, (uint64_t)offset + s <= cache->shape[dim], "cache: offset %u + %llu exceeds capacity %llu", offset, (unsigned long long)s, (unsigned long long)cache->shape[dim]);
    DevGuard g(dev->ordinal);
    const size_t es = dt_esize(cache->dt);
    size_t outer = 1, inner = 1;
    for (uint32_t i = 0; i < dim; ++i) outer *= cache->shape[i];
    for (uint32_t i = dim + 1; i < rank; ++i) inner *= cache->shape[i];
    const size_t cpitch = cache->shape[dim] * inner * es;
    // append: cache[:, offset:offset+s, :] = src
    rcu_status st = copy2d(dev, src->data, (char*)cache->data + (size_t)offset * inner * es, outer, s * inner * es, s * inner * es, cpitch);
    if (st != RCU_OK) return st;
    if (dst && dst->data) {
        RCU_REQUIRE(dev, dst->dt == cache->dt && dst->rank == rank && dst->shape[dim] == offset + s, "cache: dst must be [.., offset+s, ..]");
        RCU_REQUIRE(dev, dst->data != cache->data && dst->data != src->data, "cache cannot run in place");   // ops/cache.rs:40-42
        const size_t drow = (offset + s) * inner * es;
        st = copy2d(dev, cache->data, dst->data, outer, drow, cpitch, drow);
    }
    return st;
}

rcu_status rcu_index_write(rcu_device* dev, rcu_tensor* dst, const rcu_tensor* src, const uint64_t* start) {
    if (!dev) return RCU_ERR_INVALID_ARG;
    RCU_REQUIRE(dev, t_valid(dst) && t_valid(src) && start, "index_write: invalid argument");
    RCU_REQUIRE(dev, dst->rank == src->rank && dst->dt == src->dt && movable_dtype(dst->dt), "index_write: rank/dtype mismatch");
    const uint32_t rank = dst->rank, pad = 4 - rank;
    for (uint32_t i = 0; i < rank; ++i)
        RCU_REQUIRE(dev, start[i] + src->shape[i] <= dst->shape[i], "index_write: block exceeds dst on axis %u", i);
    DevGuard g(dev->ordinal);
    // iterate the source; destination offset = remap with dst strides: express as a remap from dst's
    // point of view is not possible (scatter), so copy row slabs of the innermost axis.
    uint64_t d4[4], s4[4], b4[4];
    t_promote4(dst, d4);
    t_promote4(src, s4);
    for (uint32_t i = 0; i < 4; ++i) b4[i] = i < pad ? 0 : start[i - pad];
    const size_t es = dt_esize(dst->dt);
    const size_t dstr[4] = {(size_t)(d4[1] * d4[2] * d4[3]), (size_t)(d4[2] * d4[3]), (size_t)d4[3], 1};
    // rows of s4[3] contiguous elements; group the two middle axes into pitched copies
    for (uint64_t i0 = 0; i0 < s4[0]; ++i0)
        for (uint64_t i1 = 0; i1 < s4[1]; ++i1) {
            const char* sp = (const char*)src->data + ((i0 * s4[1] + i1) * s4[2] * s4[3]) * es;
            char* dp = (char*)dst->data + ((b4[0] + i0) * dstr[0] + (b4[1] + i1) * dstr[1] + b4[2] * dstr[2] + b4[3]) * es;
            rcu_status st = copy2d(dev, sp, dp, s4[2], s4[3] * es, s4[3] * es, d4[3] * es);
            if (st != RCU_OK) return st;
        }
    return RCU_OK;
}

}  // extern "C"
