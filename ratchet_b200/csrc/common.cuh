// Internal helpers shared by every translation unit of libratchet_cuda.so.
#pragma once
#include <cstdlib>

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <map>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/ratchet_cuda.h"

// ------------------------------------------------------------------------------------------------
// Device handle
// ------------------------------------------------------------------------------------------------
struct rcu_pool {
    // size-class free lists; blocks are cudaMalloc'd once and recycled (no stream-ordered reuse
    // hazards: one stream per device, frees and allocations are issued in program order).
    std::multimap<uint64_t, void*> free_blocks;
    std::unordered_map<void*, uint64_t> live;      // ptr -> block size
    std::unordered_map<void*, uint64_t> all;       // every block owned by the pool
    uint64_t in_use = 0, reserved = 0;
};

struct rcu_device {
    int ordinal = 0;
    cudaStream_t stream = nullptr;
    bool owns_stream = false;
    int sm_count = 148;
    int smem_optin = 0;
    uint64_t launches = 0;
    std::string last_error;
    rcu_pool pool;
    int* d_status = nullptr;     // device-side status block: [0] bounds / timeout flags raised by kernels, [2..3] wait limit in ns (u64)
    uint64_t wait_limit_ns = 2000000000ull;
    bool const_weights = false;  // rcu_set_constant_weights: GEMVs may request weight rows before their predecessor ends
    int* h_status = nullptr;     // pinned host mirror
    rcu_resolve_stats last_resolve = {};   // counters of the last lazy-graph resolve (graph.cu)
    uint32_t debug_flags = 0;    // RCU_DEBUG_* (rcu_set_debug; RCU_NO_REUSE / RCU_PROFILE in the environment at creation)
    struct OpTime { uint64_t count = 0; double us = 0.0; uint64_t bytes = 0; };
    std::map<std::string, OpTime> op_times;   // per-op timing table of the lazy resolver (RCU_DEBUG_PROFILE)
    void* comm = nullptr;        // communicator state, owned by comm.cu
    // per-device resources created lazily by individual ops; run at rcu_device_destroy
    std::vector<std::pair<void (*)(void*), void*>> cleanup;
};

rcu_status rcu_fail(rcu_device* dev, rcu_status st, const char* fmt, ...);

#define RCU_CUDA(dev, expr)                                                                     \
    do {                                                                                        \
        cudaError_t _e = (expr);                                                                \
        if (_e != cudaSuccess)                                                                  \
            return rcu_fail((dev), RCU_ERR_CUDA, "%s failed: %s (%s:%d)", #expr,                \
                            cudaGetErrorString(_e), __FILE__, __LINE__);                        \
    } while (0)

#define RCU_REQUIRE(dev, cond, ...)                                                             \
    do {                                                                                        \
        if (!(cond)) return rcu_fail((dev), RCU_ERR_INVALID_ARG, __VA_ARGS__);                  \
    } while (0)

// Checks the launch itself (configuration errors); execution errors surface at rcu_sync.
#define RCU_LAUNCH_CHECK(dev)                                                                   \
    do {                                                                                        \
        (dev)->launches++;                                                                      \
        RCU_CUDA((dev), cudaGetLastError());                                                    \
    } while (0)

// Every kernel of the library begins with this: wait for the kernel before it in the stream (a no-op unless this
// one was launched as its programmatic dependent), then let the next kernel's blocks be scheduled.  Launched through
// rcu_launch, consecutive kernels overlap their launch and start-up with the predecessor's tail; nothing of a kernel's
// own work precedes the wait, so stream order is what the memory sees.
__device__ __forceinline__ void rcu_kernel_entry() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

// The entry of kernels that fill an SM on their own (the tensor-core GEMMs: one or two CTAs hold all of its shared
// memory): they wait, but leave the trigger to their completion, so that the next kernel's blocks do not move in while
// this one still wants every resource.
__device__ __forceinline__ void rcu_kernel_entry_wait_only() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// kern<<<grid, block, smem, dev->stream>>>(args...) as a programmatic dependent of the kernel before it
// (RCU_NO_PDL in the environment launches it plainly).  The kernel must call rcu_kernel_entry() first.
template <class... P, class... A>
inline cudaError_t rcu_launch(rcu_device* dev, void (*kern)(P...), dim3 grid, dim3 block, size_t smem, A&&... args) {
    static const bool pdl = std::getenv("RCU_NO_PDL") == nullptr;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = dev->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, static_cast<P>(args)...);
}

struct DevGuard {
    int prev = -1;
    explicit DevGuard(int ordinal) {
        cudaGetDevice(&prev);
        if (prev != ordinal) cudaSetDevice(ordinal);
        else prev = -1;
    }
    ~DevGuard() {
        if (prev >= 0) cudaSetDevice(prev);
    }
};

// ------------------------------------------------------------------------------------------------
// dtype / layout helpers (dtype/mod.rs, dtype/blocks.rs, gpu/align.rs)
// ------------------------------------------------------------------------------------------------
inline bool dt_is_q8(int dt) { return dt == RCU_Q8_0F || dt == RCU_Q8_0H; }
inline bool dt_is_q4k(int dt) { return dt == RCU_Q4_KF || dt == RCU_Q4_KH; }
inline bool dt_is_quant(int dt) { return dt_is_q8(dt) || dt_is_q4k(dt); }
inline bool dt_is_float(int dt) { return dt == RCU_F32 || dt == RCU_F16 || dt == RCU_BF16; }
inline uint64_t dt_esize(int dt) { return (dt == RCU_F16 || dt == RCU_BF16) ? 2 : 4; }
inline uint64_t align256(uint64_t n) { return (n + 255) / 256 * 256; }

inline uint64_t t_numel(const rcu_tensor* t) {
    uint64_t n = 1;
    for (uint32_t i = 0; i < t->rank; ++i) n *= t->shape[i];
    return n;
}
inline bool t_same_shape(const rcu_tensor* a, const rcu_tensor* b) {
    if (a->rank != b->rank) return false;
    for (uint32_t i = 0; i < a->rank; ++i)
        if (a->shape[i] != b->shape[i]) return false;
    return true;
}
inline bool t_valid(const rcu_tensor* t) { return t && t->rank >= 1 && t->rank <= RCU_MAX_RANK && t->data; }

// 4-D promotion by left padding with 1 (Shape::promote, shape.rs:94-98)
inline void t_promote4(const rcu_tensor* t, uint64_t out[4]) {
    uint32_t pad = 4 - t->rank;
    for (uint32_t i = 0; i < 4; ++i) out[i] = i < pad ? 1 : t->shape[i - pad];
}

inline int grid_for(uint64_t work_items, int per_block, int max_blocks) {
    uint64_t b = (work_items + per_block - 1) / per_block;
    if (b < 1) b = 1;
    if (b > (uint64_t)max_blocks) b = max_blocks;
    return (int)b;
}

// status-word bits raised by kernels
enum { RCU_DEVFLAG_BOUNDS = 1, RCU_DEVFLAG_TIMEOUT = 2 };
constexpr size_t kStatusBlockBytes = 16;

// ------------------------------------------------------------------------------------------------
// Device-side numeric helpers
// ------------------------------------------------------------------------------------------------
#ifdef __CUDACC__
template <class T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <class T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// round a float through T (T arithmetic = f32 op then round to nearest even)
template <class T> __device__ __forceinline__ float rnd(float v) { return to_f32<T>(from_f32<T>(v)); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// How long a device-side wait may last before it gives up, in nanoseconds (rcu_set_wait_limit_ns); kept in
// the device's status block next to the flag word every waiting kernel already holds a pointer to.
__device__ __forceinline__ unsigned long long rcu_wait_limit(const int* status) {
    return *reinterpret_cast<const volatile unsigned long long*>(status + 2);
}

// streaming 16-byte load that does not allocate in L1 (weights are read exactly once)
__device__ __forceinline__ uint4 ld_stream_v4(const void* p) {
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.L2::128B.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(p));
    return r;
}
#endif
