// Device handle, caching device allocator, transfers and layout queries.
//
// Stands in for ratchet-core's WgpuDevice (gpu/device.rs:18-119), BufferPool
// (gpu/pools/buffer_pool.rs) and GPUBuffer transfers (storage/gpu_buffer.rs:49-60,200-218).
#include <cstdlib>

#include "common.cuh"

rcu_status rcu_fail(rcu_device* dev, rcu_status st, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    if (dev) dev->last_error = buf;
    return st;
}

static rcu_status create_common(int ordinal, cudaStream_t stream, bool own, rcu_device** out) {
    if (!out) return RCU_ERR_INVALID_ARG;
    *out = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || ordinal < 0 || ordinal >= count) return RCU_ERR_CUDA;
    rcu_device* dev = new rcu_device();
    dev->ordinal = ordinal;
    DevGuard g(ordinal);
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, ordinal) != cudaSuccess) { delete dev; return RCU_ERR_CUDA; }
    if (prop.major != 10) {
        // This library carries sm_100a code only; there is no other code path to fall back to.
        delete dev;
        return RCU_ERR_UNSUPPORTED;
    }
    dev->sm_count = prop.multiProcessorCount;
    dev->smem_optin = (int)prop.sharedMemPerBlockOptin;
    if (own) {
        if (cudaStreamCreateWithFlags(&dev->stream, cudaStreamNonBlocking) != cudaSuccess) { delete dev; return RCU_ERR_CUDA; }
        dev->owns_stream = true;
    } else {
        dev->stream = stream;
    }
    if (cudaMalloc(&dev->d_status, kStatusBlockBytes) != cudaSuccess || cudaMallocHost(&dev->h_status, sizeof(int)) != cudaSuccess) {
        delete dev;
        return RCU_ERR_OOM;
    }
    if (const char* e = std::getenv("RCU_NO_REUSE")) dev->debug_flags |= std::atoi(e) ? RCU_DEBUG_NO_REUSE : 0;
    if (const char* e = std::getenv("RCU_PROFILE")) dev->debug_flags |= std::atoi(e) ? RCU_DEBUG_PROFILE : 0;
    if (const char* e = std::getenv("RCU_LOG")) dev->debug_flags |= std::atoi(e) ? RCU_DEBUG_LOG : 0;
    cudaMemsetAsync(dev->d_status, 0, kStatusBlockBytes, dev->stream);
    cudaMemcpyAsync(reinterpret_cast<char*>(dev->d_status) + 8, &dev->wait_limit_ns, 8, cudaMemcpyHostToDevice, dev->stream);
    cudaStreamSynchronize(dev->stream);
    *dev->h_status = 0;
    *out = dev;
    return RCU_OK;
}

extern "C" {

rcu_status rcu_device_create(int ordinal, rcu_device** out) { return create_common(ordinal, nullptr, true, out); }

rcu_status rcu_device_create_on_stream(int ordinal, void* cuda_stream, rcu_device** out) {
    return create_common(ordinal, (cudaStream_t)cuda_stream, false, out);
}

void rcu_device_destroy(rcu_device* dev) {
    if (!dev) return;
    DevGuard g(dev->ordinal);
    cudaStreamSynchronize(dev->stream);
    for (auto it = dev->cleanup.rbegin(); it != dev->cleanup.rend(); ++it) it->first(it->second);
    for (auto& kv : dev->pool.all) cudaFree(kv.first);
    if (dev->d_status) cudaFree(dev->d_status);
    if (dev->h_status) cudaFreeHost(dev->h_status);
    if (dev->owns_stream) cudaStreamDestroy(dev->stream);
    delete dev;
}

const char* rcu_last_error(rcu_device* dev) { return dev ? dev->last_error.c_str() : "null device"; }
uint64_t rcu_launch_count(rcu_device* dev) { return dev ? dev->launches : 0; }
int rcu_sm_count(rcu_device* dev) { return dev ? dev->sm_count : 0; }

// ---------------------------------------------------------------------------------- allocator
// Size classes: multiples of 256 B up to 1 MiB, then multiples of 1 MiB (keeps reuse likely for the
// repeated intermediate sizes of a decode step while bounding internal fragmentation to < 1 MiB).
static uint64_t size_class(uint64_t n) {
    if (n < 16) n = 16;  // buffer_pool.rs:80-94 minimum
    if (n <= (1u << 20)) return align256(n);
    const uint64_t mib = 1u << 20;
    return (n + mib - 1) / mib * mib;
}

rcu_status rcu_alloc(rcu_device* dev, uint64_t nbytes, void** dptr) {
    if (!dev || !dptr) return RCU_ERR_INVALID_ARG;
    DevGuard g(dev->ordinal);
    uint64_t sz = size_class(nbytes);
    auto it = dev->pool.free_blocks.find(sz);
    void* p = nullptr;
    if (it != dev->pool.free_blocks.end()) {
        p = it->second;
        dev->pool.free_blocks.erase(it);
    } else {
        cudaError_t e = cudaMalloc(&p, sz);
        if (e != cudaSuccess) {
            // release cached blocks and retry once
            cudaGetLastError();
            rcu_pool_trim(dev);
            e = cudaMalloc(&p, sz);
            if (e != cudaSuccess) {
                cudaGetLastError();
                return rcu_fail(dev, RCU_ERR_OOM, "cudaMalloc(%llu) failed: %s", (unsigned long long)sz, cudaGetErrorString(e));
            }
        }
        dev->pool.all[p] = sz;
        dev->pool.reserved += sz;
    }
    dev->pool.live[p] = sz;
    dev->pool.in_use += sz;
    *dptr = p;
    return RCU_OK;
}

rcu_status rcu_free(rcu_device* dev, void* dptr) {
    if (!dev) return RCU_ERR_INVALID_ARG;
    if (!dptr) return RCU_OK;
    auto it = dev->pool.live.find(dptr);
    if (it == dev->pool.live.end()) return rcu_fail(dev, RCU_ERR_INVALID_ARG, "rcu_free: pointer not owned by this device's pool");
    dev->pool.free_blocks.emplace(it->second, dptr);
    dev->pool.in_use -= it->second;
    dev->pool.live.erase(it);
    return RCU_OK;
}

rcu_status rcu_pool_trim(rcu_device* dev) {
    if (!dev) return RCU_ERR_INVALID_ARG;
    DevGuard g(dev->ordinal);
    cudaStreamSynchronize(dev->stream);
    for (auto& kv : dev->pool.free_blocks) {
        cudaFree(kv.second);
        dev->pool.reserved -= kv.first;
        dev->pool.all.erase(kv.second);
    }
    dev->pool.free_blocks.clear();
    return RCU_OK;
}

void rcu_pool_stats(rcu_device* dev, uint64_t* in_use, uint64_t* reserved) {
    if (in_use) *in_use = dev ? dev->pool.in_use : 0;
    if (reserved) *reserved = dev ? dev->pool.reserved : 0;
}

// ---------------------------------------------------------------------------------- transfers
rcu_status rcu_h2d(rcu_device* dev, void* dst, const void* src, uint64_t nbytes) {
    if (!dev || (nbytes && (!dst || !src))) return RCU_ERR_INVALID_ARG;
    DevGuard g(dev->ordinal);
    RCU_CUDA(dev, cudaMemcpyAsync(dst, src, nbytes, cudaMemcpyHostToDevice, dev->stream));
    return RCU_OK;
}

static rcu_status check_status_word(rcu_device* dev) {
    int flags = *dev->h_status;
    if (flags) {
        *dev->h_status = 0;
        cudaMemsetAsync(dev->d_status, 0, sizeof(int), dev->stream);
        if (flags & RCU_DEVFLAG_TIMEOUT) return rcu_fail(dev, RCU_ERR_TIMEOUT, "a device-side bounded wait gave up");
        if (flags & RCU_DEVFLAG_BOUNDS) return rcu_fail(dev, RCU_ERR_BOUNDS, "a kernel saw an index outside its tensor (clamped)");
    }
    return RCU_OK;
}

rcu_status rcu_d2h(rcu_device* dev, void* dst, const void* src, uint64_t nbytes) {
    if (!dev || (nbytes && (!dst || !src))) return RCU_ERR_INVALID_ARG;
    DevGuard g(dev->ordinal);
    RCU_CUDA(dev, cudaMemcpyAsync(dst, src, nbytes, cudaMemcpyDeviceToHost, dev->stream));
    RCU_CUDA(dev, cudaMemcpyAsync(dev->h_status, dev->d_status, sizeof(int), cudaMemcpyDeviceToHost, dev->stream));
    RCU_CUDA(dev, cudaStreamSynchronize(dev->stream));
    return check_status_word(dev);
}

rcu_status rcu_d2h_async(rcu_device* dev, void* dst, const void* src, uint64_t nbytes) {
    if (!dev || (nbytes && (!dst || !src))) return RCU_ERR_INVALID_ARG;
    DevGuard g(dev->ordinal);
    RCU_CUDA(dev, cudaMemcpyAsync(dst, src, nbytes, cudaMemcpyDeviceToHost, dev->stream));
    return RCU_OK;
}

rcu_status rcu_stream_wait(rcu_device* dev, rcu_device* other) {
    if (!dev || !other) return RCU_ERR_INVALID_ARG;
    RCU_REQUIRE(dev, dev->ordinal == other->ordinal, "stream_wait: the handles are on different GPUs");
    DevGuard g(dev->ordinal);
    cudaEvent_t ev;
    RCU_CUDA(dev, cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
    cudaError_t e = cudaEventRecord(ev, other->stream);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(dev->stream, ev, 0);
    cudaEventDestroy(ev);                 // released once the wait has been satisfied
    if (e != cudaSuccess) return rcu_fail(dev, RCU_ERR_CUDA, "stream_wait: %s", cudaGetErrorString(e));
    return RCU_OK;
}

rcu_status rcu_d2d(rcu_device* dev, void* dst, const void* src, uint64_t nbytes) {
    if (!dev || (nbytes && (!dst || !src))) return RCU_ERR_INVALID_ARG;
    DevGuard g(dev->ordinal);
    RCU_CUDA(dev, cudaMemcpyAsync(dst, src, nbytes, cudaMemcpyDeviceToDevice, dev->stream));
    return RCU_OK;
}

rcu_status rcu_memset(rcu_device* dev, void* dst, int value, uint64_t nbytes) {
    if (!dev || (nbytes && !dst)) return RCU_ERR_INVALID_ARG;
    DevGuard g(dev->ordinal);
    RCU_CUDA(dev, cudaMemsetAsync(dst, value, nbytes, dev->stream));
    return RCU_OK;
}

rcu_status rcu_sync(rcu_device* dev) {
    if (!dev) return RCU_ERR_INVALID_ARG;
    DevGuard g(dev->ordinal);
    RCU_CUDA(dev, cudaMemcpyAsync(dev->h_status, dev->d_status, sizeof(int), cudaMemcpyDeviceToHost, dev->stream));
    RCU_CUDA(dev, cudaStreamSynchronize(dev->stream));
    return check_status_word(dev);
}

rcu_status rcu_set_constant_weights(rcu_device* dev, int on) {
    if (!dev) return RCU_ERR_INVALID_ARG;
    dev->const_weights = on != 0;
    return RCU_OK;
}

rcu_status rcu_set_wait_limit_ns(rcu_device* dev, uint64_t nanoseconds) {
    if (!dev || nanoseconds == 0) return RCU_ERR_INVALID_ARG;
    DevGuard g(dev->ordinal);
    dev->wait_limit_ns = nanoseconds;
    // ordered on the stream: kernels launched after this call see the new limit
    RCU_CUDA(dev, cudaMemcpyAsync(reinterpret_cast<char*>(dev->d_status) + 8, &dev->wait_limit_ns, 8, cudaMemcpyHostToDevice, dev->stream));
    RCU_CUDA(dev, cudaStreamSynchronize(dev->stream));
    return RCU_OK;
}

// ---------------------------------------------------------------------------------- layouts
uint64_t rcu_dtype_nbytes(int32_t dt, uint64_t numel) {
    switch (dt) {
        case RCU_Q8_0F: return align256(numel) + align256(numel / 32 * 4);
        case RCU_Q8_0H: return align256(numel) + align256(numel / 32 * 2);
        case RCU_Q4_KF:
        case RCU_Q4_KH: {
            uint64_t fp = dt == RCU_Q4_KF ? 4 : 2, nb = numel / 256;
            return align256(numel / 2) + align256(nb * 12) + 2 * align256(nb * fp);
        }
        default: {
            uint64_t n = numel * dt_esize(dt);
            if (n < 16) n = 16;          // MIN_STORAGE_BUFFER_SIZE
            return (n + 3) / 4 * 4;      // align_for_copy
        }
    }
}

int rcu_dtype_segments(int32_t dt, uint64_t numel, uint64_t off[4]) {
    if (dt_is_q8(dt)) {
        off[0] = 0;
        off[1] = align256(numel);
        return 2;
    }
    if (dt_is_q4k(dt)) {
        uint64_t fp = dt == RCU_Q4_KF ? 4 : 2, nb = numel / 256;
        off[0] = 0;
        off[1] = align256(numel / 2);
        off[2] = off[1] + align256(nb * 12);
        off[3] = off[2] + align256(nb * fp);
        return 4;
    }
    off[0] = 0;
    return 1;
}

int32_t rcu_activation_dtype(int32_t dt) {
    switch (dt) {
        case RCU_Q8_0H: case RCU_Q4_KH: return RCU_F16;
        case RCU_Q8_0F: case RCU_Q4_KF: return RCU_F32;
        default: return dt;
    }
}

}  // extern "C"
