/*
 * ratchet_cuda.h — C ABI of the sm_100a CUDA device for ratchet-core's tensor-op hot path.
 *
 * ratchet has no FFI surface of its own: a device is an arm of three internal Rust enums/traits
 * (Device, Storage, and the per-op resolve path).  Every entry point below names the reference
 * interface it stands in for, by path inside the reference repository.  A Rust `-sys` crate binds
 * these symbols one to one; the Python package binds the same symbols with ctypes.
 *
 * Conventions
 *   - Every call returns an rcu_status; nothing aborts or throws across this boundary.  A
 *     human-readable message for the last failing call on a device is kept per device
 *     (rcu_last_error).
 *   - One CUDA stream per rcu_device.  All launches and copies are asynchronous on that stream;
 *     only rcu_d2h and rcu_sync block.  Calls on one handle must be serialised by the caller
 *     (the reference drives one device from one thread at a time); distinct handles are independent.
 *   - Tensors are contiguous, row-major, rank <= 4, described by a caller-owned POD (rcu_tensor).
 *     Ops never allocate their output: the caller passes `dst` (ratchet-core/src/tensor.rs:817-821).
 *   - A quantised tensor is ONE buffer holding ratchet's segments back to back, each padded to
 *     256 bytes (ratchet-core/src/dtype/blocks.rs:69-82,124-148); `shape` is the logical shape.
 *   - There is no CPU fallback: an unsupported combination returns RCU_ERR_UNSUPPORTED.
 */
#ifndef RATCHET_CUDA_H
#define RATCHET_CUDA_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define RCU_MAX_RANK 4
#define RCU_MAX_CONCAT 8 /* ratchet-core/src/ops/concat.rs:120-124 */

typedef enum {
    RCU_OK = 0,
    RCU_ERR_INVALID_ARG = 1, /* InvariantError / OpGuards panics in the reference (op.rs:217-228) */
    RCU_ERR_UNSUPPORTED = 2, /* dtype/shape combination with no kernel (InvariantError::UnsupportedDType) */
    RCU_ERR_OOM = 3,         /* DeviceError / allocator failure */
    RCU_ERR_CUDA = 4,        /* CUDA runtime error */
    RCU_ERR_NCCL = 5,
    RCU_ERR_TIMEOUT = 6,     /* a bounded device-side wait gave up */
    RCU_ERR_BOUNDS = 7,      /* index outside a tensor (e.g. gather id) */
    RCU_ERR_INPLACE = 8      /* OperationError::InplaceError (ops/concat.rs:35-37) */
} rcu_status;

/* ratchet-core/src/dtype/mod.rs:11-23 */
typedef enum {
    RCU_F32 = 0,
    RCU_F16 = 1,
    RCU_BF16 = 2,
    RCU_I32 = 3,
    RCU_U32 = 4,
    RCU_Q8_0F = 5, /* int8 x32 blocks, f32 scale */
    RCU_Q8_0H = 6, /* int8 x32 blocks, f16 scale */
    RCU_Q4_KF = 7, /* GGUF Q4_K super-blocks, f32 d/dmin */
    RCU_Q4_KH = 8  /* GGUF Q4_K super-blocks, f16 d/dmin */
} rcu_dtype;

/* ops/binary.rs:19-45, ops/unary.rs:23-60, ops/norm/mod.rs:18-60 */
typedef enum { RCU_ADD = 0, RCU_SUB = 1, RCU_MUL = 2, RCU_DIV = 3 } rcu_binary_op;
typedef enum {
    RCU_GELU = 0, RCU_TANH = 1, RCU_EXP = 2, RCU_LOG = 3, RCU_SIN = 4, RCU_COS = 5, RCU_ABS = 6, RCU_SQRT = 7,
    RCU_RELU = 8, RCU_FLOOR = 9, RCU_CEIL = 10, RCU_NEG = 11, RCU_SILU = 12, RCU_SIGMOID = 13
} rcu_unary_op;
typedef enum { RCU_LAYER_NORM = 0, RCU_RMS_NORM = 1, RCU_GROUP_NORM = 2 } rcu_norm_kind;
typedef enum { RCU_REDUCE_SUM = 0, RCU_REDUCE_MAX = 1, RCU_REDUCE_MEAN = 2 } rcu_reduce_kind;

/* StorageView + storage pointer of a resolved tensor (ratchet-core/src/tensor.rs:131-151). */
typedef struct {
    int32_t dt;                    /* rcu_dtype */
    uint32_t rank;                 /* 1..RCU_MAX_RANK */
    uint64_t shape[RCU_MAX_RANK];  /* row-major, contiguous */
    void* data;                    /* device pointer */
} rcu_tensor;

typedef struct rcu_device rcu_device;

/* ------------------------------------------------------------------ device (device.rs:25-93) */
/* Device::request_device(DeviceRequest::GPU): open CUDA device `ordinal` with its own stream. */
rcu_status rcu_device_create(int ordinal, rcu_device** out);
/* Same, but every launch goes to the caller's cudaStream_t (e.g. the stream of a host framework). */
rcu_status rcu_device_create_on_stream(int ordinal, void* cuda_stream, rcu_device** out);
void rcu_device_destroy(rcu_device* dev);
const char* rcu_last_error(rcu_device* dev);
/* Number of kernels this handle has launched since creation (profiling aid, gpu/profiler.rs). */
uint64_t rcu_launch_count(rcu_device* dev);
int rcu_sm_count(rcu_device* dev);

/* Debug switches of a device (also read from the environment when the device is created: RCU_NO_REUSE=1,
 * RCU_PROFILE=1, RCU_LOG=1).  RCU_DEBUG_NO_REUSE: the lazy resolver gives every tensor a buffer of its own and runs nothing
 * in place (the reference's RATCHET_DEBUG, gpu/buffer_allocator/allocator.rs:121).  RCU_DEBUG_PROFILE: the lazy
 * resolver brackets every node with an event pair and blocks at the end of each resolve, filling a per-op table
 * (the reference's `gpu-profiling` feature, gpu/profiler.rs:95-237, executable.rs:140-179).  RCU_DEBUG_LOG: every
 * resolve writes one line per launching node (op, dtype, shape, in place or not) and a summary (nodes, launches,
 * buffers, planned against unshared bytes) to stderr, where the reference logs its kernel keys and allocation totals
 * (op.rs:312, gpu/buffer_allocator/allocator.rs:330-337). */
#define RCU_DEBUG_NO_REUSE 1u
#define RCU_DEBUG_PROFILE 2u
#define RCU_DEBUG_LOG 4u
rcu_status rcu_set_debug(rcu_device* dev, uint32_t flags);
/* The per-op table as text — kernel key (op and operand dtype), count, total microseconds, share, GB/s over the
 * operands' bytes — sorted by time.  Returns the bytes needed (with the terminator); writes at most `capacity`.
 * reset != 0 clears the table. */
uint64_t rcu_profile_report(rcu_device* dev, char* buf, uint64_t capacity, int reset);

/* ------------------------------------------------------------------ storage (storage/gpu_buffer.rs) */
/* BufferAllocator / BufferPool: pooled device memory (gpu/pools/buffer_pool.rs:80-94 rounds sizes
 * up to 4 B with a 16 B minimum; this pool rounds to 256 B size classes and caches freed blocks). */
rcu_status rcu_alloc(rcu_device* dev, uint64_t nbytes, void** dptr);
rcu_status rcu_free(rcu_device* dev, void* dptr);
/* Return cached blocks to the driver (WgpuDevice::begin_pass garbage collection analogue). */
rcu_status rcu_pool_trim(rcu_device* dev);
/* bytes currently handed out / bytes held by the pool (allocator.rs:330-337 logs the same) */
void rcu_pool_stats(rcu_device* dev, uint64_t* in_use, uint64_t* reserved);
/* GPUBuffer::from_bytes (storage/gpu_buffer.rs:49-60) and to_cpu (200-218). d2h blocks. */
/* h2d from pageable memory returns when the source has been read; from pinned memory it is fully
 * asynchronous: the source must stay untouched until the next rcu_sync / rcu_d2h on this device. */
rcu_status rcu_h2d(rcu_device* dev, void* dst, const void* src, uint64_t nbytes);
rcu_status rcu_d2h(rcu_device* dev, void* dst, const void* src, uint64_t nbytes);
/* d2h without the wait: `dst` should be pinned memory and is valid after the next rcu_sync / rcu_d2h on this
 * handle.  With a second handle on a stream of its own (rcu_device_create_on_stream) and rcu_stream_wait, the
 * copy of one step's result overlaps the next step's kernels. */
rcu_status rcu_d2h_async(rcu_device* dev, void* dst, const void* src, uint64_t nbytes);
/* Work queued on `dev` after this call starts only when everything queued on `other` (same GPU) so far has
 * finished.  Does not block the host. */
rcu_status rcu_stream_wait(rcu_device* dev, rcu_device* other);
rcu_status rcu_d2d(rcu_device* dev, void* dst, const void* src, uint64_t nbytes);
rcu_status rcu_memset(rcu_device* dev, void* dst, int value, uint64_t nbytes);
/* device.poll(Wait) (tensor.rs:856).  Also reports what kernels flagged since the last check:
 * RCU_ERR_BOUNDS (an index outside its tensor) or RCU_ERR_TIMEOUT (a bounded device-side wait gave up). */
rcu_status rcu_sync(rcu_device* dev);
/* Every device-side wait (on a peer's data, on another CTA, on an asynchronous copy) gives up after this
 * long, raises the time-out flag and lets its kernel run to the end, so the context stays usable; default
 * two seconds.  The reference has no counterpart (its only wait is device.poll).  Applies to kernels
 * launched after the call. */
rcu_status rcu_set_wait_limit_ns(rcu_device* dev, uint64_t nanoseconds);
/* A promise about the weight operand (lhs) of the matrix-vector products that follow: on != 0 says that no work
 * still in flight on this handle's stream writes those buffers (a loaded model's Linear weights,
 * ratchet-nn/src/linear.rs:10-24).  The GEMV kernels are then launched as programmatic dependents of their
 * predecessor and request their first weight rows while it drains; activations, bias and output are touched only
 * after the predecessor has completed, as always.  Off by default: through rcu_matmul the predecessor may be the
 * kernel that produced the weights.  The lazy resolver switches it on by itself for weights that were uploaded with
 * rcu_lazy_from_host (resident before the call returned).  No counterpart in the reference. */
rcu_status rcu_set_constant_weights(rcu_device* dev, int on);

/* ------------------------------------------------------------------ layouts (dtype/blocks.rs) */
/* DType::segments total: bytes of the single buffer that holds `numel` elements of `dt`. */
uint64_t rcu_dtype_nbytes(int32_t dt, uint64_t numel);
/* Byte offsets of the segments: Q8_0 -> {qs, d}; Q4_K -> {qs, scales, dmin, d}; returns count. */
int rcu_dtype_segments(int32_t dt, uint64_t numel, uint64_t offsets[4]);
/* DType::activation_dt (dtype/mod.rs:97-105) */
int32_t rcu_activation_dtype(int32_t dt);

/* ------------------------------------------------------------------ ops */
/* dequantize (quant.rs:132-164) on the device: bit-exact with the CPU routine. src is Q8_0F/H or
 * Q4_KF/H, dst is F32 (…F) or F16 (…H) of the same shape. */
rcu_status rcu_dequantize(rcu_device* dev, const rcu_tensor* src, rcu_tensor* dst);
/* quantize (quant.rs:19-99) on the host: `src` holds `numel` f32 (dt = RCU_Q8_0F) or f16 (dt = RCU_Q8_0H)
 * values, `host_out` receives the ratchet buffer (rcu_dtype_nbytes(dt, numel) bytes, padding zeroed).  Bit for
 * bit the reference's output, including its corner cases (all-zero blocks, NaN, Rust's saturating casts).
 * numel must be a multiple of 32.  The Q4_K arms of the reference emit an absmax layout that nothing
 * consumes: RCU_ERR_UNSUPPORTED (Q4_K buffers come from rcu_gguf_transcode).  Touches no device. */
rcu_status rcu_quantize(int32_t dt, const void* src, uint64_t numel, void* host_out, uint64_t out_bytes);
/* The same on the device: src F32 -> dst Q8_0F, src F16 -> dst Q8_0H, same shape; same bits as rcu_quantize. */
rcu_status rcu_quantize_device(rcu_device* dev, const rcu_tensor* src, rcu_tensor* dst);

/* Matmul (ops/matmul/mod.rs:381-545; Tensor::gemm tensor.rs:409-419).  dst dtype = rhs dtype.
 * Allowed (lhs, rhs) pairs: (F32,F32) (F16,F16) (Q8_0F,F32) (Q8_0H,F16) (Q4_KF,F32) (Q4_KH,F16)
 * as in check_dtypes (mod.rs:518-534), plus (Q8_0F,F16): f32 block scales with f16 activations.
 * bias (nullable) is a vector over dst's last dimension, in the rhs dtype. */
rcu_status rcu_matmul(rcu_device* dev, const rcu_tensor* lhs, const rcu_tensor* rhs, const rcu_tensor* bias,
                      int trans_lhs, int trans_rhs, int trans_dst, rcu_tensor* dst);
/* Matmul::compute_dst_shape (mod.rs:392-466): fills dst->rank/shape/dt, touches no memory. */
rcu_status rcu_matmul_dst_shape(const rcu_tensor* lhs, const rcu_tensor* rhs, int trans_lhs, int trans_rhs,
                                int trans_dst, rcu_tensor* dst);

/* Binary (ops/binary.rs): same-shape operands, or `b` broadcastable to `a`'s shape (the reference
 * materialises the broadcast first, tensor.rs:252-278; here it is folded into the kernel).
 * dst may alias a (in-place, binary.rs:130-132). */
rcu_status rcu_binary(rcu_device* dev, int op, const rcu_tensor* a, const rcu_tensor* b, rcu_tensor* dst);
/* Unary (ops/unary.rs); dst may alias x. */
rcu_status rcu_unary(rcu_device* dev, int op, const rcu_tensor* x, rcu_tensor* dst);
/* Cast (ops/cast.rs; cpu/mod.rs:127-156: f32<->f16, f32<->bf16 convert, f32<->i32/u32 reinterpret). */
rcu_status rcu_cast(rcu_device* dev, const rcu_tensor* x, rcu_tensor* dst);
/* Norm (ops/norm/mod.rs): LayerNorm / RMSNorm over the last dimension; bias nullable;
 * GroupNorm takes x [B,C,L] with `groups`. */
rcu_status rcu_norm(rcu_device* dev, int kind, const rcu_tensor* x, const rcu_tensor* scale, const rcu_tensor* bias,
                    float eps, uint32_t groups, rcu_tensor* dst);
/* Softmax (ops/softmax.rs) over `dim`, which must be the last dimension; dst may alias x. */
rcu_status rcu_softmax(rcu_device* dev, const rcu_tensor* x, uint32_t dim, rcu_tensor* dst);
/* Row reduction over the last dimension (the reduce step shared by Norm and Softmax; cpu/norm.rs:72-89). */
rcu_status rcu_reduce(rcu_device* dev, int kind, const rcu_tensor* x, rcu_tensor* dst);
/* RoPE (ops/rope.rs): x [B,H,S,D], rotates the first `dim` features; dst may alias x. */
rcu_status rcu_rope(rcu_device* dev, const rcu_tensor* x, uint32_t dim, float base, uint32_t offset, rcu_tensor* dst);
/* Concat (ops/concat.rs): n <= 8 inputs along `dim`. */
rcu_status rcu_concat(rcu_device* dev, const rcu_tensor* const* inputs, uint32_t n, uint32_t dim, rcu_tensor* dst);
/* IndexSelect (ops/select.rs): src rank 2 (float or Q8_0), ids rank-1 I32; Q8_0 tables are
 * dequantised while gathering into the activation dtype. An id outside the table sets RCU_ERR_BOUNDS
 * on the next rcu_sync/rcu_d2h (the row is clamped, select.rs:157). */
rcu_status rcu_index_select(rcu_device* dev, const rcu_tensor* src, const rcu_tensor* ids, uint32_t dim, rcu_tensor* dst);
/* Reindex (ops/reindex/{permute,slice,broadcast}.rs) */
rcu_status rcu_permute(rcu_device* dev, const rcu_tensor* src, const uint32_t* perm, rcu_tensor* dst);
rcu_status rcu_slice(rcu_device* dev, const rcu_tensor* src, const uint64_t* start, const uint64_t* stop, rcu_tensor* dst);
rcu_status rcu_broadcast(rcu_device* dev, const rcu_tensor* src, rcu_tensor* dst);
/* Cache (ops/cache.rs): cache[..., offset:offset+s, ...] = src along `dim`, and
 * dst = cache[..., :offset+s, ...].  When dst->data is NULL only the append happens and the
 * caller reads the prefix of `cache` directly (valid for dim <= 1 leading size-1 dims, or when the
 * consumer takes a row stride). */
rcu_status rcu_cache(rcu_device* dev, rcu_tensor* cache, const rcu_tensor* src, uint32_t dim, uint32_t offset, rcu_tensor* dst);
/* IndexWrite (ops/index_write.rs): dst[start + i] = src[i]. */
rcu_status rcu_index_write(rcu_device* dev, rcu_tensor* dst, const rcu_tensor* src, const uint64_t* start);
/* Conv (ops/conv.rs): conv1d with kernel size 3; x [B,Cin,L], w [Cout,Cin,3], bias [Cout]. */
rcu_status rcu_conv1d(rcu_device* dev, const rcu_tensor* x, const rcu_tensor* w, const rcu_tensor* bias,
                      uint32_t stride, uint32_t padding, rcu_tensor* dst);

/* ------------------------------------------------------------------ lazy tensor graph (tensor.rs)
 * rcu_lazy is ratchet-core's `Tensor` (tensor.rs:45-47): a reference-counted node of a lazy DAG.
 * Builders validate their arguments and compute the output view exactly when the reference's
 * builder methods do (tensor.rs:294-510); nothing runs on the device until rcu_lazy_resolve
 * (Tensor::resolve, tensor.rs:861-863), which walks the graph in the reference's execution order
 * (tensor.rs:696-740), plans buffers by liveness with greedy-by-size sharing and in-place leasing
 * (gpu/buffer_allocator/allocator.rs:141-340) and launches one kernel per node on the device's
 * stream.  A handle owns one reference; rcu_lazy_release drops it (Drop for Tensor).  Builders
 * retain their sources, so a source handle may be released right after building on it — which is
 * what lets an op run in place (tensor.rs:823-824: only when the op is the source's sole owner). */
typedef struct rcu_lazy rcu_lazy;

/* Tensor::from_data / from_quantized: copy host bytes into a new pooled device buffer (resolved leaf). */
rcu_status rcu_lazy_from_host(rcu_device* dev, int32_t dt, uint32_t rank, const uint64_t* shape, const void* host,
                              uint64_t nbytes, rcu_lazy** out);
/* Tensor::zeros */
rcu_status rcu_lazy_zeros(rcu_device* dev, int32_t dt, uint32_t rank, const uint64_t* shape, rcu_lazy** out);
/* A resolved leaf over device memory the caller owns (never freed by the library).  `dev` may be NULL for a
 * graph that is only built and inspected (rcu_lazy_execution_order) and never resolved. */
rcu_status rcu_lazy_wrap(rcu_device* dev, const rcu_tensor* t, rcu_lazy** out);
void rcu_lazy_retain(rcu_lazy* t);
void rcu_lazy_release(rcu_lazy* t);
/* shape / dtype / device pointer (NULL until resolved); returns 1 if resolved (Tensor::resolved). */
int rcu_lazy_info(const rcu_lazy* t, rcu_tensor* out);
/* Arc::strong_count of the node (handles + consumers). */
uint32_t rcu_lazy_strong_count(const rcu_lazy* t);

rcu_status rcu_lazy_binary(int op, rcu_lazy* a, rcu_lazy* b, rcu_lazy** out);
rcu_status rcu_lazy_unary(int op, rcu_lazy* x, rcu_lazy** out);
rcu_status rcu_lazy_cast(rcu_lazy* x, int32_t dt, rcu_lazy** out);
rcu_status rcu_lazy_norm(int kind, rcu_lazy* x, rcu_lazy* scale, rcu_lazy* bias, float eps, uint32_t groups, rcu_lazy** out);
rcu_status rcu_lazy_softmax(rcu_lazy* x, uint32_t dim, rcu_lazy** out);
rcu_status rcu_lazy_rope(rcu_lazy* x, uint32_t dim, float base, uint32_t offset, rcu_lazy** out);
rcu_status rcu_lazy_matmul(rcu_lazy* lhs, rcu_lazy* rhs, rcu_lazy* bias, int trans_lhs, int trans_rhs, int trans_dst, rcu_lazy** out);
rcu_status rcu_lazy_conv1d(rcu_lazy* x, rcu_lazy* w, rcu_lazy* bias, uint32_t stride, uint32_t padding, rcu_lazy** out);
rcu_status rcu_lazy_view(rcu_lazy* x, uint32_t rank, const uint64_t* shape, rcu_lazy** out);
rcu_status rcu_lazy_slice(rcu_lazy* x, const uint64_t* start, const uint64_t* stop, rcu_lazy** out);
rcu_status rcu_lazy_permute(rcu_lazy* x, const uint32_t* perm, rcu_lazy** out);
rcu_status rcu_lazy_broadcast(rcu_lazy* x, uint32_t rank, const uint64_t* shape, rcu_lazy** out);
rcu_status rcu_lazy_concat(rcu_lazy* const* inputs, uint32_t n, uint32_t dim, rcu_lazy** out);
rcu_status rcu_lazy_index_select(rcu_lazy* src, rcu_lazy* ids, uint32_t dim, rcu_lazy** out);
rcu_status rcu_lazy_cache(rcu_lazy* cache, rcu_lazy* src, uint32_t dim, uint32_t offset, rcu_lazy** out);
rcu_status rcu_lazy_index_write(rcu_lazy* dst, rcu_lazy* src, const uint64_t* start, rcu_lazy** out);

/* Tensor::id (tensor.rs:100-104): process-wide unique, increasing with creation. */
uint64_t rcu_lazy_id(const rcu_lazy* t);
/* Tensor::execution_order (tensor.rs:696-740): ids of every node `t` depends on, `t` last, in the order resolve
 * runs them.  *n_nodes receives the count; at most `capacity` ids are written.  Touches no device. */
rcu_status rcu_lazy_execution_order(rcu_lazy* t, uint64_t* ids, uint32_t capacity, uint32_t* n_nodes);
/* Tensor::resolve: run every unresolved node `t` depends on.  Asynchronous on the device stream. */
rcu_status rcu_lazy_resolve(rcu_lazy* t);
/* Tensor::to(Device::CPU): resolve if needed, copy to host, block. */
rcu_status rcu_lazy_to_host(rcu_lazy* t, void* host, uint64_t nbytes);
/* Counters of the last resolve on this device: nodes visited, kernels launched, ops run in place,
 * bytes of distinct buffers planned vs bytes if every node had its own (allocator.rs:330-337). */
typedef struct { uint32_t nodes, launched, inplace, buffers; uint64_t planned_bytes, naive_bytes; } rcu_resolve_stats;
void rcu_last_resolve_stats(rcu_device* dev, rcu_resolve_stats* out);

/* ------------------------------------------------------------------ fused decode step
 * One decoder-only transformer step at sequence length 1 — the graph Phi3::schedule builds per
 * token (ratchet-models/src/phi3/model.rs:134-156, attn.rs:88-159, mlp.rs:31-39) — executed as a
 * fixed sequence of fused kernels replayed from a CUDA graph instead of ~43 kernels per layer:
 *   embedding row gather (Q8_0 dequant) -> per layer { RMSNorm+qkv GEMV, RoPE + KV append +
 *   split-KV attention, o GEMV + residual, RMSNorm + gate_up GEMV + SiLU gate, down GEMV + residual }
 *   -> RMSNorm + lm_head GEMV (-> optional argmax).
 * Weights are ratchet Q8_0 buffers (Q8_0H or Q8_0F), activations f16, norm scales f32, KV caches
 * f16 [n_kv_heads, max_cache, head_dim] per layer as ratchet-nn allocates them (kv_cache.rs:11-18).
 * All pointers are device memory owned by the caller and must outlive the decoder. */
typedef struct rcu_comm rcu_comm;       /* exchange window between the GPUs of a node (declared with rcu_comm_* below) */
typedef struct rcu_decoder rcu_decoder;
typedef struct {
    uint32_t n_layers, d_model, n_heads, n_kv_heads, head_dim, ffn, vocab, max_cache, rope_dim;
    float rope_base, rms_eps;
    int32_t weight_dt; /* RCU_Q8_0H or RCU_Q8_0F */
} rcu_decoder_config;
typedef struct {
    const void* attn_norm; /* f32 [d_model] */
    const void* qkv;       /* Q8_0 [(n_heads + 2 n_kv_heads) * head_dim, d_model] */
    const void* o;         /* Q8_0 [d_model, n_heads * head_dim] */
    const void* ffn_norm;  /* f32 [d_model] */
    const void* gate_up;   /* Q8_0 [2 ffn, d_model]: gate rows then up rows */
    const void* down;      /* Q8_0 [d_model, ffn] */
    void* k_cache;         /* f16 [n_kv_heads, max_cache, head_dim] */
    void* v_cache;
} rcu_decoder_layer;
rcu_status rcu_decoder_create(rcu_device* dev, const rcu_decoder_config* cfg, const rcu_decoder_layer* layers,
                              const void* tok_embd /* Q8_0 [vocab, d_model] */, const void* out_norm /* f32 [d_model] */,
                              const void* lm_head /* Q8_0 [vocab, d_model] */, rcu_decoder** out);
/* The same decoder sharded over the GPUs of one node, one process per GPU (no counterpart in the
 * reference, which drives one device).  `cfg` describes the WHOLE model; rank r of a world of g
 * passes its own shards: qkv = the q, k and v rows of heads [r H/g, (r+1) H/g) (q rows, then k, then v),
 * o / down = rows [r d/g, (r+1) d/g), gate_up = gate rows then up rows of ffn columns
 * [r f/g, (r+1) f/g), lm_head = rows [r V/g, (r+1) V/g), KV caches for its own kv heads; norms and
 * the embedding table are whole.  `comm` must be a fresh window (rcu_comm_create + every peer
 * imported) with slots of at least 4 * max(d_model, ffn, vocab, n_heads * head_dim) bytes; the decoder
 * owns its flags from here on.  All ranks must call rcu_decoder_step with the same token, in step;
 * logits and arg-max are complete and identical on every rank.  A peer that stops answering ends
 * each wait after two seconds; the next rcu_sync then returns RCU_ERR_TIMEOUT. */
rcu_status rcu_decoder_create_sharded(rcu_device* dev, rcu_comm* comm, const rcu_decoder_config* cfg, const rcu_decoder_layer* layers,
                                      const void* tok_embd, const void* out_norm, const void* lm_head, rcu_decoder** out);
void rcu_decoder_destroy(rcu_decoder* dec);
/* Number of KV entries already in the caches = position of the next token (KVCache::entries). */
rcu_status rcu_decoder_set_position(rcu_decoder* dec, uint32_t position);
uint32_t rcu_decoder_position(const rcu_decoder* dec);
/* Run one step for the token id at `token_dev` (device int32). Writes f16 logits [vocab] to
 * `logits_dev` and, when `argmax_dev` is not NULL, the arg-max token id (device int32) — which may
 * be the same address as `token_dev` for greedy generation without a host round trip.  Advances the
 * position by one (KVCache::update(1)).  Asynchronous on the device stream. */
rcu_status rcu_decoder_step(rcu_decoder* dec, const int32_t* token_dev, void* logits_dev, int32_t* argmax_dev);
/* Kernels per step of the captured graph (profiling aid). */
uint32_t rcu_decoder_kernels_per_step(const rcu_decoder* dec);
/* Profiling aid in the spirit of the reference's per-op timestamps (gpu/profiler.rs:95-237): runs one step
 * like rcu_decoder_step (no arg-max), outside the CUDA graph, and returns the device clock (nanoseconds) at
 * which the first CTA of the data-flow kernel began each of its jobs and had that job's input vector staged
 * (for attention: had its own tiles folded) — per layer: qkv, attention, o, gate/up, down; then lm_head — plus
 * one final stamp at its end: 2 n_jobs + 1 values; then, for each of the six job kinds (qkv, attention, o,
 * gate/up, down, lm_head), four sums of SM clock cycles spent by the grid's first warp waiting for a ring slot,
 * multiplying, storing results and requesting the next items: 24 more values.  Blocks until the step is done.
 * RCU_ERR_INVALID_ARG if the decoder runs kernel by kernel (shapes the data-flow kernel does not take). */
rcu_status rcu_decoder_profile_step(rcu_decoder* dec, const int32_t* token_dev, void* logits_dev, uint64_t* stamps_ns,
                                    uint32_t capacity, uint32_t* n_stamps);

/* Decode attention for one layer, standalone (the kernel rcu_decoder_step uses): RoPE on q and k
 * (ops/rope.rs), append k/v at `position` (ops/cache.rs), softmax(q.K^T * scale).V over
 * position + 1 entries (phi3/attn.rs:142-157).  qkv is f16 [(n_heads + 2 n_kv_heads) * head_dim];
 * out is f16 [n_heads * head_dim].  Split-KV partial results go through device scratch memory that
 * the device handle allocates on first use. */
rcu_status rcu_attn_decode(rcu_device* dev, const void* qkv, void* k_cache, void* v_cache, uint32_t n_heads,
                           uint32_t n_kv_heads, uint32_t head_dim, uint32_t max_cache, uint32_t rope_dim, float rope_base,
                           uint32_t position, void* out);

/* rcu_attn_decode without any device allocation.  It has no counterpart in the reference.  It exists
 * for callers that cannot allocate device memory when they need attention: plug-ins running inside a
 * host framework that owns the device heap, latency-bound serving loops that cannot take the device
 * synchronisation of an allocation, processes that have given all free memory to their KV caches.
 * The split-KV scratch is a fixed 2.04 MiB array inside the library's device image (held by every GPU
 * that loads the library until the process exits), which limits this variant to n_heads <= 64,
 * head_dim <= 128 and max_cache <= 4096 positions; larger requests return RCU_ERR_INVALID_ARG with a
 * message naming the limit.
 * Same arguments and results as rcu_attn_decode.  The first call on a device looks up the array's
 * device address and should be made before any stream capture.  All calls on a device share the
 * array: calls that overlap on the GPU race, so keep them on one stream or otherwise ordered. */
rcu_status rcu_attn_decode_static(rcu_device* dev, const void* qkv, void* k_cache, void* v_cache, uint32_t n_heads,
                                  uint32_t n_kv_heads, uint32_t head_dim, uint32_t max_cache, uint32_t rope_dim,
                                  float rope_base, uint32_t position, void* out);

/* ------------------------------------------------------------------ row-sharded Linear over the GPUs of a node
 * No counterpart in the reference, which is single-device (gpu/device.rs:15-16).  A Linear's weight
 * W[N,K] (ratchet-nn/src/linear.rs:17-24) is split by rows: rank r of g holds rows [r N/g, (r+1) N/g)
 * as its own ratchet Q8_0 buffer.  One process per GPU; each creates a window (full-size f16 output slots,
 * arrival counters), exports it as a 64-byte CUDA IPC handle, the host framework exchanges the handles, and every
 * rank imports its peers'.  rcu_gemv_q8_allgather runs the local GEMV; each warp stores its finished rows into
 * every peer's window over NVLink as it goes, each CTA then counts itself in on every peer, and the kernel ends
 * once every peer's CTAs have arrived here (bounded: RCU_ERR_TIMEOUT at the next sync).  Every rank must call with
 * shards of the same shape.  *y_full is the device pointer of the gathered f16 [N] output, valid until the call
 * after next.  The kernel is launched so that it may begin requesting weights while the previous kernel on the
 * stream is still finishing: a weight shard produced on the device must be complete (rcu_sync) before the call. */
rcu_status rcu_comm_create(rcu_device* dev, int rank, int world, uint64_t slot_bytes, rcu_comm** out);
rcu_status rcu_comm_export(rcu_comm* comm, void* handle64);
rcu_status rcu_comm_import(rcu_comm* comm, int peer, const void* handle64);
/* The same for a peer window that lives in this process on the same device (CUDA IPC handles cannot be opened
 * by the process that exported them): links `other`'s window as rank `peer`.  `other` must outlive `comm`. */
rcu_status rcu_comm_import_local(rcu_comm* comm, int peer, rcu_comm* other);
void rcu_comm_destroy(rcu_comm* comm);
int rcu_comm_rank(const rcu_comm* comm);
int rcu_comm_world(const rcu_comm* comm);
rcu_status rcu_gemv_q8_allgather(rcu_comm* comm, const rcu_tensor* w_shard, const rcu_tensor* x, const rcu_tensor* bias_shard,
                                 void** y_full);

/* ------------------------------------------------------------------ GGUF files (host side)
 * ratchet-loader/src/gguf/gguf.rs:422-509 (header, metadata, tensor infos; GGUF v1-v3) and
 * gguf/dtype.rs:39-198 (transcode of ggml blocks into ratchet's segment layout).  The file is
 * memory-mapped; nothing here touches a device.  Errors: rcu_gguf_last_error() (per thread). */
typedef struct rcu_gguf rcu_gguf;
typedef struct {
    const char* name;      /* owned by the handle */
    uint32_t rank;         /* 1..4 */
    uint64_t shape[4];     /* ratchet order, outermost first (GGUF stores innermost first; gguf.rs:470) */
    uint32_t ggml_type;    /* 0 F32, 1 F16, 8 Q8_0, 12 Q4_K; others can be listed but not transcoded */
    uint64_t numel;
    uint64_t file_bytes;   /* bytes of the tensor in the file (0 for unsupported types) */
} rcu_gguf_tensor_info;
rcu_status rcu_gguf_open(const char* path, rcu_gguf** out);
void rcu_gguf_close(rcu_gguf* g);
const char* rcu_gguf_last_error(void);
uint32_t rcu_gguf_version(const rcu_gguf* g);
uint64_t rcu_gguf_tensor_count(const rcu_gguf* g);
int64_t rcu_gguf_find(const rcu_gguf* g, const char* name);            /* index or -1 */
rcu_status rcu_gguf_tensor(const rcu_gguf* g, uint64_t index, rcu_gguf_tensor_info* out);
rcu_status rcu_gguf_meta_u64(const rcu_gguf* g, const char* key, uint64_t* out);   /* integer and bool values */
rcu_status rcu_gguf_meta_f64(const rcu_gguf* g, const char* key, double* out);
rcu_status rcu_gguf_meta_str(const rcu_gguf* g, const char* key, char* buf, uint64_t buf_bytes);
/* dtype `ratchet_from_gguf` picks (gguf.rs:113-156): Q8_0 / Q4_K take f16 scales on an f16-capable device. -1: unsupported. */
int32_t rcu_gguf_target_dtype(uint32_t ggml_type, int f16_device);
/* Writes tensor `index` as dtype `dt` in ratchet's layout into `host_out` (rcu_dtype_nbytes(dt, numel) bytes). */
rcu_status rcu_gguf_transcode(const rcu_gguf* g, uint64_t index, int32_t dt, void* host_out, uint64_t out_bytes);

#ifdef __cplusplus
}
#endif
#endif /* RATCHET_CUDA_H */
