//! Raw bindings of `libratchet_cuda.so`: one declaration per symbol of `include/ratchet_cuda.h`, same
//! order, same argument names.
//!
//! UNVERIFIED: written without a Rust toolchain at hand (none is installed where this library is built).
//! `tests/test_rust_bindings.py` parses this file and the C header and fails on any missing symbol, arity
//! mismatch or argument type that does not correspond, so the two cannot drift apart unnoticed.
//!
//! Linking: `build.rs` adds `RATCHET_CUDA_LIB_DIR` (default `../../ratchet_b200`) to the search path.
#![allow(non_camel_case_types)]

use std::os::raw::{c_char, c_int, c_void};

pub const RCU_MAX_RANK: usize = 4;
pub const RCU_MAX_CONCAT: usize = 8;

/// `rcu_status`
pub type rcu_status = c_int;
pub const RCU_OK: rcu_status = 0;
pub const RCU_ERR_INVALID_ARG: rcu_status = 1;
pub const RCU_ERR_UNSUPPORTED: rcu_status = 2;
pub const RCU_ERR_OOM: rcu_status = 3;
pub const RCU_ERR_CUDA: rcu_status = 4;
pub const RCU_ERR_NCCL: rcu_status = 5;
pub const RCU_ERR_TIMEOUT: rcu_status = 6;
pub const RCU_ERR_BOUNDS: rcu_status = 7;
pub const RCU_ERR_INPLACE: rcu_status = 8;

/// `rcu_dtype` (ratchet-core/src/dtype/mod.rs:11-23)
pub const RCU_F32: i32 = 0;
pub const RCU_F16: i32 = 1;
pub const RCU_BF16: i32 = 2;
pub const RCU_I32: i32 = 3;
pub const RCU_U32: i32 = 4;
pub const RCU_Q8_0F: i32 = 5;
pub const RCU_Q8_0H: i32 = 6;
pub const RCU_Q4_KF: i32 = 7;
pub const RCU_Q4_KH: i32 = 8;

/// `rcu_binary_op`, `rcu_unary_op`, `rcu_norm_kind`, `rcu_reduce_kind`
pub const RCU_ADD: c_int = 0;
pub const RCU_SUB: c_int = 1;
pub const RCU_MUL: c_int = 2;
pub const RCU_DIV: c_int = 3;
pub const RCU_GELU: c_int = 0;
pub const RCU_TANH: c_int = 1;
pub const RCU_EXP: c_int = 2;
pub const RCU_LOG: c_int = 3;
pub const RCU_SIN: c_int = 4;
pub const RCU_COS: c_int = 5;
pub const RCU_ABS: c_int = 6;
pub const RCU_SQRT: c_int = 7;
pub const RCU_RELU: c_int = 8;
pub const RCU_FLOOR: c_int = 9;
pub const RCU_CEIL: c_int = 10;
pub const RCU_NEG: c_int = 11;
pub const RCU_SILU: c_int = 12;
pub const RCU_SIGMOID: c_int = 13;
pub const RCU_LAYER_NORM: c_int = 0;
pub const RCU_RMS_NORM: c_int = 1;
pub const RCU_GROUP_NORM: c_int = 2;
pub const RCU_REDUCE_SUM: c_int = 0;
pub const RCU_REDUCE_MAX: c_int = 1;
pub const RCU_REDUCE_MEAN: c_int = 2;
pub const RCU_DEBUG_NO_REUSE: u32 = 1;
pub const RCU_DEBUG_PROFILE: u32 = 2;
pub const RCU_DEBUG_LOG: u32 = 4;

/// StorageView + storage pointer of a resolved tensor.
#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct rcu_tensor {
    pub dt: i32,
    pub rank: u32,
    pub shape: [u64; RCU_MAX_RANK],
    pub data: *mut c_void,
}

#[repr(C)]
#[derive(Clone, Copy, Debug, Default)]
pub struct rcu_resolve_stats {
    pub nodes: u32,
    pub launched: u32,
    pub inplace: u32,
    pub buffers: u32,
    pub planned_bytes: u64,
    pub naive_bytes: u64,
}

#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct rcu_decoder_config {
    pub n_layers: u32,
    pub d_model: u32,
    pub n_heads: u32,
    pub n_kv_heads: u32,
    pub head_dim: u32,
    pub ffn: u32,
    pub vocab: u32,
    pub max_cache: u32,
    pub rope_dim: u32,
    pub rope_base: f32,
    pub rms_eps: f32,
    pub weight_dt: i32,
}

#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct rcu_decoder_layer {
    pub attn_norm: *const c_void,
    pub qkv: *const c_void,
    pub o: *const c_void,
    pub ffn_norm: *const c_void,
    pub gate_up: *const c_void,
    pub down: *const c_void,
    pub k_cache: *mut c_void,
    pub v_cache: *mut c_void,
}

#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct rcu_gguf_tensor_info {
    pub name: *const c_char,
    pub rank: u32,
    pub shape: [u64; 4],
    pub ggml_type: u32,
    pub numel: u64,
    pub file_bytes: u64,
}

macro_rules! opaque {
    ($($name:ident),*) => { $(#[repr(C)] pub struct $name { _private: [u8; 0] })* };
}
opaque!(rcu_device, rcu_lazy, rcu_comm, rcu_decoder, rcu_gguf);

#[link(name = "ratchet_cuda")]
extern "C" {
    pub fn rcu_device_create(ordinal: c_int, out: *mut *mut rcu_device) -> rcu_status;
    pub fn rcu_device_create_on_stream(ordinal: c_int, cuda_stream: *mut c_void, out: *mut *mut rcu_device) -> rcu_status;
    pub fn rcu_device_destroy(dev: *mut rcu_device);
    pub fn rcu_last_error(dev: *mut rcu_device) -> *const c_char;
    pub fn rcu_launch_count(dev: *mut rcu_device) -> u64;
    pub fn rcu_sm_count(dev: *mut rcu_device) -> c_int;
    pub fn rcu_set_debug(dev: *mut rcu_device, flags: u32) -> rcu_status;
    pub fn rcu_profile_report(dev: *mut rcu_device, buf: *mut c_char, capacity: u64, reset: c_int) -> u64;
    pub fn rcu_alloc(dev: *mut rcu_device, nbytes: u64, dptr: *mut *mut c_void) -> rcu_status;
    pub fn rcu_free(dev: *mut rcu_device, dptr: *mut c_void) -> rcu_status;
    pub fn rcu_pool_trim(dev: *mut rcu_device) -> rcu_status;
    pub fn rcu_pool_stats(dev: *mut rcu_device, in_use: *mut u64, reserved: *mut u64);
    pub fn rcu_h2d(dev: *mut rcu_device, dst: *mut c_void, src: *const c_void, nbytes: u64) -> rcu_status;
    pub fn rcu_d2h(dev: *mut rcu_device, dst: *mut c_void, src: *const c_void, nbytes: u64) -> rcu_status;
    pub fn rcu_d2h_async(dev: *mut rcu_device, dst: *mut c_void, src: *const c_void, nbytes: u64) -> rcu_status;
    pub fn rcu_stream_wait(dev: *mut rcu_device, other: *mut rcu_device) -> rcu_status;
    pub fn rcu_d2d(dev: *mut rcu_device, dst: *mut c_void, src: *const c_void, nbytes: u64) -> rcu_status;
    pub fn rcu_memset(dev: *mut rcu_device, dst: *mut c_void, value: c_int, nbytes: u64) -> rcu_status;
    pub fn rcu_sync(dev: *mut rcu_device) -> rcu_status;
    pub fn rcu_set_wait_limit_ns(dev: *mut rcu_device, nanoseconds: u64) -> rcu_status;
    pub fn rcu_set_constant_weights(dev: *mut rcu_device, on: c_int) -> rcu_status;
    pub fn rcu_dtype_nbytes(dt: i32, numel: u64) -> u64;
    pub fn rcu_dtype_segments(dt: i32, numel: u64, offsets: *mut u64) -> c_int;
    pub fn rcu_activation_dtype(dt: i32) -> i32;
    pub fn rcu_dequantize(dev: *mut rcu_device, src: *const rcu_tensor, dst: *mut rcu_tensor) -> rcu_status;
    pub fn rcu_quantize(dt: i32, src: *const c_void, numel: u64, host_out: *mut c_void, out_bytes: u64) -> rcu_status;
    pub fn rcu_quantize_device(dev: *mut rcu_device, src: *const rcu_tensor, dst: *mut rcu_tensor) -> rcu_status;
    pub fn rcu_matmul(dev: *mut rcu_device, lhs: *const rcu_tensor, rhs: *const rcu_tensor, bias: *const rcu_tensor, trans_lhs: c_int, trans_rhs: c_int, trans_dst: c_int, dst: *mut rcu_tensor) -> rcu_status;
    pub fn rcu_matmul_dst_shape(lhs: *const rcu_tensor, rhs: *const rcu_tensor, trans_lhs: c_int, trans_rhs: c_int, trans_dst: c_int, dst: *mut rcu_tensor) -> rcu_status;
    pub fn rcu_binary(dev: *mut rcu_device, op: c_int, a: *const rcu_tensor, b: *const rcu_tensor, dst: *mut rcu_tensor) -> rcu_status;
    pub fn rcu_unary(dev: *mut rcu_device, op: c_int, x: *const rcu_tensor, dst: *mut rcu_tensor) -> rcu_status;
    pub fn rcu_cast(dev: *mut rcu_device, x: *const rcu_tensor, dst: *mut rcu_tensor) -> rcu_status;
    pub fn rcu_norm(dev: *mut rcu_device, kind: c_int, x: *const rcu_tensor, scale: *const rcu_tensor, bias: *const rcu_tensor, eps: f32, groups: u32, dst: *mut rcu_tensor) -> rcu_status;
    pub fn rcu_softmax(dev: *mut rcu_device, x: *const rcu_tensor, dim: u32, dst: *mut rcu_tensor) -> rcu_status;
    pub fn rcu_reduce(dev: *mut rcu_device, kind: c_int, x: *const rcu_tensor, dst: *mut rcu_tensor) -> rcu_status;
    pub fn rcu_rope(dev: *mut rcu_device, x: *const rcu_tensor, dim: u32, base: f32, offset: u32, dst: *mut rcu_tensor) -> rcu_status;
    pub fn rcu_concat(dev: *mut rcu_device, inputs: *const *const rcu_tensor, n: u32, dim: u32, dst: *mut rcu_tensor) -> rcu_status;
    pub fn rcu_index_select(dev: *mut rcu_device, src: *const rcu_tensor, ids: *const rcu_tensor, dim: u32, dst: *mut rcu_tensor) -> rcu_status;
    pub fn rcu_permute(dev: *mut rcu_device, src: *const rcu_tensor, perm: *const u32, dst: *mut rcu_tensor) -> rcu_status;
    pub fn rcu_slice(dev: *mut rcu_device, src: *const rcu_tensor, start: *const u64, stop: *const u64, dst: *mut rcu_tensor) -> rcu_status;
    pub fn rcu_broadcast(dev: *mut rcu_device, src: *const rcu_tensor, dst: *mut rcu_tensor) -> rcu_status;
    pub fn rcu_cache(dev: *mut rcu_device, cache: *mut rcu_tensor, src: *const rcu_tensor, dim: u32, offset: u32, dst: *mut rcu_tensor) -> rcu_status;
    pub fn rcu_index_write(dev: *mut rcu_device, dst: *mut rcu_tensor, src: *const rcu_tensor, start: *const u64) -> rcu_status;
    pub fn rcu_conv1d(dev: *mut rcu_device, x: *const rcu_tensor, w: *const rcu_tensor, bias: *const rcu_tensor, stride: u32, padding: u32, dst: *mut rcu_tensor) -> rcu_status;
    pub fn rcu_lazy_from_host(dev: *mut rcu_device, dt: i32, rank: u32, shape: *const u64, host: *const c_void, nbytes: u64, out: *mut *mut rcu_lazy) -> rcu_status;
    pub fn rcu_lazy_zeros(dev: *mut rcu_device, dt: i32, rank: u32, shape: *const u64, out: *mut *mut rcu_lazy) -> rcu_status;
    pub fn rcu_lazy_wrap(dev: *mut rcu_device, t: *const rcu_tensor, out: *mut *mut rcu_lazy) -> rcu_status;
    pub fn rcu_lazy_retain(t: *mut rcu_lazy);
    pub fn rcu_lazy_release(t: *mut rcu_lazy);
    pub fn rcu_lazy_info(t: *const rcu_lazy, out: *mut rcu_tensor) -> c_int;
    pub fn rcu_lazy_strong_count(t: *const rcu_lazy) -> u32;
    pub fn rcu_lazy_binary(op: c_int, a: *mut rcu_lazy, b: *mut rcu_lazy, out: *mut *mut rcu_lazy) -> rcu_status;
    pub fn rcu_lazy_unary(op: c_int, x: *mut rcu_lazy, out: *mut *mut rcu_lazy) -> rcu_status;
    pub fn rcu_lazy_cast(x: *mut rcu_lazy, dt: i32, out: *mut *mut rcu_lazy) -> rcu_status;
    pub fn rcu_lazy_norm(kind: c_int, x: *mut rcu_lazy, scale: *mut rcu_lazy, bias: *mut rcu_lazy, eps: f32, groups: u32, out: *mut *mut rcu_lazy) -> rcu_status;
    pub fn rcu_lazy_softmax(x: *mut rcu_lazy, dim: u32, out: *mut *mut rcu_lazy) -> rcu_status;
    pub fn rcu_lazy_rope(x: *mut rcu_lazy, dim: u32, base: f32, offset: u32, out: *mut *mut rcu_lazy) -> rcu_status;
    pub fn rcu_lazy_matmul(lhs: *mut rcu_lazy, rhs: *mut rcu_lazy, bias: *mut rcu_lazy, trans_lhs: c_int, trans_rhs: c_int, trans_dst: c_int, out: *mut *mut rcu_lazy) -> rcu_status;
    pub fn rcu_lazy_conv1d(x: *mut rcu_lazy, w: *mut rcu_lazy, bias: *mut rcu_lazy, stride: u32, padding: u32, out: *mut *mut rcu_lazy) -> rcu_status;
    pub fn rcu_lazy_view(x: *mut rcu_lazy, rank: u32, shape: *const u64, out: *mut *mut rcu_lazy) -> rcu_status;
    pub fn rcu_lazy_slice(x: *mut rcu_lazy, start: *const u64, stop: *const u64, out: *mut *mut rcu_lazy) -> rcu_status;
    pub fn rcu_lazy_permute(x: *mut rcu_lazy, perm: *const u32, out: *mut *mut rcu_lazy) -> rcu_status;
    pub fn rcu_lazy_broadcast(x: *mut rcu_lazy, rank: u32, shape: *const u64, out: *mut *mut rcu_lazy) -> rcu_status;
    pub fn rcu_lazy_concat(inputs: *const *mut rcu_lazy, n: u32, dim: u32, out: *mut *mut rcu_lazy) -> rcu_status;
    pub fn rcu_lazy_index_select(src: *mut rcu_lazy, ids: *mut rcu_lazy, dim: u32, out: *mut *mut rcu_lazy) -> rcu_status;
    pub fn rcu_lazy_cache(cache: *mut rcu_lazy, src: *mut rcu_lazy, dim: u32, offset: u32, out: *mut *mut rcu_lazy) -> rcu_status;
    pub fn rcu_lazy_index_write(dst: *mut rcu_lazy, src: *mut rcu_lazy, start: *const u64, out: *mut *mut rcu_lazy) -> rcu_status;
    pub fn rcu_lazy_id(t: *const rcu_lazy) -> u64;
    pub fn rcu_lazy_execution_order(t: *mut rcu_lazy, ids: *mut u64, capacity: u32, n_nodes: *mut u32) -> rcu_status;
    pub fn rcu_lazy_resolve(t: *mut rcu_lazy) -> rcu_status;
    pub fn rcu_lazy_to_host(t: *mut rcu_lazy, host: *mut c_void, nbytes: u64) -> rcu_status;
    pub fn rcu_last_resolve_stats(dev: *mut rcu_device, out: *mut rcu_resolve_stats);
    pub fn rcu_decoder_create(dev: *mut rcu_device, cfg: *const rcu_decoder_config, layers: *const rcu_decoder_layer, tok_embd: *const c_void, out_norm: *const c_void, lm_head: *const c_void, out: *mut *mut rcu_decoder) -> rcu_status;
    pub fn rcu_decoder_create_sharded(dev: *mut rcu_device, comm: *mut rcu_comm, cfg: *const rcu_decoder_config, layers: *const rcu_decoder_layer, tok_embd: *const c_void, out_norm: *const c_void, lm_head: *const c_void, out: *mut *mut rcu_decoder) -> rcu_status;
    pub fn rcu_decoder_destroy(dec: *mut rcu_decoder);
    pub fn rcu_decoder_set_position(dec: *mut rcu_decoder, position: u32) -> rcu_status;
    pub fn rcu_decoder_position(dec: *const rcu_decoder) -> u32;
    pub fn rcu_decoder_step(dec: *mut rcu_decoder, token_dev: *const i32, logits_dev: *mut c_void, argmax_dev: *mut i32) -> rcu_status;
    pub fn rcu_decoder_kernels_per_step(dec: *const rcu_decoder) -> u32;
    pub fn rcu_decoder_profile_step(dec: *mut rcu_decoder, token_dev: *const i32, logits_dev: *mut c_void, stamps_ns: *mut u64, capacity: u32, n_stamps: *mut u32) -> rcu_status;
    pub fn rcu_attn_decode(dev: *mut rcu_device, qkv: *const c_void, k_cache: *mut c_void, v_cache: *mut c_void, n_heads: u32, n_kv_heads: u32, head_dim: u32, max_cache: u32, rope_dim: u32, rope_base: f32, position: u32, out: *mut c_void) -> rcu_status;
    pub fn rcu_attn_decode_static(dev: *mut rcu_device, qkv: *const c_void, k_cache: *mut c_void, v_cache: *mut c_void, n_heads: u32, n_kv_heads: u32, head_dim: u32, max_cache: u32, rope_dim: u32, rope_base: f32, position: u32, out: *mut c_void) -> rcu_status;
    pub fn rcu_comm_create(dev: *mut rcu_device, rank: c_int, world: c_int, slot_bytes: u64, out: *mut *mut rcu_comm) -> rcu_status;
    pub fn rcu_comm_export(comm: *mut rcu_comm, handle64: *mut c_void) -> rcu_status;
    pub fn rcu_comm_import(comm: *mut rcu_comm, peer: c_int, handle64: *const c_void) -> rcu_status;
    pub fn rcu_comm_import_local(comm: *mut rcu_comm, peer: c_int, other: *mut rcu_comm) -> rcu_status;
    pub fn rcu_comm_destroy(comm: *mut rcu_comm);
    pub fn rcu_comm_rank(comm: *const rcu_comm) -> c_int;
    pub fn rcu_comm_world(comm: *const rcu_comm) -> c_int;
    pub fn rcu_gemv_q8_allgather(comm: *mut rcu_comm, w_shard: *const rcu_tensor, x: *const rcu_tensor, bias_shard: *const rcu_tensor, y_full: *mut *mut c_void) -> rcu_status;
    pub fn rcu_gguf_open(path: *const c_char, out: *mut *mut rcu_gguf) -> rcu_status;
    pub fn rcu_gguf_close(g: *mut rcu_gguf);
    pub fn rcu_gguf_last_error() -> *const c_char;
    pub fn rcu_gguf_version(g: *const rcu_gguf) -> u32;
    pub fn rcu_gguf_tensor_count(g: *const rcu_gguf) -> u64;
    pub fn rcu_gguf_find(g: *const rcu_gguf, name: *const c_char) -> i64;
    pub fn rcu_gguf_tensor(g: *const rcu_gguf, index: u64, out: *mut rcu_gguf_tensor_info) -> rcu_status;
    pub fn rcu_gguf_meta_u64(g: *const rcu_gguf, key: *const c_char, out: *mut u64) -> rcu_status;
    pub fn rcu_gguf_meta_f64(g: *const rcu_gguf, key: *const c_char, out: *mut f64) -> rcu_status;
    pub fn rcu_gguf_meta_str(g: *const rcu_gguf, key: *const c_char, buf: *mut c_char, buf_bytes: u64) -> rcu_status;
    pub fn rcu_gguf_target_dtype(ggml_type: u32, f16_device: c_int) -> i32;
    pub fn rcu_gguf_transcode(g: *const rcu_gguf, index: u64, dt: i32, host_out: *mut c_void, out_bytes: u64) -> rcu_status;
}
