//! The resolve arm.
//!
//! In ratchet-core (crates/ratchet-core/src/tensor.rs):
//! ```ignore
//! fn resolve_inner(self, debug: bool) -> Result<Tensor, TensorError> {             // :772-777
//!     match self.device().clone() {
//!         Device::CPU => self.resolve_cpu(),
//!         Device::GPU(device) => self.resolve_gpu(&device, debug),
//!         Device::CUDA(device) => self.resolve_cuda(&device),
//!     }
//! }
//! fn resolve_cuda(self, device: &CudaDevice) -> Result<Tensor, TensorError> {
//!     let order = self.execution_order();                                            // :696-740
//!     let mut allocations = device.allocate_cfg(&order)?;   // liveness + greedy by size, as allocator.rs:141-340
//!     for t in order.iter() {
//!         if t.resolved() { continue; }
//!         t.update_storage(Storage::CUDA(allocations.remove(&t.id()).ok_or(TensorError::NoStorage(t.id()))?));
//!         let can_inplace = t.op().supports_inplace() && t.op().srcs()[0].strong_count() == 1;   // :823-824
//!         ratchet_cuda::resolve::run(device, &CudaOp::from_lazy(t.op(), can_inplace)?, &refs_of(t.op().srcs()), &ref_of(t))?;
//!     }
//!     device.sync()?;                                                                // :856
//!     Ok(self)
//! }
//! Tensor::to: (Device::CUDA(_), Device::CPU) => self.cuda_to_cpu(), (Device::CPU, Device::CUDA(_)) => self.to_cuda(device)   // :949-975
//! ```
//! `CudaOp::from_lazy` is the one function that needs ratchet-core's op structs (their fields are
//! `pub(crate)`): it belongs inside ratchet-core next to `cpu::apply_operation` (cpu/mod.rs:20-38) and is
//! a match with one arm per `LazyOp` variant, each reading the same fields the CPU arm reads.
//!
//! Alternatively the whole graph can be handed over: `rcu_lazy_*` builds the same DAG on the library's
//! side and `rcu_lazy_resolve` orders, plans and runs it (one FFI call per node at build time, none at
//! run time).
use std::os::raw::c_void;

use ratchet_cuda_sys as sys;

use crate::device::{CudaDevice, CudaError};

/// What `run` needs to know about a resolved tensor: dtype, shape, device pointer
/// (`StorageView` + `Storage::CUDA`, tensor.rs:131-151).
#[derive(Clone, Copy, Debug)]
pub struct CudaTensorRef {
    pub dt: i32,
    pub rank: u32,
    pub shape: [u64; 4],
    pub data: *mut c_void,
}

impl CudaTensorRef {
    fn raw(&self) -> sys::rcu_tensor {
        sys::rcu_tensor { dt: self.dt, rank: self.rank, shape: self.shape, data: self.data }
    }
}

/// One variant per `LazyOp` variant that launches something (op.rs:12-31); `Const` and `View` launch
/// nothing (`compile_gpu` returns `None` for them, tensor.rs:763-764).
#[derive(Clone, Debug)]
pub enum CudaOp {
    /// `Binary` (ops/binary.rs:19-45): lhs, rhs
    Binary { op: i32 },
    /// `Unary` (ops/unary.rs:23-60)
    Unary { op: i32 },
    /// `Cast` (ops/cast.rs:15-30): the destination dtype is the output tensor's
    Cast,
    /// `Matmul` (ops/matmul/mod.rs:381-390): lhs, rhs, optional bias
    Matmul { trans_lhs: bool, trans_rhs: bool, trans_dst: bool, has_bias: bool },
    /// `NormOp` (ops/norm/mod.rs:18-60): x, scale, optional bias
    Norm { kind: i32, eps: f32, groups: u32, has_bias: bool },
    /// `Softmax` (ops/softmax.rs:15-25)
    Softmax { dim: u32 },
    /// `RoPE` (ops/rope.rs:16-30)
    RoPE { dim: u32, base: f32, offset: u32 },
    /// `Concat` (ops/concat.rs:14-25): up to eight inputs
    Concat { dim: u32 },
    /// `IndexSelect` (ops/select.rs:14-25): table, ids
    Select { dim: u32 },
    /// `Reindex::Permute` / `Slice` / `Broadcast` (ops/reindex/*.rs)
    Permute { perm: [u32; 4] },
    Slice { start: [u64; 4], stop: [u64; 4] },
    Broadcast,
    /// `Cache` (ops/cache.rs:25-40): cache, source
    Cache { dim: u32, offset: u32 },
    /// `IndexWrite` (ops/index_write.rs:15-30): destination (= srcs[0], in place), source
    IndexWrite { start: [u64; 4] },
    /// `Conv` (ops/conv.rs:16-30): x, weight, bias
    Conv { stride: u32, padding: u32 },
}

/// `cpu::apply_operation` / `CPUOperation::apply_cpu` for the CUDA device: launches the kernel(s) of one
/// node into `dst` (already allocated by the caller, as on every ratchet device).  Asynchronous on the
/// device's stream.
pub fn run(device: &CudaDevice, op: &CudaOp, srcs: &[CudaTensorRef], dst: &CudaTensorRef) -> Result<(), CudaError> {
    let dev = device.raw();
    let mut d = dst.raw();
    let s: Vec<sys::rcu_tensor> = srcs.iter().map(|t| t.raw()).collect();
    let need = |n: usize| -> Result<(), CudaError> {
        if s.len() < n { Err(CudaError::InvalidArg(format!("{op:?} takes {n} sources, got {}", s.len()))) } else { Ok(()) }
    };
    let opt = |i: usize, present: bool| -> *const sys::rcu_tensor { if present { &s[i] } else { std::ptr::null() } };
    let st = unsafe {
        match op {
            CudaOp::Binary { op: o } => { need(2)?; sys::rcu_binary(dev, *o, &s[0], &s[1], &mut d) }
            CudaOp::Unary { op: o } => { need(1)?; sys::rcu_unary(dev, *o, &s[0], &mut d) }
            CudaOp::Cast => { need(1)?; sys::rcu_cast(dev, &s[0], &mut d) }
            CudaOp::Matmul { trans_lhs, trans_rhs, trans_dst, has_bias } => {
                need(if *has_bias { 3 } else { 2 })?;
                sys::rcu_matmul(dev, &s[0], &s[1], opt(2, *has_bias), *trans_lhs as i32, *trans_rhs as i32, *trans_dst as i32, &mut d)
            }
            CudaOp::Norm { kind, eps, groups, has_bias } => {
                need(if *has_bias { 3 } else { 2 })?;
                sys::rcu_norm(dev, *kind, &s[0], &s[1], opt(2, *has_bias), *eps, *groups, &mut d)
            }
            CudaOp::Softmax { dim } => { need(1)?; sys::rcu_softmax(dev, &s[0], *dim, &mut d) }
            CudaOp::RoPE { dim, base, offset } => { need(1)?; sys::rcu_rope(dev, &s[0], *dim, *base, *offset, &mut d) }
            CudaOp::Concat { dim } => {
                need(1)?;
                let ptrs: Vec<*const sys::rcu_tensor> = s.iter().map(|t| t as *const _).collect();
                sys::rcu_concat(dev, ptrs.as_ptr(), ptrs.len() as u32, *dim, &mut d)
            }
            CudaOp::Select { dim } => { need(2)?; sys::rcu_index_select(dev, &s[0], &s[1], *dim, &mut d) }
            CudaOp::Permute { perm } => { need(1)?; sys::rcu_permute(dev, &s[0], perm.as_ptr(), &mut d) }
            CudaOp::Slice { start, stop } => { need(1)?; sys::rcu_slice(dev, &s[0], start.as_ptr(), stop.as_ptr(), &mut d) }
            CudaOp::Broadcast => { need(1)?; sys::rcu_broadcast(dev, &s[0], &mut d) }
            CudaOp::Cache { dim, offset } => {
                need(2)?;
                let mut cache = s[0];
                sys::rcu_cache(dev, &mut cache, &s[1], *dim, *offset, &mut d)
            }
            CudaOp::IndexWrite { start } => { need(2)?; sys::rcu_index_write(dev, &mut d, &s[1], start.as_ptr()) }
            CudaOp::Conv { stride, padding } => { need(3)?; sys::rcu_conv1d(dev, &s[0], &s[1], &s[2], *stride, *padding, &mut d) }
        }
    };
    device.check(st)
}

/// `Matmul::compute_dst_shape` (ops/matmul/mod.rs:392-466) through the library: no device work.
pub fn matmul_dst_shape(lhs: &CudaTensorRef, rhs: &CudaTensorRef, trans_lhs: bool, trans_rhs: bool, trans_dst: bool) -> Option<(u32, [u64; 4])> {
    let mut d = sys::rcu_tensor { dt: 0, rank: 0, shape: [1; 4], data: std::ptr::null_mut() };
    let st = unsafe { sys::rcu_matmul_dst_shape(&lhs.raw(), &rhs.raw(), trans_lhs as i32, trans_rhs as i32, trans_dst as i32, &mut d) };
    if st == sys::RCU_OK { Some((d.rank, d.shape)) } else { None }
}
