//! `Device::CUDA` for ratchet-core: the three seams a backend has to fill, written against
//! `ratchet-cuda-sys`.
//!
//! UNVERIFIED: written without a Rust toolchain at hand.  The modules mirror, arm for arm, what
//! ratchet-core does for its wgpu device:
//!   * `device`  — `enum Device`, `Device::request_device` (crates/ratchet-core/src/device.rs:25-93)
//!   * `storage` — `enum Storage`, `trait DeviceStorage` (crates/ratchet-core/src/storage/mod.rs:15-132)
//!   * `resolve` — `Tensor::resolve_inner` / `resolve_gpu` (crates/ratchet-core/src/tensor.rs:772-859),
//!                 `Tensor::to` (tensor.rs:949-975), one arm per `LazyOp` as `cpu::apply_operation` has
//!                 (crates/ratchet-core/src/cpu/mod.rs:20-42)
//! Each item says which lines of ratchet-core it is to be spliced into.
pub mod device;
pub mod resolve;
pub mod storage;

pub use device::{CudaDevice, CudaError};
pub use resolve::{CudaOp, CudaTensorRef};
pub use storage::CudaBuffer;
