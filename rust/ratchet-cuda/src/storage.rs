//! The storage arm.
//!
//! In ratchet-core (crates/ratchet-core/src/storage/mod.rs):
//! ```ignore
//! pub enum Storage { CPU(CPUBuffer), GPU(GPUBuffer), CUDA(CudaBuffer) }                    // :15-19
//! Storage::from_quantized / zeros / from_slice / from_bytes: Device::CUDA(d) => Storage::CUDA(CudaBuffer::from_bytes(bytes, d)?)   // :25-63
//! Storage::deep_clone: Storage::CUDA(c) => Ok(Storage::CUDA(c.deep_clone()?))             // :106-117
//! impl DeviceStorage for CudaBuffer { to_device, to_cpu, n_bytes, dump }                   // :122-132
//! ```
//! `CPUBuffer::to_device` (storage/cpu_buffer.rs:126-147) gains the mirror arm
//! `Device::CUDA(d) => CudaBuffer::from_bytes(self.inner().as_bytes(), d)`.
use std::os::raw::c_void;

use ratchet_cuda_sys as sys;

use crate::device::{CudaDevice, CudaError};

/// Counterpart of `GPUBuffer` (storage/gpu_buffer.rs:19-60): a block of the device's caching pool.
/// Quantised tensors are ONE buffer holding ratchet's segments back to back, each padded to 256 bytes
/// (dtype/blocks.rs:69-82,124-148) — exactly the bytes `Tensor::from_quantized` already holds.
#[derive(Debug)]
pub struct CudaBuffer {
    ptr: *mut c_void,
    n_bytes: usize,
    device: CudaDevice,
}

unsafe impl Send for CudaBuffer {}
unsafe impl Sync for CudaBuffer {}

impl Drop for CudaBuffer {
    fn drop(&mut self) {
        // the pool reuses the block in stream order; nothing to wait for
        unsafe { sys::rcu_free(self.device.raw(), self.ptr) };
    }
}

impl CudaBuffer {
    /// Uninitialised block of `n_bytes` (what `allocate_cfg` hands `resolve_gpu` per tensor, tensor.rs:817-821).
    pub fn alloc(n_bytes: usize, device: &CudaDevice) -> Result<Self, CudaError> {
        let mut ptr: *mut c_void = std::ptr::null_mut();
        device.check(unsafe { sys::rcu_alloc(device.raw(), n_bytes as u64, &mut ptr) })?;
        Ok(Self { ptr, n_bytes, device: device.clone() })
    }

    /// `GPUBuffer::from_bytes` (storage/gpu_buffer.rs:49-60).
    pub fn from_bytes(bytes: &[u8], device: &CudaDevice) -> Result<Self, CudaError> {
        let buf = Self::alloc(bytes.len().max(16), device)?;      // MIN_STORAGE_BUFFER_SIZE
        device.check(unsafe { sys::rcu_h2d(device.raw(), buf.ptr, bytes.as_ptr() as *const c_void, bytes.len() as u64) })?;
        // pageable source: rcu_h2d returns once it has been read
        Ok(buf)
    }

    /// `GPUBuffer::zeros` (storage/gpu_buffer.rs:36-47).
    pub fn zeros(n_bytes: usize, device: &CudaDevice) -> Result<Self, CudaError> {
        let buf = Self::alloc(n_bytes.max(16), device)?;
        device.check(unsafe { sys::rcu_memset(device.raw(), buf.ptr, 0, buf.n_bytes as u64) })?;
        Ok(buf)
    }

    /// `GPUBuffer::deep_clone` (storage/gpu_buffer.rs:152-170).
    pub fn deep_clone(&self) -> Result<Self, CudaError> {
        let out = Self::alloc(self.n_bytes, &self.device)?;
        self.device.check(unsafe { sys::rcu_d2d(self.device.raw(), out.ptr, self.ptr, self.n_bytes as u64) })?;
        Ok(out)
    }

    /// `DeviceStorage::to_cpu` (storage/gpu_buffer.rs:200-218): blocking copy; the caller wraps the bytes
    /// in a `CPUBuffer::from_bytes(&bytes, alignment)`.
    pub fn to_cpu_bytes(&self) -> Result<Vec<u8>, CudaError> {
        let mut out = vec![0u8; self.n_bytes];
        self.device.check(unsafe { sys::rcu_d2h(self.device.raw(), out.as_mut_ptr() as *mut c_void, self.ptr, self.n_bytes as u64) })?;
        Ok(out)
    }

    pub fn n_bytes(&self) -> usize {
        self.n_bytes
    }

    pub fn as_ptr(&self) -> *mut c_void {
        self.ptr
    }

    pub fn device(&self) -> &CudaDevice {
        &self.device
    }
}
