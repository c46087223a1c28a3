//! The device arm.
//!
//! In ratchet-core (crates/ratchet-core/src/device.rs):
//! ```ignore
//! pub enum DeviceRequest { CPU, GPU, CUDA(i32) }                       // :25-28, new variant
//! pub enum Device { CPU, GPU(WgpuDevice), CUDA(CudaDevice) }           // :30-35, new variant
//! Device::request_device: DeviceRequest::CUDA(o) => Ok(Device::CUDA(CudaDevice::new(o)?)),   // :70-78
//! Device::compute_precision: Device::CUDA(_) => DType::F16,           // :57-62 (sm_100 has native f16)
//! Device::try_cuda(&self) -> Result<&CudaDevice, DeviceError>          // beside try_gpu, :84-92
//! DeviceError::Cuda(#[from] CudaError)                                 // :6-23, new variant
//! ```
use std::ffi::CStr;
use std::sync::Arc;

use ratchet_cuda_sys as sys;

#[derive(Clone, Debug, thiserror::Error)]
pub enum CudaError {
    #[error("invalid argument: {0}")]
    InvalidArg(String),
    #[error("no kernel for this dtype / shape combination: {0}")]
    Unsupported(String),
    #[error("device allocation failed: {0}")]
    OutOfMemory(String),
    #[error("CUDA runtime error: {0}")]
    Runtime(String),
    #[error("a bounded device-side wait gave up: {0}")]
    Timeout(String),
    #[error("index outside a tensor: {0}")]
    Bounds(String),
    #[error("the op was asked to run in place and cannot: {0}")]
    Inplace(String),
}

/// Owns one `rcu_device` (a CUDA device ordinal plus the stream every launch goes to).
struct Handle(*mut sys::rcu_device);

// ratchet-core's `Tensor` is `Send` (tensor.rs:49); one thread drives a device at a time, which is all
// the C ABI asks for.
unsafe impl Send for Handle {}
unsafe impl Sync for Handle {}

impl Drop for Handle {
    fn drop(&mut self) {
        unsafe { sys::rcu_device_destroy(self.0) }
    }
}

/// Counterpart of `WgpuDevice` (gpu/device.rs:18-119): cheap to clone, compared by ordinal.
#[derive(Clone)]
pub struct CudaDevice {
    handle: Arc<Handle>,
    ordinal: i32,
}

impl std::fmt::Debug for CudaDevice {
    fn fmt(&self, f: &mut std::fmt::Formatter<'_>) -> std::fmt::Result {
        write!(f, "CUDA:{}", self.ordinal)
    }
}

impl PartialEq for CudaDevice {
    fn eq(&self, other: &Self) -> bool {
        self.ordinal == other.ordinal
    }
}

impl CudaDevice {
    /// `WgpuDevice::new` (gpu/device.rs:32-78).  Fails without an sm_100 GPU: there is no fallback.
    pub fn new(ordinal: i32) -> Result<Self, CudaError> {
        let mut raw: *mut sys::rcu_device = std::ptr::null_mut();
        let st = unsafe { sys::rcu_device_create(ordinal, &mut raw) };
        if st != sys::RCU_OK || raw.is_null() {
            return Err(CudaError::Runtime(format!("cannot open CUDA device {ordinal} (status {st})")));
        }
        Ok(Self { handle: Arc::new(Handle(raw)), ordinal })
    }

    pub fn ordinal(&self) -> i32 {
        self.ordinal
    }

    pub fn raw(&self) -> *mut sys::rcu_device {
        self.handle.0
    }

    /// Turns a status into a `Result`, attaching the device's message for the failing call.
    pub fn check(&self, st: sys::rcu_status) -> Result<(), CudaError> {
        if st == sys::RCU_OK {
            return Ok(());
        }
        let msg = unsafe {
            let p = sys::rcu_last_error(self.raw());
            if p.is_null() { String::new() } else { CStr::from_ptr(p).to_string_lossy().into_owned() }
        };
        Err(match st {
            sys::RCU_ERR_INVALID_ARG => CudaError::InvalidArg(msg),
            sys::RCU_ERR_UNSUPPORTED => CudaError::Unsupported(msg),
            sys::RCU_ERR_OOM => CudaError::OutOfMemory(msg),
            sys::RCU_ERR_TIMEOUT => CudaError::Timeout(msg),
            sys::RCU_ERR_BOUNDS => CudaError::Bounds(msg),
            sys::RCU_ERR_INPLACE => CudaError::Inplace(msg),
            _ => CudaError::Runtime(msg),
        })
    }

    /// `device.poll(Wait)` at the end of `resolve_gpu` (tensor.rs:856).
    pub fn sync(&self) -> Result<(), CudaError> {
        self.check(unsafe { sys::rcu_sync(self.raw()) })
    }

    /// `WgpuDevice::begin_pass` (gpu/device.rs:104-107): hand cached blocks nobody took back to the driver.
    pub fn trim_pool(&self) -> Result<(), CudaError> {
        self.check(unsafe { sys::rcu_pool_trim(self.raw()) })
    }
}
