//! CUDA (B200, sm_100a) device backend for the quantized-linear path.
//!
//! Mirrors the conventions of the wgpu backend next to it (`src/gpu/layers.rs:12-57`): an
//! `Arc`-shared context, device failures reported as `EngineError::GpuError(String)`.  There is
//! no CPU fallback: if the library cannot reach an sm_100 device every call returns `GpuError`.
pub mod ffi;
pub mod layers;
pub mod qlinear;
pub mod tensor;

use crate::error::{EngineError, Result};
use std::ffi::CStr;
use std::os::raw::{c_char, c_int};
use std::sync::{Arc, OnceLock};

pub use layers::{CudaPlan, CudaQLinearLayer, PlanItem, ToCuda};
pub use qlinear::CudaQLinear;
pub use tensor::CudaTensor;

/// Text of the calling thread's last library error.
fn last_error() -> String {
    let mut buf = [0 as c_char; 512];
    unsafe {
        ffi::nne_last_error(buf.as_mut_ptr(), buf.len());
        CStr::from_ptr(buf.as_ptr()).to_string_lossy().into_owned()
    }
}

/// Status code -> the reference's error enum (`src/error.rs:10-52`).
pub(crate) fn check(status: c_int) -> Result<()> {
    match status {
        ffi::NNE_OK => Ok(()),
        ffi::NNE_ERR_INVALID_ARGUMENT => Err(EngineError::InvalidArgument(last_error())),
        // The caller knows both shapes and rebuilds ShapeMismatch itself; this arm is a backstop.
        ffi::NNE_ERR_SHAPE_MISMATCH => Err(EngineError::InvalidArgument(last_error())),
        _ => Err(EngineError::GpuError(last_error())),
    }
}

/// One device context, shared by every layer placed on that device.
#[derive(Debug)]
pub struct CudaContext {
    raw: *mut ffi::nne_ctx,
    pub device: i32,
    pub sm_count: i32,
}

// The library serialises host-pointer calls on a per-context mutex and device handles are
// immutable after creation, so the context may be shared between threads.
unsafe impl Send for CudaContext {}
unsafe impl Sync for CudaContext {}

impl CudaContext {
    pub fn new(device: i32) -> Result<Arc<Self>> {
        let mut raw = std::ptr::null_mut();
        check(unsafe { ffi::nne_cuda_ctx_create(device, &mut raw) })?;
        let (mut dev, mut sms) = (0, 0);
        check(unsafe {
            ffi::nne_cuda_ctx_info(
                raw,
                &mut dev,
                &mut sms,
                std::ptr::null_mut(),
                std::ptr::null_mut(),
                std::ptr::null_mut(),
            )
        })?;
        Ok(Arc::new(Self { raw, device: dev, sm_count: sms }))
    }

    /// Process-wide default context on the device named by `NNE_CUDA_DEVICE` (default 0).
    pub fn global() -> Result<Arc<Self>> {
        static CTX: OnceLock<std::result::Result<Arc<CudaContext>, EngineError>> = OnceLock::new();
        CTX.get_or_init(|| {
            let dev = std::env::var("NNE_CUDA_DEVICE").ok().and_then(|s| s.parse().ok()).unwrap_or(0);
            CudaContext::new(dev)
        })
        .clone()
    }

    pub(crate) fn raw(&self) -> *mut ffi::nne_ctx {
        self.raw
    }
}

impl Drop for CudaContext {
    fn drop(&mut self) {
        unsafe { ffi::nne_cuda_ctx_destroy(self.raw) };
    }
}
