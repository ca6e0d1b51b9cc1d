//! Owner of one device-resident int8 layer (`nne_qlinear*`).
use super::{check, ffi, CudaContext};
use crate::error::Result;
use std::sync::Arc;

#[derive(Debug)]
pub struct CudaQLinear {
    raw: *mut ffi::nne_qlinear,
    _ctx: Arc<CudaContext>, // keeps the context alive as long as the layer
}

// The handle is immutable after creation; forwards on it are serialised by the library.
unsafe impl Send for CudaQLinear {}
unsafe impl Sync for CudaQLinear {}

impl CudaQLinear {
    /// Upload an f32 weight `[n, k]` (and bias) and quantize it on the device.
    pub fn from_f32(ctx: &Arc<CudaContext>, w: &[f32], bias: Option<&[f32]>, n: usize, k: usize) -> Result<Self> {
        let mut raw = std::ptr::null_mut();
        let b = bias.map_or(std::ptr::null(), |b| b.as_ptr());
        check(unsafe { ffi::nne_qlinear_create_from_f32(ctx.raw(), w.as_ptr(), b, n, k, &mut raw) })?;
        Ok(Self { raw, _ctx: ctx.clone() })
    }

    /// Build the device layer from existing codes and scales (a cloned or hand-built `QLinear`).
    pub fn from_i8(ctx: &Arc<CudaContext>, q: &[i8], scales: &[f32], bias: Option<&[f32]>, n: usize, k: usize) -> Result<Self> {
        let mut raw = std::ptr::null_mut();
        let b = bias.map_or(std::ptr::null(), |b| b.as_ptr());
        check(unsafe { ffi::nne_qlinear_create_from_i8(ctx.raw(), q.as_ptr(), scales.as_ptr(), b, n, k, &mut raw) })?;
        Ok(Self { raw, _ctx: ctx.clone() })
    }

    pub(crate) fn raw(&self) -> *mut ffi::nne_qlinear {
        self.raw
    }

    /// Copy codes and scales back into the host fields of `QLinear`.
    pub fn download(&self, q: &mut [i8], scales: &mut [f32]) -> Result<()> {
        check(unsafe { ffi::nne_qlinear_download(self.raw, q.as_mut_ptr(), scales.as_mut_ptr()) })
    }

    /// y[m, n] = x[m, k] . q^T * scales (+ bias); host buffers.
    pub fn forward(&self, x: &[f32], m: usize, k: usize, y: &mut [f32]) -> Result<()> {
        check(unsafe { ffi::nne_qlinear_forward_host(self.raw, x.as_ptr(), m, k, y.as_mut_ptr()) })
    }
}

impl Drop for CudaQLinear {
    fn drop(&mut self) {
        unsafe { ffi::nne_qlinear_destroy(self.raw) };
    }
}
