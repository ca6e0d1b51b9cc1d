//! `CudaTensor`: an f32 tensor in device memory, the counterpart of the wgpu backend's `GpuTensor`
//! (`src/gpu/tensor.rs:12-100`): `from_slice` / `from_raw` upload, `to_cpu` downloads, and nothing
//! crosses PCIe in between.
use super::{check, ffi, CudaContext};
use crate::error::{EngineError, Result};
use crate::tensor::RawTensor;
use std::os::raw::c_void;
use std::sync::Arc;

/// Owner of one device allocation; freed on drop.
#[derive(Debug)]
pub(crate) struct DeviceBuffer {
    pub(crate) ptr: *mut c_void,
    ctx: Arc<CudaContext>,
}

unsafe impl Send for DeviceBuffer {}
unsafe impl Sync for DeviceBuffer {}

impl DeviceBuffer {
    pub(crate) fn new(ctx: &Arc<CudaContext>, bytes: usize) -> Result<Self> {
        let mut ptr = std::ptr::null_mut();
        check(unsafe { ffi::nne_device_alloc(ctx.raw(), bytes, &mut ptr) })?;
        Ok(Self { ptr, ctx: ctx.clone() })
    }
}

impl Drop for DeviceBuffer {
    fn drop(&mut self) {
        unsafe { ffi::nne_device_free(self.ctx.raw(), self.ptr) };
    }
}

/// A multi-dimensional f32 tensor stored in device memory.
#[derive(Clone, Debug)]
pub struct CudaTensor {
    pub(crate) buffer: Arc<DeviceBuffer>,
    pub shape: Vec<usize>,
    pub ctx: Arc<CudaContext>,
}

impl CudaTensor {
    /// Uninitialised tensor of the given shape.
    pub fn empty(shape: &[usize], ctx: &Arc<CudaContext>) -> Result<Self> {
        let n: usize = shape.iter().product();
        let buffer = Arc::new(DeviceBuffer::new(ctx, n * std::mem::size_of::<f32>())?);
        Ok(Self { buffer, shape: shape.to_vec(), ctx: ctx.clone() })
    }

    /// Creates a tensor from a host slice and shape (`GpuTensor::from_slice`).
    pub fn from_slice(slice: &[f32], shape: &[usize], ctx: &Arc<CudaContext>) -> Result<Self> {
        let expected: usize = shape.iter().product();
        if slice.len() != expected {
            return Err(EngineError::IncompatibleShapes {
                op: "CudaTensor::from_slice",
                shapes: vec![vec![slice.len()], shape.to_vec()],
            });
        }
        let t = Self::empty(shape, ctx)?;
        check(unsafe {
            ffi::nne_device_upload(ctx.raw(), t.buffer.ptr, slice.as_ptr() as *const c_void, std::mem::size_of_val(slice))
        })?;
        Ok(t)
    }

    /// Uploads a host `RawTensor` (`GpuTensor::from_raw`).
    pub fn from_raw(raw: &RawTensor, ctx: &Arc<CudaContext>) -> Result<Self> {
        let contig = raw.to_contiguous();
        Self::from_slice(contig.as_slice(), contig.shape(), ctx)
    }

    /// Downloads the tensor (`GpuTensor::to_cpu`): waits for the device, then copies.
    pub fn to_cpu(&self) -> Result<RawTensor> {
        let n: usize = self.shape.iter().product();
        let mut out = vec![0.0f32; n];
        check(unsafe {
            ffi::nne_device_download(self.ctx.raw(), out.as_mut_ptr() as *mut c_void, self.buffer.ptr, n * std::mem::size_of::<f32>())
        })?;
        Ok(RawTensor::from_vec(out, self.shape.clone()))
    }

    pub fn shape(&self) -> &[usize] {
        &self.shape
    }

    pub(crate) fn as_ptr(&self) -> *const f32 {
        self.buffer.ptr as *const f32
    }

    pub(crate) fn as_mut_ptr(&self) -> *mut f32 {
        self.buffer.ptr as *mut f32
    }
}
