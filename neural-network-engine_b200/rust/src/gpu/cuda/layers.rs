//! Device-resident layers of the CUDA backend and the `ToGpu` conversions, after the wgpu
//! backend's `src/gpu/layers.rs:12-57` (`ToGpu`, `GpuLinear`).
use super::tensor::CudaTensor;
use super::{check, ffi, CudaContext, CudaQLinear};
use crate::error::{EngineError, Result};
use crate::nn::quantized::QLinear;
use crate::tensor::RawTensor;
use std::sync::Arc;

/// Places a host object on a CUDA device (the shape of `gpu::layers::ToGpu`, with this backend's
/// context type).
pub trait ToCuda {
    type Target;
    fn to_cuda(&self, ctx: &Arc<CudaContext>) -> Result<Self::Target>;
}

impl ToCuda for RawTensor {
    type Target = CudaTensor;
    fn to_cuda(&self, ctx: &Arc<CudaContext>) -> Result<CudaTensor> {
        CudaTensor::from_raw(self, ctx)
    }
}

/// `QLinear` on the device: forwards take and return `CudaTensor`s and are asynchronous on the
/// context's stream; nothing is copied to the host until `CudaTensor::to_cpu`.
pub struct CudaQLinearLayer {
    pub in_features: usize,
    pub out_features: usize,
    inner: Arc<CudaQLinear>,
    ctx: Arc<CudaContext>,
}

impl CudaQLinearLayer {
    /// y[.., out] = x[.., in] . q^T * scales (+ bias), same checks as `QLinear::forward_quantized`.
    pub fn forward(&self, input: &CudaTensor) -> Result<CudaTensor> {
        let shape = input.shape();
        let ndim = shape.len();
        if ndim < 2 {
            return Err(EngineError::InvalidArgument(format!(
                "QLinear forward expects tensor with at least 2 dimensions, got {:?}",
                shape
            )));
        }
        let k = shape[ndim - 1];
        if k != self.in_features {
            return Err(EngineError::ShapeMismatch { expected: vec![self.in_features], actual: vec![k] });
        }
        let m: usize = shape[..ndim - 1].iter().product();
        let mut out_shape = shape.to_vec();
        out_shape[ndim - 1] = self.out_features;
        let out = CudaTensor::empty(&out_shape, &self.ctx)?;
        let stream = unsafe { ffi::nne_cuda_ctx_stream(self.ctx.raw()) };
        check(unsafe { ffi::nne_qlinear_forward_dev(self.inner.raw(), input.as_ptr(), m, k, out.as_mut_ptr(), stream) })?;
        Ok(out)
    }

    pub(crate) fn raw(&self) -> *mut ffi::nne_qlinear {
        self.inner.raw()
    }
}

impl ToCuda for QLinear {
    type Target = CudaQLinearLayer;
    /// The layer's codes already live on the device when `ctx` is the process-wide context it was
    /// built on; another context receives its own copy of codes, scales and bias.
    fn to_cuda(&self, ctx: &Arc<CudaContext>) -> Result<CudaQLinearLayer> {
        let inner = Arc::new(CudaQLinear::from_i8(
            ctx,
            &self.qweight,
            &self.scales,
            self.bias.as_deref(),
            self.out_features,
            self.in_features,
        )?);
        Ok(CudaQLinearLayer { in_features: self.in_features, out_features: self.out_features, inner, ctx: ctx.clone() })
    }
}

/// Several forwards on fixed device tensors issued together (`nne_qlinear_plan_*`): q/k/v or
/// gate/up of a LLaMA block (`src/models/llama.rs:226-228,344-346`) as one launch at batch 1, with
/// RMSNorm / SiLU-mul / residual taken in the forwards' stride when items ask for them.  Items may
/// read tensors that earlier items of the same plan write (`y` of one as `x`, `silu_mul` or
/// `residual` of a later one): the library orders them, and at batch 1 a whole decoder block - or
/// every block between two attention calls - still is one launch.
pub struct CudaPlan {
    raw: *mut ffi::nne_plan,
    _keep: Vec<CudaTensor>, // inputs and outputs stay alive as long as the plan
    ctx: Arc<CudaContext>,
}

unsafe impl Send for CudaPlan {}

/// One forward of a `CudaPlan`.
pub struct PlanItem<'a> {
    pub layer: &'a CudaQLinearLayer,
    pub x: &'a CudaTensor,
    pub y: &'a CudaTensor,
    /// `Some((gamma, eps))`: the layer reads `RMSNorm(x)` (`src/nn/norm.rs:100-180`).
    pub rmsnorm: Option<(&'a CudaTensor, f32)>,
    /// `Some(up)`: the layer reads `silu(x) * up` (`src/models/llama.rs:343-346`).
    pub silu_mul: Option<&'a CudaTensor>,
    /// `Some(r)`: `y = forward + r`.
    pub residual: Option<&'a CudaTensor>,
}

impl CudaPlan {
    pub fn new(ctx: &Arc<CudaContext>, items: &[PlanItem<'_>], m: usize) -> Result<Self> {
        let mut raw_items = Vec::with_capacity(items.len());
        let mut keep = Vec::new();
        for it in items {
            let (op, gamma, eps) = match it.rmsnorm {
                Some((g, e)) => (ffi::NNE_INPUT_RMSNORM, g.as_ptr(), e),
                None if it.silu_mul.is_some() => (ffi::NNE_INPUT_SILU_MUL, std::ptr::null(), 0.0),
                None => (ffi::NNE_INPUT_PLAIN, std::ptr::null(), 0.0),
            };
            raw_items.push(ffi::nne_plan_item {
                layer: it.layer.raw(),
                x: it.x.as_ptr(),
                y: it.y.as_mut_ptr(),
                input_op: op,
                eps,
                gamma,
                x2: it.silu_mul.map_or(std::ptr::null(), |t| t.as_ptr()),
                residual: it.residual.map_or(std::ptr::null(), |t| t.as_ptr()),
            });
            keep.push(it.x.clone());
            keep.push(it.y.clone());
            for t in [it.rmsnorm.map(|p| p.0), it.silu_mul, it.residual].into_iter().flatten() {
                keep.push(t.clone());
            }
        }
        let mut raw = std::ptr::null_mut();
        check(unsafe { ffi::nne_qlinear_plan_create_fused(ctx.raw(), raw_items.len(), raw_items.as_ptr(), m, &mut raw) })?;
        Ok(Self { raw, _keep: keep, ctx: ctx.clone() })
    }

    /// Issues all forwards on the context's stream (asynchronous).
    pub fn run(&self) -> Result<()> {
        let stream = unsafe { ffi::nne_cuda_ctx_stream(self.ctx.raw()) };
        check(unsafe { ffi::nne_qlinear_plan_run(self.raw, stream) })
    }

    pub fn launches(&self) -> i32 {
        unsafe { ffi::nne_qlinear_plan_launches(self.raw) }
    }
}

impl Drop for CudaPlan {
    fn drop(&mut self) {
        unsafe { ffi::nne_qlinear_plan_destroy(self.raw) };
    }
}
