//! INT8 quantization and quantized linear layers, computed on a B200 through `gpu::cuda`.
//!
//! Drop-in for the CPU implementation: same public types, fields, methods, trait impls and error
//! behaviour.  The host copies of `qweight`/`scales`/`bias` stay populated (tests and user code
//! read them); the device-resident layer rides along as a private, lazily created handle.

use crate::autograd::Tensor;
use crate::error::{EngineError, Result};
use crate::gpu::cuda::{check, ffi, CudaContext, CudaQLinear};
use crate::nn::linear::Linear;
use crate::nn::module::Module;
use crate::tensor::RawTensor;
use std::sync::{Arc, OnceLock};

/// Quantized INT8 multi-dimensional tensor with symmetric scaling.
#[derive(Clone, Debug)]
pub struct Int8Tensor {
    pub data: Vec<i8>,
    pub shape: Vec<usize>,
    pub scale: f32,
}

impl Int8Tensor {
    /// Quantizes a float `RawTensor` into a symmetric `Int8Tensor` (one scale for the tensor).
    /// Infallible like the CPU version; a device failure panics with the library's message.
    pub fn from_raw(raw: &RawTensor) -> Self {
        let slice = raw.to_contiguous();
        let values = slice.as_slice();
        let mut data = vec![0i8; values.len()];
        let mut scale = 1.0f32;
        let ctx = CudaContext::global().expect("CUDA backend unavailable");
        check(unsafe {
            ffi::nne_quantize_tensor(ctx.raw(), values.as_ptr(), values.len(), data.as_mut_ptr(), &mut scale)
        })
        .expect("nne_quantize_tensor failed");
        Self { data, shape: raw.shape().to_vec(), scale }
    }

    /// Dequantizes back to an FP32 `RawTensor`: `q as f32 * scale`.
    pub fn dequantize(&self) -> RawTensor {
        let mut out = vec![0.0f32; self.data.len()];
        let ctx = CudaContext::global().expect("CUDA backend unavailable");
        check(unsafe {
            ffi::nne_dequantize_rows(ctx.raw(), self.data.as_ptr(), &self.scale, 1, self.data.len(), out.as_mut_ptr())
        })
        .expect("nne_dequantize_rows failed");
        RawTensor::from_vec(out, self.shape.clone())
    }

    pub fn memory_bytes(&self) -> usize {
        self.data.len() + std::mem::size_of::<Self>()
    }
}

/// Device state of a `QLinear`: created on first use from the public fields, so a layer built by
/// struct literal or `Clone` works exactly like one from `from_linear`.
#[derive(Debug, Default)]
struct DeviceSlot(OnceLock<std::result::Result<Arc<CudaQLinear>, EngineError>>);

impl Clone for DeviceSlot {
    fn clone(&self) -> Self {
        // A clone owns its own host vectors; its device copy is rebuilt lazily from them.
        DeviceSlot::default()
    }
}

/// Quantized Linear layer storing weights in INT8 with per-row scaling.
#[derive(Clone, Debug)]
pub struct QLinear {
    pub qweight: Vec<i8>,
    pub scales: Vec<f32>,
    pub bias: Option<Vec<f32>>,
    pub in_features: usize,
    pub out_features: usize,
    #[doc(hidden)]
    device: DeviceSlot,
}

impl QLinear {
    /// Quantizes an FP32 `Linear` into an INT8 `QLinear`.  The row loop of the CPU version runs
    /// on the device; codes and scales come back bit-identical.  Infallible: a device failure is
    /// kept and returned as `EngineError::GpuError` by the first `forward`.
    pub fn from_linear(linear: &Linear) -> Self {
        let w_raw = linear.weight.data().to_contiguous();
        let w_slice = w_raw.as_slice();
        let (in_features, out_features) = (linear.in_features, linear.out_features);
        assert_eq!(
            w_slice.len(),
            out_features * in_features,
            "Weight slice length must match out_features * in_features"
        );
        let bias = linear.bias.as_ref().map(|b| b.data().to_contiguous().as_slice().to_vec());
        let mut qweight = vec![0i8; w_slice.len()];
        let mut scales = vec![0.0f32; out_features];
        let slot = DeviceSlot::default();
        let built = CudaContext::global().and_then(|ctx| {
            let dev = CudaQLinear::from_f32(&ctx, w_slice, bias.as_deref(), out_features, in_features)?;
            dev.download(&mut qweight, &mut scales)?;
            Ok(Arc::new(dev))
        });
        let _ = slot.0.set(built);
        Self { qweight, scales, bias, in_features, out_features, device: slot }
    }

    /// Builds a layer from its public fields (a loaded or hand-made set of codes); the device copy
    /// is created from them on first use.  Equivalent to a struct literal in the CPU version.
    pub fn from_parts(qweight: Vec<i8>, scales: Vec<f32>, bias: Option<Vec<f32>>, in_features: usize, out_features: usize) -> Self {
        assert_eq!(qweight.len(), out_features * in_features, "qweight length must match out_features * in_features");
        assert_eq!(scales.len(), out_features, "one scale per output channel");
        Self { qweight, scales, bias, in_features, out_features, device: DeviceSlot::default() }
    }

    fn device(&self) -> Result<&Arc<CudaQLinear>> {
        self.device
            .0
            .get_or_init(|| {
                let ctx = CudaContext::global()?;
                CudaQLinear::from_i8(&ctx, &self.qweight, &self.scales, self.bias.as_deref(), self.out_features, self.in_features)
                    .map(Arc::new)
            })
            .as_ref()
            .map_err(|e| e.clone())
    }

    /// y = x W^T (int8, per-row scales) + b.  Input `[.., in_features]` with at least 2 dims.
    pub fn forward_quantized(&self, input: &Tensor) -> Result<Tensor> {
        let in_shape = input.shape();
        let ndim = in_shape.len();
        if ndim < 2 {
            return Err(EngineError::InvalidArgument(format!(
                "QLinear forward expects tensor with at least 2 dimensions, got {:?}",
                in_shape
            )));
        }
        let in_k = in_shape[ndim - 1];
        if in_k != self.in_features {
            return Err(EngineError::ShapeMismatch { expected: vec![self.in_features], actual: vec![in_k] });
        }
        let num_rows: usize = in_shape[..ndim - 1].iter().product();
        let input_contig = input.data().to_contiguous();
        let mut out_shape = in_shape.to_vec();
        out_shape[ndim - 1] = self.out_features;
        let mut out_data = vec![0.0f32; num_rows * self.out_features];
        self.device()?.forward(input_contig.as_slice(), num_rows, in_k, &mut out_data)?;
        Ok(Tensor::new(RawTensor::from_vec(out_data, out_shape), false))
    }

    /// Dequantizes the INT8 weights back into a standard FP32 `Linear` layer.
    pub fn to_linear(&self) -> Linear {
        let mut w = vec![0.0f32; self.qweight.len()];
        let ctx = CudaContext::global().expect("CUDA backend unavailable");
        check(unsafe {
            ffi::nne_dequantize_rows(ctx.raw(), self.qweight.as_ptr(), self.scales.as_ptr(), self.out_features, self.in_features, w.as_mut_ptr())
        })
        .expect("nne_dequantize_rows failed");
        let weight = Tensor::new(RawTensor::from_vec(w, vec![self.out_features, self.in_features]), true);
        let bias = self.bias.as_ref().map(|b| Tensor::new(RawTensor::from_vec(b.clone(), vec![self.out_features]), true));
        Linear { weight, bias, in_features: self.in_features, out_features: self.out_features }
    }

    pub fn memory_bytes(&self) -> usize {
        self.qweight.len()
            + self.scales.len() * std::mem::size_of::<f32>()
            + self.bias.as_ref().map_or(0, |b| b.len() * std::mem::size_of::<f32>())
    }
}

impl Module for QLinear {
    fn forward(&self, input: &Tensor) -> Result<Tensor> {
        self.forward_quantized(input)
    }

    fn parameters(&self) -> Vec<Tensor> {
        Vec::new()
    }
}
