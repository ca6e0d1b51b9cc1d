//! SafeTensors save/load for `QLinear`: `I8` codes plus `F32` scales and bias.
//!
//! `src/io/safetensors.rs` writes and accepts `F32` only (its loader rejects every other dtype,
//! `:68-74`), so a quantized layer could not be stored as it is.  A layer `prefix` is three
//! tensors - `{prefix}.qweight` I8 `[out, in]`, `{prefix}.scales` F32 `[out]`, `{prefix}.bias` F32
//! `[out]` (absent without bias) - and loading fills the public fields of `QLinear` directly; the
//! device copy is then built from them by `nne_qlinear_create_from_i8`, nothing is re-quantized.
//! Same container handling as `save_safetensors` / `load_safetensors` (`:12-51`, `:53-100`).

use crate::error::{EngineError, Result};
use crate::nn::quantized::QLinear;
use safetensors::tensor::{Dtype, SafeTensors, TensorView};
use std::collections::HashMap;
use std::fs::File;
use std::io::{Read, Write};
use std::path::Path;

fn ser_err(msg: String) -> EngineError {
    EngineError::SerializationError(msg)
}

/// Saves named `QLinear` layers into one SafeTensors file.
pub fn save_qlinears<P: AsRef<Path>>(layers: &HashMap<String, QLinear>, path: P) -> Result<()> {
    // byte storage first: the views borrow from it
    let mut blobs: Vec<(String, Dtype, Vec<usize>, Vec<u8>)> = Vec::new();
    for (prefix, ql) in layers {
        let codes: Vec<u8> = ql.qweight.iter().map(|&q| q as u8).collect();
        blobs.push((format!("{prefix}.qweight"), Dtype::I8, vec![ql.out_features, ql.in_features], codes));
        let f32_bytes = |v: &[f32]| v.iter().flat_map(|x| x.to_le_bytes()).collect::<Vec<u8>>();
        blobs.push((format!("{prefix}.scales"), Dtype::F32, vec![ql.out_features], f32_bytes(&ql.scales)));
        if let Some(b) = &ql.bias {
            blobs.push((format!("{prefix}.bias"), Dtype::F32, vec![ql.out_features], f32_bytes(b)));
        }
    }
    let mut views: HashMap<String, TensorView> = HashMap::new();
    for (name, dtype, shape, bytes) in &blobs {
        let view = TensorView::new(*dtype, shape.clone(), bytes)
            .map_err(|e| ser_err(format!("Failed to create SafeTensors view: {}", e)))?;
        views.insert(name.clone(), view);
    }
    let bytes = safetensors::serialize(&views, &None)
        .map_err(|e| ser_err(format!("SafeTensors serialization error: {}", e)))?;
    let mut file = File::create(path).map_err(|e| ser_err(format!("Failed to create file: {}", e)))?;
    file.write_all(&bytes).map_err(|e| ser_err(format!("Failed to write SafeTensors file: {}", e)))?;
    Ok(())
}

/// Loads layer `prefix` from a SafeTensors file written by `save_qlinears`.
pub fn load_qlinear<P: AsRef<Path>>(path: P, prefix: &str) -> Result<QLinear> {
    let mut file = File::open(path).map_err(|e| ser_err(format!("Failed to open SafeTensors file: {}", e)))?;
    let mut buffer = Vec::new();
    file.read_to_end(&mut buffer).map_err(|e| ser_err(format!("Failed to read SafeTensors file: {}", e)))?;
    let st = SafeTensors::deserialize(&buffer)
        .map_err(|e| ser_err(format!("SafeTensors deserialization error: {}", e)))?;
    let get = |name: String, want: Dtype| -> Result<Option<(Vec<usize>, Vec<u8>)>> {
        match st.tensor(&name) {
            Err(_) => Ok(None),
            Ok(view) if view.dtype() != want => Err(ser_err(format!(
                "Unsupported SafeTensors dtype {:?} for tensor '{}': expected {:?}",
                view.dtype(),
                name,
                want
            ))),
            Ok(view) => Ok(Some((view.shape().to_vec(), view.data().to_vec()))),
        }
    };
    let (qshape, qbytes) = get(format!("{prefix}.qweight"), Dtype::I8)?
        .ok_or_else(|| ser_err(format!("SafeTensors file holds no tensor '{prefix}.qweight'")))?;
    let (sshape, sbytes) = get(format!("{prefix}.scales"), Dtype::F32)?
        .ok_or_else(|| ser_err(format!("SafeTensors file holds no tensor '{prefix}.scales'")))?;
    if qshape.len() != 2 || sshape != vec![qshape[0]] || qbytes.len() != qshape[0] * qshape[1] || sbytes.len() != 4 * qshape[0] {
        return Err(ser_err(format!("tensors of layer '{prefix}' have inconsistent shapes")));
    }
    let to_f32 = |b: &[u8]| b.chunks_exact(4).map(|c| f32::from_le_bytes([c[0], c[1], c[2], c[3]])).collect::<Vec<f32>>();
    let bias = match get(format!("{prefix}.bias"), Dtype::F32)? {
        Some((bshape, bbytes)) => {
            if bshape != vec![qshape[0]] || bbytes.len() != 4 * qshape[0] {
                return Err(ser_err(format!("'{prefix}.bias' must be F32 [out_features]")));
            }
            Some(to_f32(&bbytes))
        }
        None => None,
    };
    Ok(QLinear::from_parts(
        qbytes.iter().map(|&b| b as i8).collect(),
        to_f32(&sbytes),
        bias,
        qshape[1],
        qshape[0],
    ))
}
