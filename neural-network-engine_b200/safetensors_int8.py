"""int8 on-disk format for QLinear: SafeTensors files holding `I8` codes and `F32` scales / bias.

The reference's SafeTensors module (src/io/safetensors.rs:12-51 save, :53-100 load) stores and
accepts F32 tensors only - its loader rejects every other dtype (:68-74) - and its `Checkpoint` is
f32-only (src/io/checkpoint.rs:16), so a QLinear cannot be saved or loaded pre-quantized there: a
layer has to be uploaded as f32 (4x the bytes) and quantized again at every start-up.  This module
is the same container with one more dtype.  A layer `prefix` is three tensors,

    {prefix}.qweight  I8   [out_features, in_features]   (QLinear.qweight, src/nn/quantized.rs:80-81)
    {prefix}.scales   F32  [out_features]                (:82-83)
    {prefix}.bias     F32  [out_features]                (:84-85; absent when the layer has none)

and loading goes straight into `QLinear.from_fields` -> `nne_qlinear_create_from_i8`: the codes
reach the device as they are, nothing is re-quantized.  F32 tensors written here are readable by
the reference's loader; files it wrote load here.

Container layout (the published SafeTensors format): 8-byte little-endian header length, a JSON
header mapping tensor names to {"dtype", "shape", "data_offsets": [begin, end)} (offsets relative
to the end of the header, optional "__metadata__" of string pairs), then the raw little-endian
tensor bytes back to back.  The header is padded with spaces to a multiple of 8 bytes."""
from __future__ import annotations

import json
import struct
from typing import Dict, Iterable, Optional, Tuple

import numpy as np

_DTYPES = {"F32": np.dtype("<f4"), "I8": np.dtype("i1")}
_NAMES = {np.dtype("<f4"): "F32", np.dtype("i1"): "I8"}
_MAX_HEADER = 100_000_000  # the format's own limit on the header size


class SerializationError(Exception):
    """EngineError::SerializationError(String), src/error.rs."""


def save_tensors(tensors: Dict[str, np.ndarray], path: str, metadata: Optional[Dict[str, str]] = None) -> None:
    """Writes named F32 / I8 arrays as one SafeTensors file (names sorted, data back to back)."""
    header, blobs, off = {}, [], 0
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    for name in sorted(tensors):
        a = np.ascontiguousarray(tensors[name])
        if a.dtype == np.float32:
            a = a.astype("<f4", copy=False)
        if a.dtype not in _NAMES:
            raise SerializationError(f"Unsupported dtype {a.dtype} for tensor '{name}': F32 and I8 only")
        raw = a.tobytes()
        header[name] = {"dtype": _NAMES[a.dtype], "shape": list(a.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    text = json.dumps(header, separators=(",", ":")).encode("utf-8")
    text += b" " * (-len(text) % 8)
    try:
        with open(path, "wb") as f:
            f.write(struct.pack("<Q", len(text)))
            f.write(text)
            for b in blobs:
                f.write(b)
    except OSError as e:
        raise SerializationError(f"Failed to write SafeTensors file: {e}") from e


def load_tensors(path: str, only: Optional[Iterable[str]] = None) -> Dict[str, np.ndarray]:
    """Reads a SafeTensors file holding F32 and I8 tensors.  Any other dtype is an error naming
    the tensor, as in the reference's loader (src/io/safetensors.rs:68-74)."""
    try:
        with open(path, "rb") as f:
            buf = f.read()
    except OSError as e:
        raise SerializationError(f"Failed to open SafeTensors file: {e}") from e
    if len(buf) < 8:
        raise SerializationError("SafeTensors deserialization error: file shorter than its length field")
    (hlen,) = struct.unpack("<Q", buf[:8])
    if hlen > _MAX_HEADER or 8 + hlen > len(buf):
        raise SerializationError("SafeTensors deserialization error: header length out of range")
    try:
        header = json.loads(buf[8:8 + hlen].decode("utf-8"))
    except (UnicodeDecodeError, json.JSONDecodeError) as e:
        raise SerializationError(f"SafeTensors deserialization error: {e}") from e
    if not isinstance(header, dict):
        raise SerializationError("SafeTensors deserialization error: header is not an object")
    data = memoryview(buf)[8 + hlen:]
    want = None if only is None else set(only)
    out, spans = {}, []
    for name, info in header.items():
        if name == "__metadata__":
            continue
        try:
            dtype, shape, (b, e) = info["dtype"], [int(s) for s in info["shape"]], info["data_offsets"]
        except (KeyError, TypeError, ValueError) as ex:
            raise SerializationError(f"SafeTensors deserialization error: bad entry for '{name}'") from ex
        if not (0 <= b <= e <= len(data)):
            raise SerializationError(f"SafeTensors deserialization error: offsets of '{name}' outside the file")
        spans.append((b, e))
        if want is not None and name not in want:
            continue
        if dtype not in _DTYPES:
            raise SerializationError(
                f"Unsupported SafeTensors dtype {dtype} for tensor '{name}'. Only F32 and I8 are supported.")
        dt = _DTYPES[dtype]
        count = int(np.prod(shape, dtype=np.int64)) if shape else 1
        if e - b != count * dt.itemsize:
            raise SerializationError(
                f"SafeTensors tensor '{name}': {e - b} bytes do not match shape {shape} of {dtype}")
        out[name] = np.frombuffer(data[b:e], dtype=dt).reshape(shape).copy()
    spans.sort()
    pos = 0
    for b, e in spans:  # the format wants the tensors back to back with no hole and no overlap
        if b != pos:
            raise SerializationError("SafeTensors deserialization error: tensor data is not contiguous")
        pos = e
    return out


# ---- QLinear <-> file ---------------------------------------------------------------------------
def qlinear_tensors(prefix: str, ql) -> Dict[str, np.ndarray]:
    """The tensors of one layer under their file names."""
    n, k = ql.out_features, ql.in_features
    t = {f"{prefix}.qweight": np.asarray(ql.qweight, dtype=np.int8).reshape(n, k),
         f"{prefix}.scales": np.asarray(ql.scales, dtype=np.float32).reshape(n)}
    if ql.bias is not None:
        t[f"{prefix}.bias"] = np.asarray(ql.bias, dtype=np.float32).reshape(n)
    return t


def save_qlinears(layers: Dict[str, object], path: str) -> None:
    """Saves named QLinear layers (their public fields: codes, scales, bias) into one file."""
    tensors = {}
    for prefix, ql in layers.items():
        tensors.update(qlinear_tensors(prefix, ql))
    save_tensors(tensors, path, {"format": "nn::quantized::QLinear int8 per-output-channel"})


def load_qlinear_fields(path: str, prefix: str) -> Tuple[np.ndarray, np.ndarray, Optional[np.ndarray]]:
    """(qweight [N, K] int8, scales [N] f32, bias [N] f32 or None) of layer `prefix`."""
    names = [f"{prefix}.qweight", f"{prefix}.scales", f"{prefix}.bias"]
    t = load_tensors(path, only=names)
    if names[0] not in t or names[1] not in t:
        raise SerializationError(f"SafeTensors file holds no layer '{prefix}' (qweight and scales)")
    q, s, b = t[names[0]], t[names[1]], t.get(names[2])
    if q.dtype != np.int8 or q.ndim != 2:
        raise SerializationError(f"'{names[0]}' must be I8 [out_features, in_features]")
    if s.dtype != np.float32 or s.shape != (q.shape[0],):
        raise SerializationError(f"'{names[1]}' must be F32 [out_features]")
    if b is not None and (b.dtype != np.float32 or b.shape != (q.shape[0],)):
        raise SerializationError(f"'{names[2]}' must be F32 [out_features]")
    return q, s, b


def load_qlinear(path: str, prefix: str, ctx=None):
    """Loads layer `prefix` as a device-resident QLinear (codes uploaded as stored)."""
    from .quantized import QLinear
    q, s, b = load_qlinear_fields(path, prefix)
    return QLinear.from_fields(q.reshape(-1), s, b, q.shape[1], q.shape[0], ctx)
