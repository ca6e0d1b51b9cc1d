"""Host-side mirror of the reference module ``nn::quantized`` (src/nn/quantized.rs).

Same names, fields, argument meaning and error behaviour as the reference's ``Int8Tensor``
(src/nn/quantized.rs:20-73) and ``QLinear`` (src/nn/quantized.rs:78-250); host tensors are numpy
arrays where the reference uses ``RawTensor``/``Tensor``.  Every computation is a call through
the ``nne_cuda`` C ABI into CUDA kernels: there is no CPU path in this module.
"""
from __future__ import annotations

import ctypes as C
import threading
from typing import List, Optional, Sequence

import numpy as np

from . import _lib
from ._lib import NneError, check, load


# ---- errors: the three EngineError variants this path can return (src/error.rs:10-52) --------
class EngineError(Exception):
    pass


class InvalidArgument(EngineError):
    """EngineError::InvalidArgument(String), src/error.rs:41-42."""


class ShapeMismatch(EngineError):
    """EngineError::ShapeMismatch{expected, actual}, src/error.rs:11-15."""

    def __init__(self, expected: Sequence[int], actual: Sequence[int]):
        super().__init__(f"Shape mismatch error: expected shape {list(expected)}, got {list(actual)}")
        self.expected = list(expected)
        self.actual = list(actual)


class GpuError(EngineError):
    """EngineError::GpuError(String), src/error.rs:47-48: any device-side failure."""


def _raise_mapped(err: NneError):
    if err.status == _lib.INVALID_ARGUMENT:
        raise InvalidArgument(err.message) from err
    raise GpuError(err.message) from err


def _ptr(a: Optional[np.ndarray]):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


# ---- device context: the Arc<GpuContext> of the existing device backend (src/gpu/layers.rs:12-16)
class CudaContext:
    def __init__(self, device: int = 0):
        lib = load()
        h = C.c_void_p()
        try:
            check(lib.nne_cuda_ctx_create(int(device), C.byref(h)))
        except NneError as e:
            raise GpuError(e.message) from e
        self._h = h
        dev, sms, maj, minr, mem = C.c_int(), C.c_int(), C.c_int(), C.c_int(), C.c_size_t()
        check(lib.nne_cuda_ctx_info(h, C.byref(dev), C.byref(sms), C.byref(maj), C.byref(minr),
                                    C.byref(mem)))
        self.device, self.sm_count = dev.value, sms.value
        self.compute_capability = (maj.value, minr.value)
        self.total_mem_bytes = mem.value

    @property
    def handle(self) -> C.c_void_p:
        if self._h is None:
            raise GpuError("context was destroyed")
        return self._h

    def check(self) -> None:
        """Synchronises the device; raises GpuError if a kernel's bounded wait ran out."""
        try:
            check(load().nne_cuda_ctx_check(self.handle))
        except NneError as e:
            raise GpuError(e.message) from e

    def close(self):
        if getattr(self, "_h", None) is not None:
            load().nne_cuda_ctx_destroy(self._h)
            self._h = None

    def __del__(self):  # pragma: no cover - best effort
        try:
            self.close()
        except Exception:
            pass


_default_ctx = {}
_default_lock = threading.Lock()


def default_context(device: int = 0) -> CudaContext:
    """One shared context per device, created on first use."""
    with _default_lock:
        ctx = _default_ctx.get(device)
        if ctx is None or ctx._h is None:
            ctx = CudaContext(device)
            _default_ctx[device] = ctx
        return ctx


# ---- boundary type: the fields of nn::Linear that the path reads (src/nn/linear.rs:9-14) -------
class Linear:
    """f32 dense layer as a plain container: weight [out_features, in_features], optional bias."""

    def __init__(self, weight: np.ndarray, bias: Optional[np.ndarray] = None):
        weight = np.asarray(weight, dtype=np.float32)
        if weight.ndim != 2:
            raise InvalidArgument(f"Linear weight must be 2-D, got shape {list(weight.shape)}")
        self.weight = weight
        self.bias = None if bias is None else np.asarray(bias, dtype=np.float32)
        self.out_features, self.in_features = int(weight.shape[0]), int(weight.shape[1])
        if self.bias is not None and self.bias.shape != (self.out_features,):
            raise InvalidArgument("Linear bias must have shape [out_features]")


class Int8Tensor:
    """Symmetric per-tensor int8 tensor; fields as src/nn/quantized.rs:20-28."""

    # size_of::<Int8Tensor>() on a 64-bit target: two Vecs of 24 bytes, one f32, padded to 8.
    _SIZE_OF_SELF = 56

    def __init__(self, data: np.ndarray, shape: List[int], scale: float):
        self.data = data
        self.shape = list(shape)
        self.scale = scale

    @classmethod
    def from_raw(cls, raw: np.ndarray, ctx: Optional[CudaContext] = None) -> "Int8Tensor":
        """Int8Tensor::from_raw (src/nn/quantized.rs:32-57), computed on the GPU."""
        ctx = ctx or default_context()
        vals = np.ascontiguousarray(raw, dtype=np.float32)  # to_contiguous(), :33
        data = np.empty(vals.size, dtype=np.int8)
        scale = np.empty(1, dtype=np.float32)
        try:
            check(load().nne_quantize_tensor(ctx.handle, _ptr(vals), vals.size, _ptr(data),
                                             _ptr(scale)))
        except NneError as e:
            _raise_mapped(e)
        return cls(data, list(vals.shape), np.float32(scale[0]))

    def dequantize(self, ctx: Optional[CudaContext] = None) -> np.ndarray:
        """Int8Tensor::dequantize (src/nn/quantized.rs:60-67), computed on the GPU."""
        ctx = ctx or default_context()
        out = np.empty(self.data.size, dtype=np.float32)
        scale = np.array([self.scale], dtype=np.float32)
        try:
            check(load().nne_dequantize_rows(ctx.handle, _ptr(self.data), _ptr(scale), 1,
                                             self.data.size, _ptr(out)))
        except NneError as e:
            _raise_mapped(e)
        return out.reshape(self.shape)

    def memory_bytes(self) -> int:
        """src/nn/quantized.rs:70-72."""
        return int(self.data.size) + self._SIZE_OF_SELF


class QLinear:
    """int8 linear layer with per-output-channel scales; public fields as
    src/nn/quantized.rs:78-88.  The host copies ``qweight``/``scales``/``bias`` stay populated
    (the reference's tests read them); the device-resident layer is a private handle."""

    def __init__(self, qweight, scales, bias, in_features, out_features, _handle=None, _ctx=None,
                 _error=None):
        self.qweight = qweight
        self.scales = scales
        self.bias = bias
        self.in_features = int(in_features)
        self.out_features = int(out_features)
        self._handle = _handle
        self._ctx = _ctx
        self._error = _error  # a device failure at construction, surfaced by the first forward

    # -- construction --------------------------------------------------------------------------
    @classmethod
    def from_linear(cls, linear: Linear, ctx: Optional[CudaContext] = None) -> "QLinear":
        """QLinear::from_linear (src/nn/quantized.rs:92-141).  Infallible like the reference: a
        device failure is kept and raised as GpuError by the first forward."""
        n, k = linear.out_features, linear.in_features
        w = np.ascontiguousarray(linear.weight, dtype=np.float32)
        assert w.size == n * k, "Weight slice length must match out_features * in_features"
        bias = None if linear.bias is None else np.ascontiguousarray(linear.bias, dtype=np.float32)
        qweight = np.empty(n * k, dtype=np.int8)
        scales = np.empty(n, dtype=np.float32)
        handle, err = None, None
        try:
            ctx = ctx or default_context()
            h = C.c_void_p()
            check(load().nne_qlinear_create_from_f32(ctx.handle, _ptr(w), _ptr(bias), n, k,
                                                     C.byref(h)))
            handle = h
            check(load().nne_qlinear_download(h, _ptr(qweight), _ptr(scales)))
        except (NneError, GpuError) as e:
            err = getattr(e, "message", str(e))
        return cls(qweight, scales, None if bias is None else bias.copy(), k, n, handle, ctx, err)

    @classmethod
    def from_fields(cls, qweight, scales, bias, in_features, out_features,
                    ctx: Optional[CudaContext] = None) -> "QLinear":
        """Builds the device layer from the public fields of an existing QLinear."""
        n, k = int(out_features), int(in_features)
        q = np.ascontiguousarray(qweight, dtype=np.int8).reshape(-1)
        s = np.ascontiguousarray(scales, dtype=np.float32).reshape(-1)
        b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32).reshape(-1)
        if q.size != n * k or s.size != n or (b is not None and b.size != n):
            raise InvalidArgument("field sizes do not match in_features/out_features")
        ctx = ctx or default_context()
        h = C.c_void_p()
        try:
            check(load().nne_qlinear_create_from_i8(ctx.handle, _ptr(q), _ptr(s), _ptr(b), n, k,
                                                    C.byref(h)))
        except NneError as e:
            _raise_mapped(e)
        return cls(q, s, b, k, n, h, ctx, None)

    def clone(self) -> "QLinear":
        """#[derive(Clone)]: deep copy, with its own device-resident layer."""
        return QLinear.from_fields(self.qweight.copy(), self.scales.copy(),
                                   None if self.bias is None else self.bias.copy(),
                                   self.in_features, self.out_features, self._ctx)

    # -- forward -------------------------------------------------------------------------------
    def _live_handle(self):
        if self._error is not None:
            raise GpuError(self._error)
        if self._handle is None:
            raise GpuError("layer has no device handle")
        return self._handle

    def forward_quantized(self, input: np.ndarray) -> np.ndarray:
        """QLinear::forward_quantized (src/nn/quantized.rs:146-197)."""
        x = np.asarray(input)
        in_shape = list(x.shape)
        ndim = len(in_shape)
        if ndim < 2:  # :149-154
            raise InvalidArgument(
                f"QLinear forward expects tensor with at least 2 dimensions, got {in_shape}")
        in_k = in_shape[-1]
        if in_k != self.in_features:  # :156-162
            raise ShapeMismatch([self.in_features], [in_k])
        num_rows = int(np.prod(in_shape[:-1], dtype=np.int64))  # :164
        xc = np.ascontiguousarray(x, dtype=np.float32)  # :165
        out_shape = in_shape[:-1] + [self.out_features]
        out = np.zeros(num_rows * self.out_features, dtype=np.float32)  # :170
        h = self._live_handle()
        try:
            check(load().nne_qlinear_forward_host(h, _ptr(xc), num_rows, in_k, _ptr(out)))
        except NneError as e:
            if e.status == _lib.SHAPE_MISMATCH:
                raise ShapeMismatch([self.in_features], [in_k]) from e
            _raise_mapped(e)
        return out.reshape(out_shape)

    def forward(self, input: np.ndarray) -> np.ndarray:
        """impl Module for QLinear (src/nn/quantized.rs:240-243)."""
        return self.forward_quantized(input)

    def parameters(self) -> list:
        """src/nn/quantized.rs:245-248: a fixed-precision inference layer has none."""
        return []

    def forward_device(self, x_ptr: int, m: int, y_ptr: int, stream: int = 0,
                       ldy: Optional[int] = None) -> None:
        """Device-resident forward: x [m, in_features] and y [m, out_features] (row stride
        ``ldy`` floats) are device pointers; asynchronous on the CUDA stream ``stream``."""
        h = self._live_handle()
        try:
            if ldy is None:
                check(load().nne_qlinear_forward_dev(h, x_ptr, m, self.in_features, y_ptr, stream))
            else:
                check(load().nne_qlinear_forward_dev_strided(h, x_ptr, m, self.in_features, y_ptr,
                                                             ldy, stream))
        except NneError as e:
            _raise_mapped(e)

    def kernel_for(self, m: int) -> int:
        """1 = streaming GEMV, 2 = tcgen05 tensor-core kernel, 3 = generic kernel,
        4 = small-batch tcgen05 kernel (3 <= m <= 16)."""
        return int(load().nne_qlinear_kernel_for(self._live_handle(), m))

    # -- the rest of the reference surface -----------------------------------------------------
    def to_linear(self) -> Linear:
        """QLinear::to_linear (src/nn/quantized.rs:200-227); the q*scale loop runs on the GPU."""
        n, k = self.out_features, self.in_features
        w = np.empty(n * k, dtype=np.float32)
        ctx = self._ctx or default_context()
        try:
            check(load().nne_dequantize_rows(ctx.handle, _ptr(self.qweight), _ptr(self.scales), n, k,
                                             _ptr(w)))
        except NneError as e:
            _raise_mapped(e)
        return Linear(w.reshape(n, k), None if self.bias is None else self.bias.copy())

    def memory_bytes(self) -> int:
        """QLinear::memory_bytes (src/nn/quantized.rs:230-237)."""
        return int(self.qweight.size + self.scales.size * 4 +
                   (0 if self.bias is None else self.bias.size * 4))

    def close(self):
        if self._handle is not None:
            load().nne_qlinear_destroy(self._handle)
            self._handle = None

    def __del__(self):  # pragma: no cover - best effort
        try:
            self.close()
        except Exception:
            pass


class QLinearPlan:
    """Several independent ``QLinear`` forwards on fixed device buffers, issued together.

    Stands for the back-to-back ``forward`` calls a caller makes on projections that do not depend
    on each other (q/k/v at src/models/llama.rs:226-228, gate/up at :344-346).  ``x_ptrs[i]`` is a
    device pointer to ``[m, layers[i].in_features]`` f32, ``y_ptrs[i]`` to ``[m, out_features]``.
    For m = 1 the whole list is one kernel launch, for 2 <= m <= 16 one pre-pass and one launch;
    results equal per-layer ``forward_device`` bit for bit."""

    def __init__(self, layers, x_ptrs, y_ptrs, m: int, ctx: Optional[CudaContext] = None):
        ctx = ctx or layers[0]._ctx or default_context()
        n = len(layers)
        hs = (C.c_void_p * n)(*[l._live_handle() for l in layers])
        xs = (C.c_void_p * n)(*[int(p) for p in x_ptrs])
        ys = (C.c_void_p * n)(*[int(p) for p in y_ptrs])
        h = C.c_void_p()
        try:
            check(load().nne_qlinear_plan_create(ctx.handle, n, hs, xs, ys, m, C.byref(h)))
        except NneError as e:
            _raise_mapped(e)
        self._h, self._layers, self._ctx = h, list(layers), ctx  # keep the layers alive
        self._m = int(m)

    @property
    def launches(self) -> int:
        return int(load().nne_qlinear_plan_launches(self._h))

    def run(self, stream: int = 0) -> None:
        try:
            check(load().nne_qlinear_plan_run(self._h, stream))
        except NneError as e:
            _raise_mapped(e)

    def run_host(self, x_all: np.ndarray, y_all: Optional[np.ndarray] = None) -> np.ndarray:
        """Host round trip of the whole plan: ``x_all`` holds the activations of all layers one
        after another (f32), the outputs come back the same way."""
        m = self._m
        nx = sum(m * l.in_features for l in self._layers)
        ny = sum(m * l.out_features for l in self._layers)
        x_all = np.ascontiguousarray(x_all, dtype=np.float32).reshape(-1)
        if x_all.size != nx:
            raise ShapeMismatch([nx], [x_all.size])
        if y_all is None:
            y_all = np.empty(ny, dtype=np.float32)
        if y_all.size != ny or y_all.dtype != np.float32 or not y_all.flags.c_contiguous:
            raise InvalidArgument("y_all must be a contiguous f32 array of the plan's output size")
        try:
            check(load().nne_qlinear_plan_run_host(self._h, _ptr(x_all), _ptr(y_all)))
        except NneError as e:
            _raise_mapped(e)
        return y_all

    def close(self):
        if getattr(self, "_h", None) is not None:
            load().nne_qlinear_plan_destroy(self._h)
            self._h = None

    def __del__(self):  # pragma: no cover - best effort
        try:
            self.close()
        except Exception:
            pass


# ---- device-resident tensors: GpuTensor / ToGpu / GpuLinear of the device backend -----------------
class CudaTensor:
    """f32 tensor in device memory; the `GpuTensor` of this backend (src/gpu/tensor.rs:12-16):
    `from_slice` / `from_raw` upload (:19-50), `to_cpu` downloads (:53-95), `shape` (:98-100)."""

    def __init__(self, ptr: int, shape, ctx: CudaContext, owner: bool = True):
        self.ptr, self.shape, self.ctx, self._owner = int(ptr), [int(s) for s in shape], ctx, owner

    @classmethod
    def empty(cls, shape, ctx: Optional[CudaContext] = None) -> "CudaTensor":
        ctx = ctx or default_context()
        n = int(np.prod(shape, dtype=np.int64)) if len(shape) else 1
        p = C.c_void_p()
        try:
            check(load().nne_device_alloc(ctx.handle, 4 * n, C.byref(p)))
        except NneError as e:
            _raise_mapped(e)
        return cls(p.value, shape, ctx)

    @classmethod
    def from_raw(cls, raw: np.ndarray, ctx: Optional[CudaContext] = None) -> "CudaTensor":
        a = np.ascontiguousarray(raw, dtype=np.float32)  # to_contiguous(), src/gpu/tensor.rs:48
        t = cls.empty(a.shape, ctx)
        try:
            check(load().nne_device_upload(t.ctx.handle, t.ptr, _ptr(a), a.nbytes))
        except NneError as e:
            _raise_mapped(e)
        return t

    @classmethod
    def from_slice(cls, values, shape, ctx: Optional[CudaContext] = None) -> "CudaTensor":
        a = np.asarray(values, dtype=np.float32).reshape(-1)
        if a.size != int(np.prod(shape, dtype=np.int64)):  # IncompatibleShapes, src/gpu/tensor.rs:21-26
            raise InvalidArgument(f"GpuTensor::from_slice: {a.size} values for shape {list(shape)}")
        return cls.from_raw(a.reshape(shape), ctx)

    def numel(self) -> int:
        return int(np.prod(self.shape, dtype=np.int64)) if self.shape else 1

    def to_cpu(self) -> np.ndarray:
        out = np.empty(self.shape, dtype=np.float32)
        try:
            check(load().nne_device_download(self.ctx.handle, _ptr(out), self.ptr, out.nbytes))
        except NneError as e:
            _raise_mapped(e)
        return out

    def close(self):
        if self._owner and self.ptr:
            load().nne_device_free(self.ctx.handle, self.ptr)
        self.ptr = 0

    def __del__(self):  # pragma: no cover - best effort
        try:
            self.close()
        except Exception:
            pass


class CudaQLinear:
    """`QLinear` placed on the device: the `GpuLinear` of this backend (src/gpu/layers.rs:24-43).
    `forward` takes and returns device tensors and is asynchronous on the context's stream; nothing
    crosses PCIe until `to_cpu`."""

    def __init__(self, layer: "QLinear", ctx: CudaContext):
        self.layer, self.ctx = layer, ctx
        self.in_features, self.out_features = layer.in_features, layer.out_features

    def forward(self, input: CudaTensor) -> CudaTensor:
        if len(input.shape) < 2:
            raise InvalidArgument(
                f"QLinear forward expects tensor with at least 2 dimensions, got {input.shape}")
        if input.shape[-1] != self.in_features:
            raise ShapeMismatch([self.in_features], [input.shape[-1]])
        m = int(np.prod(input.shape[:-1], dtype=np.int64))
        out = CudaTensor.empty(input.shape[:-1] + [self.out_features], self.ctx)
        self.layer.forward_device(input.ptr, m, out.ptr, load().nne_cuda_ctx_stream(self.ctx.handle) or 0)
        return out


def _qlinear_to_gpu(self, ctx: Optional[CudaContext] = None) -> CudaQLinear:
    """`impl ToGpu for QLinear` (the trait of src/gpu/layers.rs:12-15): the layer's device-resident
    form.  Its weights already live on the device, so nothing is uploaded again when the context is
    the layer's own; another context gets its own copy of the codes."""
    ctx = ctx or self._ctx or default_context()
    if self._ctx is not None and ctx is not self._ctx:
        return CudaQLinear(QLinear.from_fields(self.qweight, self.scales, self.bias, self.in_features,
                                               self.out_features, ctx), ctx)
    return CudaQLinear(self, ctx)


QLinear.to_gpu = _qlinear_to_gpu


# ---- the steps either side of a QLinear in a decoder block ---------------------------------------
def rmsnorm_device(ctx: CudaContext, x_ptr: int, gamma_ptr: int, eps: float, rows: int, cols: int,
                   y_ptr: int, stream: int = 0) -> None:
    """RMSNorm::forward (src/nn/norm.rs:141-165) on device buffers."""
    try:
        check(load().nne_rmsnorm_dev(ctx.handle, x_ptr, gamma_ptr, eps, rows, cols, y_ptr, stream))
    except NneError as e:
        _raise_mapped(e)


def silu_mul_device(ctx: CudaContext, gate_ptr: int, up_ptr: int, n: int, out_ptr: int, stream: int = 0) -> None:
    """silu(gate) * up (src/models/llama.rs:343-346) on device buffers."""
    try:
        check(load().nne_silu_mul_dev(ctx.handle, gate_ptr, up_ptr, n, out_ptr, stream))
    except NneError as e:
        _raise_mapped(e)


def add_device(ctx: CudaContext, a_ptr: int, b_ptr: int, n: int, out_ptr: int, stream: int = 0) -> None:
    """The residual add of a decoder block (src/models/llama.rs:377-392) on device buffers."""
    try:
        check(load().nne_add_dev(ctx.handle, a_ptr, b_ptr, n, out_ptr, stream))
    except NneError as e:
        _raise_mapped(e)


class FusedPlan(QLinearPlan):
    """`nne_qlinear_plan_create_fused`: forwards that apply RMSNorm or silu(x) * x2 to their input and
    add a residual to their output.  `items` are dicts with keys layer, x, y and optionally
    rmsnorm=(gamma_ptr, eps), silu_mul=x2_ptr, residual=ptr (all device pointers)."""

    def __init__(self, items, m: int, ctx: Optional[CudaContext] = None):
        ctx = ctx or items[0]["layer"]._ctx or default_context()
        n = len(items)
        arr = (_lib.PlanItem * n)()
        for i, it in enumerate(items):
            arr[i].layer = it["layer"]._live_handle()
            arr[i].x, arr[i].y = int(it["x"]), int(it["y"])
            arr[i].input_op, arr[i].eps = _lib.INPUT_PLAIN, 0.0
            if it.get("rmsnorm") is not None:
                arr[i].input_op = _lib.INPUT_RMSNORM
                arr[i].gamma, arr[i].eps = int(it["rmsnorm"][0]), float(it["rmsnorm"][1])
            elif it.get("silu_mul") is not None:
                arr[i].input_op = _lib.INPUT_SILU_MUL
                arr[i].x2 = int(it["silu_mul"])
            if it.get("residual") is not None:
                arr[i].residual = int(it["residual"])
        h = C.c_void_p()
        try:
            check(load().nne_qlinear_plan_create_fused(ctx.handle, n, arr, m, C.byref(h)))
        except NneError as e:
            _raise_mapped(e)
        self._h, self._layers, self._ctx = h, [it["layer"] for it in items], ctx
        self._m = int(m)
