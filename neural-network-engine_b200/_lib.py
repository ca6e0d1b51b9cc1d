"""ctypes binding of the nne_cuda C ABI (include/nne_cuda.h).

The shared object is built in-tree by ``csrc/Makefile`` into ``lib/libnne_cuda.so``.  There is
no fallback: if the library is missing, or a call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# NNE_CUDA_LIB points the loader at another build of the same library (e.g. one with tracing).
LIB_PATH = os.environ.get("NNE_CUDA_LIB") or os.path.join(_HERE, "lib", "libnne_cuda.so")

OK, INVALID_ARGUMENT, SHAPE_MISMATCH, CUDA, NCCL, TIMEOUT, OUT_OF_MEMORY, UNSUPPORTED = range(8)

c_void_pp = C.POINTER(C.c_void_p)
c_float_p = C.POINTER(C.c_float)
c_int8_p = C.POINTER(C.c_int8)

# name -> (restype, argtypes); exactly the symbols include/nne_cuda.h declares.
SIGNATURES = {
    "nne_status_string": (C.c_char_p, [C.c_int]),
    "nne_last_error": (C.c_int, [C.c_char_p, C.c_size_t]),
    "nne_cuda_ctx_create": (C.c_int, [C.c_int, c_void_pp]),
    "nne_cuda_ctx_destroy": (C.c_int, [C.c_void_p]),
    "nne_cuda_ctx_check": (C.c_int, [C.c_void_p]),
    "nne_device_alloc": (C.c_int, [C.c_void_p, C.c_size_t, c_void_pp]),
    "nne_device_free": (C.c_int, [C.c_void_p, C.c_void_p]),
    "nne_device_upload": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t]),
    "nne_device_download": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t]),
    "nne_cuda_ctx_stream": (C.c_void_p, [C.c_void_p]),
    "nne_cuda_ctx_selftest_wait": (C.c_int, [C.c_void_p, C.c_int, C.c_uint]),
    "nne_cuda_ctx_info": (C.c_int, [C.c_void_p, C.POINTER(C.c_int), C.POINTER(C.c_int),
                                    C.POINTER(C.c_int), C.POINTER(C.c_int),
                                    C.POINTER(C.c_size_t)]),
    "nne_quantize_rows": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p,
                                    C.c_void_p]),
    "nne_quantize_rows_dev": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t,
                                        C.c_void_p, C.c_void_p, C.c_void_p]),
    "nne_quantize_tensor": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p,
                                      C.c_void_p]),
    "nne_quantize_tensor_dev": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p,
                                          C.c_void_p, C.c_void_p]),
    "nne_dequantize_rows": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t,
                                      C.c_size_t, C.c_void_p]),
    "nne_dequantize_rows_dev": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t,
                                          C.c_size_t, C.c_void_p, C.c_void_p]),
    "nne_qlinear_create_from_f32": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t,
                                              C.c_size_t, c_void_pp]),
    "nne_qlinear_create_from_f32_dev": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p,
                                                  C.c_size_t, C.c_size_t, C.c_void_p,
                                                  c_void_pp]),
    "nne_qlinear_create_from_i8": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                             C.c_size_t, C.c_size_t, c_void_pp]),
    "nne_qlinear_destroy": (C.c_int, [C.c_void_p]),
    "nne_qlinear_download": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p]),
    "nne_qlinear_info": (C.c_int, [C.c_void_p, C.POINTER(C.c_size_t), C.POINTER(C.c_size_t),
                                   C.POINTER(C.c_int), c_void_pp, c_void_pp, c_void_pp]),
    "nne_qlinear_memory_bytes": (C.c_size_t, [C.c_void_p]),
    "nne_qlinear_forward_host": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t,
                                           C.c_void_p]),
    "nne_qlinear_forward_dev": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t,
                                          C.c_void_p, C.c_void_p]),
    "nne_qlinear_forward_dev_strided": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t,
                                                  C.c_size_t, C.c_void_p, C.c_size_t,
                                                  C.c_void_p]),
    "nne_qlinear_forward_dev_static": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t,
                                                 C.c_void_p, C.c_void_p]),
    "nne_qlinear_plan_create": (C.c_int, [C.c_void_p, C.c_size_t, c_void_pp, c_void_pp, c_void_pp,
                                          C.c_size_t, c_void_pp]),
    "nne_cuda_ctx_reserve_sms": (C.c_int, [C.c_void_p, C.c_int]),
    "nne_qlinear_plan_run": (C.c_int, [C.c_void_p, C.c_void_p]),
    "nne_qlinear_plan_run_host": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p]),
    "nne_qlinear_plan_destroy": (C.c_int, [C.c_void_p]),
    "nne_qlinear_plan_launches": (C.c_int, [C.c_void_p]),
    "nne_rmsnorm_dev": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_float, C.c_size_t, C.c_size_t,
                                  C.c_void_p, C.c_void_p]),
    "nne_silu_mul_dev": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p]),
    "nne_add_dev": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p]),
    "nne_qlinear_plan_create_fused": (C.c_int, [C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t, c_void_pp]),
    "nne_shard_group_create": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_size_t, c_void_pp]),
    "nne_shard_group_handle": (C.c_int, [C.c_void_p, C.c_void_p]),
    "nne_shard_group_connect": (C.c_int, [C.c_void_p, C.c_void_p]),
    "nne_shard_group_connect_local": (C.c_int, [C.c_void_p, c_void_pp]),
    "nne_shard_group_window": (C.c_int, [C.c_void_p, c_void_pp, C.POINTER(C.c_size_t)]),
    "nne_shard_group_wait": (C.c_int, [C.c_void_p, C.c_void_p]),
    "nne_shard_group_set_nccl": (C.c_int, [C.c_void_p, C.c_void_p]),
    "nne_shard_group_destroy": (C.c_int, [C.c_void_p]),
    "nne_qlinear_plan_create_sharded": (C.c_int, [C.c_void_p, C.c_size_t, c_void_pp,
                                                  C.POINTER(C.c_size_t), C.POINTER(C.c_size_t),
                                                  c_void_pp, c_void_pp, C.c_size_t, C.c_int,
                                                  c_void_pp]),
    "nne_qlinear_kernel_for": (C.c_int, [C.c_void_p, C.c_size_t]),
    "nne_launch_count": (C.c_uint64, []),
}



class PlanItem(C.Structure):
    """nne_plan_item of include/nne_cuda.h."""
    _fields_ = [("layer", C.c_void_p), ("x", C.c_void_p), ("y", C.c_void_p), ("input_op", C.c_int),
                ("eps", C.c_float), ("gamma", C.c_void_p), ("x2", C.c_void_p), ("residual", C.c_void_p)]


INPUT_PLAIN, INPUT_RMSNORM, INPUT_SILU_MUL = 0, 1, 2

_lib = None


class NneError(RuntimeError):
    """A failed C-ABI call: carries the status code and the library's error text."""

    def __init__(self, status: int, message: str):
        super().__init__(f"nne_cuda status {status}: {message}")
        self.status = status
        self.message = message


def load() -> C.CDLL:
    """Loads lib/libnne_cuda.so (once) and types every exported entry point."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `make -C {os.path.join(_HERE, 'csrc')}` "
            "(or __graft_entry__.build()); there is no CPU or PyTorch fallback")
    lib = C.CDLL(LIB_PATH, mode=C.RTLD_LOCAL)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def last_error() -> str:
    buf = C.create_string_buffer(1024)
    load().nne_last_error(buf, len(buf))
    return buf.value.decode("utf-8", "replace")


def check(status: int) -> None:
    if status != OK:
        raise NneError(status, last_error())
