"""B200 (sm_100a) backend for the int8 quantized-linear path of neural-network-engine.

Python mirror of the reference's ``nn::quantized`` API (``Int8Tensor``, ``QLinear``) over the
``nne_cuda`` C ABI.  All arithmetic runs in hand-written CUDA kernels; nothing here computes on
the CPU and nothing falls back when the library or a GPU is missing.
"""
from ._lib import NneError, load, LIB_PATH  # noqa: F401
from .quantized import (  # noqa: F401
    CudaContext,
    EngineError,
    GpuError,
    Int8Tensor,
    InvalidArgument,
    Linear,
    QLinear,
    QLinearPlan,
    ShapeMismatch,
    default_context,
)
from .sharding import ShardedQLinear, assemble, shard_rows, shard_sizes  # noqa: F401
