"""B200 (sm_100a) backend for the int8 quantized-linear path of neural-network-engine.

Python mirror of the reference's ``nn::quantized`` API (``Int8Tensor``, ``QLinear``) over the
``nne_cuda`` C ABI.  All arithmetic runs in hand-written CUDA kernels; nothing here computes on
the CPU and nothing falls back when the library or a GPU is missing.
"""
from ._lib import NneError, load, LIB_PATH  # noqa: F401
from .quantized import (  # noqa: F401
    CudaContext,
    CudaQLinear,
    CudaTensor,
    EngineError,
    FusedPlan,
    GpuError,
    Int8Tensor,
    InvalidArgument,
    Linear,
    QLinear,
    QLinearPlan,
    ShapeMismatch,
    add_device,
    default_context,
    rmsnorm_device,
    silu_mul_device,
)
from . import safetensors_int8  # noqa: F401
from .safetensors_int8 import load_qlinear, save_qlinears  # noqa: F401
from .sharding import (  # noqa: F401
    ROUTE_NCCL,
    ROUTE_PEER_STORES,
    DeviceArray,
    NcclComm,
    ShardGroup,
    ShardedPlan,
    ShardedQLinear,
    assemble,
    shard_rows,
    shard_sizes,
)
