"""magnitude_b200 — B200-native (sm_100a) GGUF block-quantized projection matmul.

The package is a thin host layer over libb200q.so (C ABI in include/b200q.h).  Importing it
loads the shared library and raises ImportError if it has not been built: there is no CPU,
PyTorch or other fallback for the products it computes.
"""
from . import _binding
from ._binding import (  # noqa: F401
    B200QError,
    ROUTE_GEMM,
    ROUTE_GEMV,
    ROUTE_NONE,
    ROUTE_SKINNY,
    SPLIT_COLUMN,
    SPLIT_ROW,
    TYPE_BF16,
    TYPE_F32,
    TYPE_MXFP4,
    TYPE_Q4_0,
    TYPE_Q4_K,
    TYPE_Q5_K,
    TYPE_Q6_K,
    TYPE_Q8_0,
)
from .projection import (  # noqa: F401
    Backend,
    GgufFile,
    Plan,
    ProjectionWeight,
    quantize,
    shard_range,
    tensor_storage_bytes,
    tensor_storage_bytes_shape,
    tp_unique_id,
)

_binding.lib()  # fail loudly at import time when the native library is absent

__version__ = _binding.lib().b200q_version().decode()
