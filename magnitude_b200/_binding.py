"""ctypes binding of libb200q.so — the C ABI declared in include/b200q.h.

There is no fallback: if the shared library is missing the import of this module raises, and
without a CUDA device every compute call returns B200Q_ERR_BACKEND, surfaced as B200QError.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, c_char_p, c_int32, c_int64, c_size_t, c_uint64, c_void_p
from pathlib import Path

LIB_NAME = "libb200q.so"
LIB_PATH = Path(__file__).resolve().parent / LIB_NAME

OK = 0
ERR_INVALID_CONFIG, ERR_BACKEND, ERR_CANCELLED, ERR_OVERLOADED, ERR_STOPPED, ERR_CALLBACK, ERR_TIMEOUT = range(1, 8)
STATUS_NAMES = {
    0: "Ok",
    1: "InvalidConfig",
    2: "Backend",
    3: "Cancelled",
    4: "Overloaded",
    5: "ExecutorStopped",
    6: "Callback",
    7: "Timeout",
}

TYPE_F32, TYPE_Q4_0, TYPE_Q8_0, TYPE_Q4_K, TYPE_Q5_K, TYPE_Q6_K, TYPE_BF16, TYPE_MXFP4 = 0, 2, 8, 12, 13, 14, 30, 39
SPLIT_COLUMN, SPLIT_ROW = 0, 1
ROUTE_NONE, ROUTE_GEMV, ROUTE_SKINNY, ROUTE_GEMM = 0, 1, 2, 3

OPT_SKINNY_MIN_M, OPT_WAIT_LIMIT_MS, OPT_TP_INIT_TIMEOUT_MS = 1, 2, 3

JOB_WAITS_FOR_EARLIER = 1
JOB_SUM_RANKS = 2
JOB_SWIGLU = 4
JOB_ACCUMULATE = 8


class Job(ctypes.Structure):
    """struct b200q_job of include/b200q.h."""

    _fields_ = [
        ("w", c_void_p * 4),
        ("n_weights", c_int32),
        ("x_dtype", c_int32),
        ("x_dev", c_void_p),
        ("ldx", c_int64),
        ("y_dev", c_void_p * 4),
        ("ldy", c_int64 * 4),
        ("y_dtype", c_int32),
        ("flags", c_int32),
        ("norm_weight", c_void_p),
        ("norm_eps", ctypes.c_float),
        ("reserved", c_int32),
    ]


# every symbol include/b200q.h declares: (restype, argtypes)
SIGNATURES = {
    "b200q_version": (c_char_p, []),
    "b200q_tensor_storage_bytes": (c_int64, [c_int32, c_int64]),
    "b200q_ctx_create": (c_int32, [c_int32, POINTER(c_void_p)]),
    "b200q_ctx_destroy": (None, [c_void_p]),
    "b200q_ctx_set_option": (c_int32, [c_void_p, c_int32, c_int64]),
    "b200q_last_error": (c_int32, [c_void_p, c_char_p, c_size_t]),
    "b200q_sync": (c_int32, [c_void_p, c_void_p, c_uint64]),
    "b200q_last_route": (c_int32, [c_void_p, POINTER(c_int32), POINTER(c_int32)]),
    "b200q_weight_upload": (c_int32, [c_void_p, c_int32, c_int64, c_int64, c_void_p, c_size_t, POINTER(c_void_p)]),
    "b200q_weight_upload_shard": (
        c_int32,
        [c_void_p, c_int32, c_int64, c_int64, c_void_p, c_size_t, c_int32, c_int32, c_int32, c_int64, POINTER(c_void_p)],
    ),
    "b200q_shard_range": (
        c_int32,
        [c_int32, c_int64, c_int64, c_int32, c_int32, c_int32, c_int64, POINTER(c_int64), POINTER(c_int64)],
    ),
    "b200q_layout_row_bytes": (c_int64, [c_int32, c_int64]),
    "b200q_layout_pack": (c_int32, [c_int32, c_int64, c_int64, c_void_p, c_size_t, c_void_p, c_size_t]),
    "b200q_weight_clone": (c_int32, [c_void_p, c_void_p, POINTER(c_void_p)]),
    "b200q_weight_info": (
        c_int32,
        [c_void_p, POINTER(c_int32), POINTER(c_int64), POINTER(c_int64), POINTER(c_size_t), POINTER(c_size_t)],
    ),
    "b200q_weight_destroy": (None, [c_void_p]),
    "b200q_dequantize": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p]),
    "b200q_matmul": (
        c_int32,
        [c_void_p, c_void_p, c_void_p, c_int32, c_int64, c_int64, c_void_p, c_int32, c_int64, c_void_p],
    ),
    "b200q_matmul_multi": (
        c_int32,
        [c_void_p, POINTER(c_void_p), c_int32, c_void_p, c_int32, c_int64, c_int64, POINTER(c_void_p), c_int32,
         POINTER(c_int64), c_void_p],
    ),
    "b200q_matmul_host": (
        c_int32,
        [c_void_p, c_void_p, c_void_p, c_int32, c_int64, c_int64, c_void_p, c_int32, c_int64],
    ),
    "b200q_matmul_multi_host": (
        c_int32,
        [c_void_p, POINTER(c_void_p), c_int32, c_void_p, c_int32, c_int64, c_int64, POINTER(c_void_p), c_int32,
         POINTER(c_int64)],
    ),
    "b200q_matmul_prefill_noalloc": (
        c_int32,
        [c_void_p, c_void_p, c_void_p, c_int32, c_int64, c_int64, c_void_p, c_int32, c_int64, c_void_p],
    ),
    "b200q_plan_create": (c_int32, [c_void_p, POINTER(Job), c_int32, c_int64, POINTER(c_void_p)]),
    "b200q_plan_run": (c_int32, [c_void_p, c_void_p, c_void_p]),
    "b200q_plan_destroy": (None, [c_void_p]),
    "b200q_tp_unique_id": (c_int32, [c_void_p]),
    "b200q_tp_init": (c_int32, [c_void_p, c_int32, c_int32, c_void_p]),
    "b200q_allreduce": (c_int32, [c_void_p, c_void_p, c_int64, c_int32, c_void_p]),
    "b200q_tp_finalize": (c_int32, [c_void_p]),
    "b200q_peer_export": (c_int32, [c_void_p, c_void_p]),
    "b200q_peer_attach": (c_int32, [c_void_p, c_int32, c_int32, c_void_p]),
    "b200q_peer_detach": (c_int32, [c_void_p]),
    "b200q_peer_buffer": (c_int32, [c_void_p, POINTER(c_void_p)]),
    "b200q_peer_attach_buffers": (c_int32, [c_void_p, c_int32, c_int32, POINTER(c_void_p)]),
}


class GgufSummary(ctypes.Structure):
    """struct b200q_gguf_summary_t of include/b200q.h."""

    _fields_ = [("version", ctypes.c_uint32), ("alignment", ctypes.c_uint32), ("tensor_count", c_uint64),
                ("metadata_count", c_uint64), ("tensor_storage_bytes", c_uint64), ("header_bytes", c_uint64),
                ("parameter_count", c_uint64), ("file_bytes", c_uint64)]


class GgufTensor(ctypes.Structure):
    """struct b200q_gguf_tensor_t of include/b200q.h."""

    _fields_ = [("name", c_char_p), ("type", ctypes.c_uint32), ("n_dims", ctypes.c_uint32), ("dims", c_uint64 * 8),
                ("elements", c_uint64), ("bytes", c_uint64), ("file_offset", c_uint64)]


SIGNATURES.update({
    "b200q_tensor_storage_bytes_shape": (c_int64, [c_int32, c_int32, POINTER(c_int64)]),
    "b200q_quantize": (c_int32, [c_int32, c_void_p, c_int64, c_int64, c_void_p, c_size_t, c_int32]),
    "b200q_gguf_open": (c_int32, [c_char_p, POINTER(c_void_p), c_char_p, c_size_t]),
    "b200q_gguf_close": (None, [c_void_p]),
    "b200q_gguf_last_error": (c_int32, [c_void_p, c_char_p, c_size_t]),
    "b200q_gguf_summary": (c_int32, [c_void_p, POINTER(GgufSummary)]),
    "b200q_gguf_metadata_string": (c_char_p, [c_void_p, c_char_p]),
    "b200q_gguf_metadata_u64": (c_int32, [c_void_p, c_char_p, POINTER(c_uint64)]),
    "b200q_gguf_tensor_info": (c_int32, [c_void_p, c_uint64, POINTER(GgufTensor)]),
    "b200q_gguf_find": (c_int32, [c_void_p, c_char_p, POINTER(c_uint64)]),
    "b200q_gguf_read_tensor": (c_int32, [c_void_p, c_uint64, c_void_p, c_size_t]),
    "b200q_gguf_upload": (c_int32, [c_void_p, c_void_p, c_uint64, c_int32, c_int32, c_int32, c_int64, POINTER(c_void_p)]),
})


class B200QError(RuntimeError):
    """A non-zero b200q_status.  `.status` is the code, `.kind` mirrors the reference's InferenceError variants."""

    def __init__(self, status: int, message: str = ""):
        self.status = int(status)
        self.kind = STATUS_NAMES.get(self.status, f"Status{self.status}")
        super().__init__(f"b200q {self.kind} ({self.status}): {message}" if message else f"b200q {self.kind} ({self.status})")


def load_library(path: Path | str | None = None) -> ctypes.CDLL:
    p = Path(path) if path else LIB_PATH
    if not p.exists():
        raise ImportError(
            f"{p} is missing: build it with `make -C magnitude_b200/csrc` (or __graft_entry__.build()). "
            "There is no CPU or PyTorch fallback for this path."
        )
    lib = ctypes.CDLL(str(p))
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here means the header and the library disagree
        fn.restype = restype
        fn.argtypes = argtypes
    return lib


_lib: ctypes.CDLL | None = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        _lib = load_library()
    return _lib
