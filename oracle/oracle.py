"""ctypes front end of the CPU oracle (oracle/ggq_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the CPU-baseline leg
of the bench.  The product package never imports it.  Parity with the reference engine is
UNPINNED (its arithmetic lives in an absent third-party dependency, see the header of
ggq_oracle.c); the oracle is pinned against the independent ``gguf`` package through
tests/golden/.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path

import numpy as np

Q4_0, Q8_0, Q4_K, Q5_K, Q6_K, MXFP4 = 2, 8, 12, 13, 14, 39
TYPE_NAMES = {Q4_0: "Q4_0", Q8_0: "Q8_0", Q4_K: "Q4_K", Q5_K: "Q5_K", Q6_K: "Q6_K", MXFP4: "MXFP4"}
_HERE = Path(__file__).resolve().parent
_LIB_PATH = _HERE / "libggq_oracle.so"
_lib = None

_i64 = ctypes.c_int64
_vp = ctypes.c_void_p


def build(force: bool = False) -> Path:
    """Compile the C oracle with the committed Makefile (no-op when up to date)."""
    src = _HERE / "ggq_oracle.c"
    if force or not _LIB_PATH.exists() or _LIB_PATH.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(_HERE)], check=True, capture_output=True)
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            build()
        L = ctypes.CDLL(str(_LIB_PATH))
        L.ggq_row_bytes.restype = _i64
        L.ggq_row_bytes.argtypes = [ctypes.c_int, _i64]
        L.ggq_block_elems.restype = _i64
        L.ggq_block_bytes.restype = _i64
        L.ggq_dequantize.argtypes = [ctypes.c_int, _vp, _vp, _i64, _i64]
        L.ggq_quantize.argtypes = [ctypes.c_int, _vp, _vp, _i64, _i64]
        L.ggq_matmul_exact.argtypes = [ctypes.c_int, _vp, _i64, _i64, _vp, _i64, _i64, _vp, _i64]
        L.ggq_matmul_cpu.argtypes = [ctypes.c_int, _vp, _i64, _i64, _vp, _i64, _i64, _vp, _i64, ctypes.c_int]
        for name in ("ggq_f32_to_bf16", "ggq_bf16_to_f32", "ggq_f32_to_f16", "ggq_f16_to_f32"):
            getattr(L, name).argtypes = [_vp, _vp, _i64]
        _lib = L
    return _lib


def _ptr(a: np.ndarray) -> int:
    return a.ctypes.data


def row_bytes(qtype: int, k: int) -> int:
    rb = lib().ggq_row_bytes(qtype, k)
    if rb < 0:
        raise ValueError(f"K={k} is not a positive multiple of the {TYPE_NAMES.get(qtype, qtype)} block")
    return rb


def quantize(qtype: int, w: np.ndarray) -> np.ndarray:
    """fp32 [N, K] -> packed uint8 [N, row_bytes]."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    n, k = w.shape
    out = np.empty((n, row_bytes(qtype, k)), dtype=np.uint8)
    if lib().ggq_quantize(qtype, _ptr(w), _ptr(out), n, k):
        raise ValueError("quantize failed")
    return out


def dequantize(qtype: int, packed: np.ndarray, k: int) -> np.ndarray:
    """packed uint8 [N, row_bytes] -> fp32 [N, K]."""
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    rb = row_bytes(qtype, k)
    n = packed.size // rb
    out = np.empty((n, k), dtype=np.float32)
    if lib().ggq_dequantize(qtype, _ptr(packed), _ptr(out), n, k):
        raise ValueError("dequantize failed")
    return out


def matmul_exact(qtype: int, packed: np.ndarray, n: int, k: int, x: np.ndarray) -> np.ndarray:
    """y[M, N] = x[M, K] . dequant(W)[N, K]^T with fp64 accumulation, rounded once to fp32."""
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, k)
    m = x.shape[0]
    y = np.empty((m, n), dtype=np.float32)
    if lib().ggq_matmul_exact(qtype, _ptr(packed), n, k, _ptr(x), m, k, _ptr(y), n):
        raise ValueError("matmul_exact failed")
    return y


def matmul_cpu(qtype: int, packed: np.ndarray, n: int, k: int, x: np.ndarray, threads: int = 0) -> np.ndarray:
    """The reference-CPU-style product: activation re-quantized to 8 bit, integer block dots."""
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, k)
    m = x.shape[0]
    y = np.empty((m, n), dtype=np.float32)
    if lib().ggq_matmul_cpu(qtype, _ptr(packed), n, k, _ptr(x), m, k, _ptr(y), n, threads):
        raise ValueError("matmul_cpu failed")
    return y


def num_threads() -> int:
    return int(lib().ggq_num_threads())


def f32_to_bf16(a: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=np.float32)
    out = np.empty(a.shape, dtype=np.uint16)
    lib().ggq_f32_to_bf16(_ptr(a), _ptr(out), a.size)
    return out


def bf16_to_f32(a: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=np.uint16)
    out = np.empty(a.shape, dtype=np.float32)
    lib().ggq_bf16_to_f32(_ptr(a), _ptr(out), a.size)
    return out


def f32_to_f16(a: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=np.float32)
    out = np.empty(a.shape, dtype=np.uint16)
    lib().ggq_f32_to_f16(_ptr(a), _ptr(out), a.size)
    return out


def f16_to_f32(a: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=np.uint16)
    out = np.empty(a.shape, dtype=np.float32)
    lib().ggq_f16_to_f32(_ptr(a), _ptr(out), a.size)
    return out


def within_tolerance(got: np.ndarray, ref: np.ndarray, rel: float) -> tuple[bool, float]:
    """|got - ref| <= rel * max(|ref|, rms(ref)) element-wise.

    The relative rule is the reference comparator's (inference/crates/icn-parity/src/compare.rs:589-597:
    tolerance = max(abs_tol, rel_tol * max(|a|, |b|))) with the absolute floor tied to the output's
    rms so near-zero outputs of a zero-mean dot product do not blow the ratio up.
    Returns (ok, worst ratio of error to allowed error).
    """
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    rms = float(np.sqrt(np.mean(ref * ref))) if ref.size else 0.0
    allowed = rel * np.maximum(np.abs(ref), rms)
    err = np.abs(got - ref)
    if not np.all(np.isfinite(got)):
        return False, float("inf")
    worst = float(np.max(err / np.maximum(allowed, 1e-300))) if ref.size else 0.0
    return bool(np.all(err <= allowed)), worst
