"""Host-side projection interface over the b200q C ABI.

Mirrors the ownership rules of the reference executor (design/inference/engine.md:49-52 in the
reference tree): a `Backend` is owned by one thread and one GPU, weights are loaded once and stay
resident, a failed call raises and leaves the backend usable unless the device itself faulted.
PyTorch is used only to hold device memory and streams; every product runs in libb200q.so.
"""
from __future__ import annotations

import ctypes
import weakref
from ctypes import byref, c_int32, c_int64, c_size_t, c_void_p
from typing import Sequence

import numpy as np

from . import _binding as B

_TORCH_DTYPE = {}


def _torch():
    import torch

    if not _TORCH_DTYPE:
        _TORCH_DTYPE.update({torch.float32: B.TYPE_F32, torch.bfloat16: B.TYPE_BF16})
    return torch


def tensor_storage_bytes(qtype: int, n_elements: int) -> int:
    """GGUF byte count of a tensor (the rule used at inference/crates/icn-models/src/gguf.rs:129)."""
    return int(B.lib().b200q_tensor_storage_bytes(qtype, n_elements))


def shard_range(qtype: int, n: int, k: int, split: int, rank: int, world: int, align_rows: int = 0) -> tuple[int, int]:
    """Rows (column split) or weights along K (row split) that `rank` of `world` owns."""
    b, e = c_int64(), c_int64()
    st = B.lib().b200q_shard_range(qtype, n, k, split, rank, world, align_rows, byref(b), byref(e))
    if st:
        raise B.B200QError(st, f"shard_range(type={qtype}, N={n}, K={k}, split={split}, rank={rank}/{world})")
    return b.value, e.value


class ProjectionWeight:
    """A quantized W[N][K] resident on one GPU (streaming layout)."""

    def __init__(self, backend: "Backend", handle: int):
        self.backend = backend
        self._h = c_void_p(handle)
        backend._children.add(self)
        t, n, k, gb, db = c_int32(), c_int64(), c_int64(), c_size_t(), c_size_t()
        backend._check(B.lib().b200q_weight_info(self._h, byref(t), byref(n), byref(k), byref(gb), byref(db)))
        self.qtype, self.n, self.k = t.value, n.value, k.value
        self.gguf_bytes, self.device_bytes = gb.value, db.value

    def clone(self) -> "ProjectionWeight":
        out = c_void_p()
        self.backend._check(B.lib().b200q_weight_clone(self.backend._h, self._h, byref(out)))
        return ProjectionWeight(self.backend, out.value)

    def close(self) -> None:
        if self._h:
            B.lib().b200q_weight_destroy(self._h)
            self._h = c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Plan:
    """A fixed list of decode projections that one launch runs back to back (see b200q_plan_create).

    The plan keeps references to the tensors it was built from; rewrite the activation tensors in
    place and call run() again for the next token.
    """

    def __init__(self, backend: "Backend", handle: int, keep):
        self.backend = backend
        self._h = c_void_p(handle)
        self._keep = keep
        backend._children.add(self)

    def run(self, stream=None) -> None:
        self.backend._check(B.lib().b200q_plan_run(self.backend._h, self._h, self.backend._stream_ptr(stream)))

    def close(self) -> None:
        if self._h:
            B.lib().b200q_plan_destroy(self._h)
            self._h = c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Backend:
    """One b200q context: one GPU, one owning thread."""

    def __init__(self, device: int = 0):
        h = c_void_p()
        st = B.lib().b200q_ctx_create(device, byref(h))
        if st:
            raise B.B200QError(st, f"cannot create a context on CUDA device {device} (no CPU fallback exists)")
        self._h = h
        self.device = device
        self._children = weakref.WeakSet()      # live weights and plans: closed before the context

    # -- errors ------------------------------------------------------------------------------
    def last_error(self) -> str:
        buf = ctypes.create_string_buffer(512)
        B.lib().b200q_last_error(self._h, buf, 512)
        return buf.value.decode(errors="replace")

    def _check(self, status: int) -> None:
        if status:
            raise B.B200QError(status, self.last_error())

    def close(self) -> None:
        if self._h:
            for child in list(self._children):      # weights and plans go first, whatever order the caller drops them in
                child.close()
            B.lib().b200q_ctx_destroy(self._h)
            self._h = c_void_p()

    def set_option(self, option: int, value: int) -> None:
        """Per-context setting (B.OPT_*), e.g. the smallest M that takes the skinny route."""
        self._check(B.lib().b200q_ctx_set_option(self._h, option, value))

    def last_route(self) -> tuple[int, int]:
        r, n = c_int32(), c_int32()
        B.lib().b200q_last_route(self._h, byref(r), byref(n))
        return r.value, n.value

    def sync(self, stream=None, timeout_ms: int = 60000) -> None:
        self._check(B.lib().b200q_sync(self._h, self._stream_ptr(stream), timeout_ms))

    # -- weights -----------------------------------------------------------------------------
    def upload(self, qtype: int, packed: np.ndarray, n: int, k: int) -> ProjectionWeight:
        packed = np.ascontiguousarray(packed, dtype=np.uint8)
        out = c_void_p()
        self._check(B.lib().b200q_weight_upload(self._h, qtype, n, k, packed.ctypes.data, packed.size, byref(out)))
        return ProjectionWeight(self, out.value)

    def upload_shard(self, qtype: int, packed: np.ndarray, n: int, k: int, split: int, rank: int, world: int,
                     align_rows: int = 0) -> ProjectionWeight:
        packed = np.ascontiguousarray(packed, dtype=np.uint8)
        out = c_void_p()
        self._check(
            B.lib().b200q_weight_upload_shard(
                self._h, qtype, n, k, packed.ctypes.data, packed.size, split, rank, world, align_rows, byref(out)
            )
        )
        return ProjectionWeight(self, out.value)

    # -- device-pointer path (torch tensors hold the memory) ---------------------------------
    @staticmethod
    def _stream_ptr(stream) -> c_void_p:
        if stream is None:
            torch = _torch()
            if torch.cuda.is_available() and torch.cuda.is_initialized():
                return c_void_p(torch.cuda.current_stream().cuda_stream)
            return c_void_p(0)
        if isinstance(stream, int):
            return c_void_p(stream)
        return c_void_p(stream.cuda_stream)

    def dequantize(self, w: ProjectionWeight, stream=None):
        torch = _torch()
        out = torch.empty((w.n, w.k), dtype=torch.float32, device=f"cuda:{self.device}")
        self._check(B.lib().b200q_dequantize(self._h, w._h, c_void_p(out.data_ptr()), self._stream_ptr(stream)))
        return out

    def project(self, w: ProjectionWeight, x, out=None, out_dtype=None, stream=None):
        """y[M, N] = x[M, K] @ W^T for a CUDA tensor x (bf16 or fp32); returns a CUDA tensor."""
        torch = _torch()
        if x.dim() == 1:
            x = x.unsqueeze(0)
        if x.stride(-1) != 1:
            x = x.contiguous()
        m = x.shape[0]
        xd = _TORCH_DTYPE.get(x.dtype)
        if xd is None:
            raise B.B200QError(B.ERR_INVALID_CONFIG, f"activation dtype {x.dtype} is not bf16/fp32")
        if out is None:
            out = torch.empty((m, w.n), dtype=out_dtype or torch.float32, device=x.device)
        yd = _TORCH_DTYPE.get(out.dtype)
        if yd is None:
            raise B.B200QError(B.ERR_INVALID_CONFIG, f"output dtype {out.dtype} is not bf16/fp32")
        ldx = x.stride(0) if m > 1 else max(x.shape[1], 1)
        ldy = out.stride(0) if m > 1 else max(out.shape[1], 1)
        self._check(
            B.lib().b200q_matmul(
                self._h, w._h, c_void_p(x.data_ptr()), xd, m, ldx, c_void_p(out.data_ptr()), yd, ldy,
                self._stream_ptr(stream),
            )
        )
        return out

    def project_multi(self, ws: Sequence[ProjectionWeight], x, outs=None, out_dtype=None, stream=None):
        """Several weights (same type and K) applied to one activation in one launch: gate+up, Q+K."""
        torch = _torch()
        if x.dim() == 1:
            x = x.unsqueeze(0)
        if x.stride(-1) != 1:
            x = x.contiguous()
        m = x.shape[0]
        xd = _TORCH_DTYPE.get(x.dtype)
        if xd is None:
            raise B.B200QError(B.ERR_INVALID_CONFIG, f"activation dtype {x.dtype} is not bf16/fp32")
        if outs is None:
            outs = [torch.empty((m, w.n), dtype=out_dtype or torch.float32, device=x.device) for w in ws]
        yd = _TORCH_DTYPE[outs[0].dtype]
        n = len(ws)
        wh = (c_void_p * n)(*[w._h for w in ws])
        yp = (c_void_p * n)(*[c_void_p(o.data_ptr()) for o in outs])
        ldy = (c_int64 * n)(*[(o.stride(0) if m > 1 else max(o.shape[1], 1)) for o in outs])
        ldx = x.stride(0) if m > 1 else max(x.shape[1], 1)
        self._check(
            B.lib().b200q_matmul_multi(
                self._h, wh, n, c_void_p(x.data_ptr()), xd, m, ldx, yp, yd, ldy, self._stream_ptr(stream)
            )
        )
        return outs

    def plan(self, jobs, waits: Sequence[bool] | None = None, sum_ranks: Sequence[bool] | None = None,
             swiglu: Sequence[bool] | None = None, accumulate: Sequence[bool] | None = None,
             norms: Sequence | None = None, norm_eps: float = 1e-5) -> Plan:
        """jobs: sequence of (weights, x, outs) with weights/outs sequences of equal length (1..4),
        x a CUDA tensor [M, K] (M <= 16, the same for every job).  waits[i] marks job i as reading
        what earlier jobs of the plan write; sum_ranks[i] marks job i's outputs as partial sums that
        the launch adds up over the attached peer ranks (row-parallel projection); swiglu[i] marks a
        job of two weights (gate, up) and ONE output that receives silu(gate x) * (up x);
        accumulate[i] makes job i add to its outputs (residual connection); norms[i], when not None,
        is a float32 CUDA tensor [K]: job i multiplies RMSNorm(x) * norms[i] instead of x."""
        torch = _torch()
        n = len(jobs)
        arr = (B.Job * n)()
        keep = []
        m = None
        for i, (ws, x, outs) in enumerate(jobs):
            if x.dim() == 1:
                x = x.unsqueeze(0)
            if x.stride(-1) != 1:
                raise B.B200QError(B.ERR_INVALID_CONFIG, "plan activations must be contiguous along K")
            if m is None:
                m = x.shape[0]
            elif m != x.shape[0]:
                raise B.B200QError(B.ERR_INVALID_CONFIG, "every job of a plan takes the same number of rows")
            glu = bool(swiglu and swiglu[i])
            if glu and len(ws) == 2 and len(outs) == 1:
                outs = [outs[0], outs[0]]
            if len(ws) != len(outs) or not 1 <= len(ws) <= 4:
                raise B.B200QError(B.ERR_INVALID_CONFIG, "a job takes 1..4 weights and as many outputs")
            j = arr[i]
            j.n_weights = len(ws)
            j.x_dtype = _TORCH_DTYPE[x.dtype]
            j.x_dev = x.data_ptr()
            j.ldx = x.stride(0) if m > 1 else max(x.shape[1], 1)
            j.y_dtype = _TORCH_DTYPE[outs[0].dtype]
            j.flags = ((B.JOB_WAITS_FOR_EARLIER if (waits and waits[i]) else 0) | (B.JOB_SUM_RANKS if (sum_ranks and sum_ranks[i]) else 0) |
                       (B.JOB_SWIGLU if glu else 0) | (B.JOB_ACCUMULATE if (accumulate and accumulate[i]) else 0))
            for k, (w, o) in enumerate(zip(ws, outs)):
                if o.dim() == 1:
                    o = o.unsqueeze(0)
                j.w[k] = w._h.value
                j.y_dev[k] = o.data_ptr()
                j.ldy[k] = o.stride(0) if m > 1 else max(o.shape[1], 1)
            gamma = norms[i] if norms else None
            if gamma is not None:
                if gamma.dtype != torch.float32 or gamma.numel() != x.shape[1] or not gamma.is_contiguous():
                    raise B.B200QError(B.ERR_INVALID_CONFIG, "a norm weight is a contiguous float32 tensor of K elements")
                j.norm_weight = gamma.data_ptr()
                j.norm_eps = norm_eps
            keep.append((list(ws), x, list(outs), gamma))
        out = c_void_p()
        self._check(B.lib().b200q_plan_create(self._h, arr, n, m or 1, byref(out)))
        return Plan(self, out.value, keep)

    # -- host-buffer path (the reference's own boundary: host in, host out) ------------------
    def project_host(self, w: ProjectionWeight, x: np.ndarray, x_dtype: int = B.TYPE_F32, out: np.ndarray | None = None,
                     y_dtype: int = B.TYPE_F32) -> np.ndarray:
        """x is a host array: float32, or uint16 holding bf16 bits when x_dtype is TYPE_BF16."""
        x = np.ascontiguousarray(x)
        if x.ndim == 1:
            x = x[None, :]
        m, k = x.shape
        if out is None:
            out = np.empty((m, w.n), dtype=np.float32 if y_dtype == B.TYPE_F32 else np.uint16)
        self._check(
            B.lib().b200q_matmul_host(
                self._h, w._h, c_void_p(x.ctypes.data), x_dtype, m, k, c_void_p(out.ctypes.data), y_dtype, max(out.shape[1], 1)
            )
        )
        return out

    def project_host_ptr(self, ws: Sequence[ProjectionWeight], x_ptr: int, x_dtype: int, m: int, ldx: int,
                         y_ptrs: Sequence[int], y_dtype: int, ldys: Sequence[int]) -> None:
        """Raw-pointer form for pinned host buffers (one launch for 1..4 weights sharing x)."""
        n = len(ws)
        wh = (c_void_p * n)(*[w._h for w in ws])
        yp = (c_void_p * n)(*[c_void_p(p) for p in y_ptrs])
        ldy = (c_int64 * n)(*ldys)
        self._check(B.lib().b200q_matmul_multi_host(self._h, wh, n, c_void_p(x_ptr), x_dtype, m, ldx, yp, y_dtype, ldy))

    # -- tensor-parallel exchange --------------------------------------------------------------
    def tp_init(self, rank: int, world: int, unique_id: bytes) -> None:
        buf = ctypes.create_string_buffer(unique_id, 128)
        self._check(B.lib().b200q_tp_init(self._h, rank, world, buf))

    def allreduce(self, y, stream=None) -> None:
        torch = _torch()
        self._check(
            B.lib().b200q_allreduce(self._h, c_void_p(y.data_ptr()), y.numel(), _TORCH_DTYPE[y.dtype], self._stream_ptr(stream))
        )

    def tp_finalize(self) -> None:
        self._check(B.lib().b200q_tp_finalize(self._h))

    # -- peer-memory exchange (ranks = processes on one NVLink node) ---------------------------
    def peer_export(self) -> bytes:
        buf = ctypes.create_string_buffer(64)
        self._check(B.lib().b200q_peer_export(self._h, buf))
        return buf.raw

    def peer_attach(self, rank: int, world: int, handles: Sequence[bytes]) -> None:
        if len(handles) != world or any(len(h) != 64 for h in handles):
            raise ValueError("peer_attach needs one 64-byte handle per rank")
        buf = ctypes.create_string_buffer(b"".join(handles), 64 * world)
        self._check(B.lib().b200q_peer_attach(self._h, rank, world, buf))

    def peer_setup(self, dist) -> None:
        """Exchanges the handles over an initialised torch.distributed group and attaches the peers."""
        mine = self.peer_export()
        handles = [None] * dist.get_world_size()
        dist.all_gather_object(handles, mine)
        self.peer_attach(dist.get_rank(), dist.get_world_size(), handles)
        dist.barrier()

    def peer_buffer(self) -> int:
        """Device address of this context's exchange buffer (single-process form of the peer exchange)."""
        out = c_void_p()
        self._check(B.lib().b200q_peer_buffer(self._h, byref(out)))
        return out.value

    def peer_attach_buffers(self, rank: int, world: int, buffers: Sequence[int]) -> None:
        arr = (c_void_p * world)(*[c_void_p(b) for b in buffers])
        self._check(B.lib().b200q_peer_attach_buffers(self._h, rank, world, arr))

    def peer_detach(self) -> None:
        self._check(B.lib().b200q_peer_detach(self._h))

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class GgufFile:
    """A parsed GGUF header (b200q_gguf_open): tensor table, metadata, and upload of its quantized matrices.

    Mirrors what the reference's bounded inspector reads (inference/crates/icn-models/src/gguf.rs:75-149);
    parsing needs no GPU.
    """

    def __init__(self, path):
        h = c_void_p()
        err = ctypes.create_string_buffer(512)
        st = B.lib().b200q_gguf_open(str(path).encode(), byref(h), err, 512)
        if st:
            raise B.B200QError(st, err.value.decode(errors="replace"))
        self._h = h
        s = B.GgufSummary()
        B.lib().b200q_gguf_summary(self._h, byref(s))
        self.version, self.alignment = s.version, s.alignment
        self.tensor_count, self.metadata_count = s.tensor_count, s.metadata_count
        self.tensor_storage_bytes, self.header_bytes = s.tensor_storage_bytes, s.header_bytes
        self.parameter_count, self.file_bytes = s.parameter_count, s.file_bytes

    def _error(self) -> str:
        buf = ctypes.create_string_buffer(512)
        B.lib().b200q_gguf_last_error(self._h, buf, 512)
        return buf.value.decode(errors="replace")

    def metadata_string(self, key: str):
        v = B.lib().b200q_gguf_metadata_string(self._h, key.encode())
        return None if v is None else v.decode(errors="replace")

    def metadata_u64(self, key: str):
        out = ctypes.c_uint64()
        return out.value if B.lib().b200q_gguf_metadata_u64(self._h, key.encode(), byref(out)) == 0 else None

    def tensor(self, index_or_name) -> dict:
        idx = index_or_name if isinstance(index_or_name, int) else self.index_of(index_or_name)
        t = B.GgufTensor()
        st = B.lib().b200q_gguf_tensor_info(self._h, idx, byref(t))
        if st:
            raise B.B200QError(st, f"no tensor {index_or_name!r}")
        return {"index": idx, "name": t.name.decode(errors="replace"), "type": t.type, "dims": list(t.dims[: t.n_dims]),
                "elements": t.elements, "bytes": t.bytes, "file_offset": t.file_offset}

    def tensors(self) -> list:
        return [self.tensor(i) for i in range(self.tensor_count)]

    def index_of(self, name: str) -> int:
        out = ctypes.c_uint64()
        st = B.lib().b200q_gguf_find(self._h, name.encode(), byref(out))
        if st:
            raise B.B200QError(st, f"no tensor named {name!r}")
        return out.value

    def read(self, index_or_name) -> np.ndarray:
        t = self.tensor(index_or_name)
        out = np.empty(t["bytes"], dtype=np.uint8)
        st = B.lib().b200q_gguf_read_tensor(self._h, t["index"], c_void_p(out.ctypes.data), out.size)
        if st:
            raise B.B200QError(st, self._error())
        return out

    def upload(self, backend: "Backend", index_or_name, split: int = B.SPLIT_COLUMN, rank: int = 0, world: int = 1,
               align_rows: int = 0) -> ProjectionWeight:
        t = self.tensor(index_or_name)
        out = c_void_p()
        st = B.lib().b200q_gguf_upload(backend._h, self._h, t["index"], split, rank, world, align_rows, byref(out))
        if st:
            raise B.B200QError(st, self._error())
        return ProjectionWeight(backend, out.value)

    def close(self) -> None:
        if self._h:
            B.lib().b200q_gguf_close(self._h)
            self._h = c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def quantize(qtype: int, w: np.ndarray, threads: int = 0) -> np.ndarray:
    """fp32 [N, K] -> packed uint8 [N, row bytes] with the format's reference quantizer (b200q_quantize)."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    if w.ndim != 2:
        raise B.B200QError(B.ERR_INVALID_CONFIG, "quantize takes a matrix [N, K]")
    n, k = w.shape
    nbytes = tensor_storage_bytes(qtype, n * k)
    if nbytes < 0:
        raise B.B200QError(B.ERR_INVALID_CONFIG, f"type {qtype} with K = {k}: unknown type or K is not a block multiple")
    out = np.empty((n, nbytes // max(n, 1)) if n else (0, 0), dtype=np.uint8)
    st = B.lib().b200q_quantize(qtype, c_void_p(w.ctypes.data), n, k, c_void_p(out.ctypes.data), out.size, threads)
    if st:
        raise B.B200QError(st, "quantize")
    return out


def tensor_storage_bytes_shape(qtype: int, dims) -> int:
    """GGUF byte count from (type, shape), dims[0] the row length — the call at icn-models/src/gguf.rs:129."""
    arr = (c_int64 * len(dims))(*dims)
    return int(B.lib().b200q_tensor_storage_bytes_shape(qtype, len(dims), arr))


def tp_unique_id() -> bytes:
    buf = ctypes.create_string_buffer(128)
    st = B.lib().b200q_tp_unique_id(buf)
    if st:
        raise B.B200QError(st, "NCCL unique id (is libnccl.so.2 loadable?)")
    return buf.raw
