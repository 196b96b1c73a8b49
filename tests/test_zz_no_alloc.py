"""The allocation-free prefill entry point against the ordinary one.

Some hosts of this library give the GPU a fixed memory plan per model and cannot let a kernel
library allocate behind their back (a late cudaMalloc may fail, or break the budget the model was
admitted under).  b200q_matmul_prefill_noalloc serves them: its scratch is a fixed array inside
the library.  This test calls it through the C ABI and checks it against b200q_matmul on two
calls in a row (the second call finds the first call's data in the shared scratch).

The file name sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
import magnitude_b200 as mb  # noqa: E402
from magnitude_b200 import _binding as B  # noqa: E402
from magnitude_b200 import ggml_quant as gq  # noqa: E402


def _noalloc(backend, w, x, out):
    st = B.lib().b200q_matmul_prefill_noalloc(
        backend._h, w._h, ctypes.c_void_p(x.data_ptr()), mb.TYPE_BF16 if x.dtype == torch.bfloat16 else mb.TYPE_F32,
        x.shape[0], x.stride(0), ctypes.c_void_p(out.data_ptr()), mb.TYPE_F32, out.stride(0),
        backend._stream_ptr(None))
    return st


def _check(orc, got, ref_entry, ref_oracle):
    # same kernels, same arithmetic as the ordinary entry point: within the prefill tolerance (5e-3), in practice identical
    err = (got - ref_entry).abs()
    rms = ref_entry.pow(2).mean().sqrt()
    assert torch.all(err <= 5e-3 * torch.maximum(ref_entry.abs(), rms))
    ok, worst = orc.within_tolerance(got.cpu().numpy(), ref_oracle, 5e-3)
    assert ok, f"against the CPU oracle: worst error {worst:.3f} x tolerance"


def test_noalloc_prefill_matches_ordinary_entry_point(backend, orc):
    n, k = 384, 2048
    rng = np.random.default_rng(0)
    for qt in (mb.TYPE_Q4_K, mb.TYPE_Q6_K):
        packed = gq.quantize(qt, rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02))
        w = backend.upload(qt, packed, n, k)
        # two calls in a row with different shapes and dtypes: the second overwrites the shared scratch.
        # M = 256 runs the two-CTA kernel (M >= 128, N > 128), M = 33 the one-CTA kernel.
        for m, dtype in ((256, torch.bfloat16), (33, torch.float32)):
            x = torch.from_numpy(rng.standard_normal((m, k), dtype=np.float32)).cuda().to(dtype)
            ref = backend.project(w, x)                      # ordinary entry point (context-owned scratch)
            assert backend.last_route()[0] == mb.ROUTE_GEMM
            out = torch.zeros((m, n), device="cuda")
            assert _noalloc(backend, w, x, out) == 0, backend.last_error()
            backend.sync()
            xr = x.float() if dtype == torch.bfloat16 else x.half().float()     # the route rounds fp32 activations to fp16
            _check(orc, out, ref, orc.matmul_exact(qt, packed, n, k, xr.cpu().numpy()))


def test_noalloc_prefill_limit_and_oversized_requests(backend, orc):
    n, k = 8, 8192
    rng = np.random.default_rng(1)
    packed = gq.quantize(mb.TYPE_Q4_K, rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02))
    w = backend.upload(mb.TYPE_Q4_K, packed, n, k)
    m = 513                                                   # 513 * 8192 > 4,194,304 elements
    x = torch.zeros((m, k), dtype=torch.bfloat16, device="cuda")
    out = torch.zeros((m, n), device="cuda")
    assert _noalloc(backend, w, x, out) == B.ERR_INVALID_CONFIG
    assert "scratch" in backend.last_error()
    # exactly at the limit: the whole array is in use
    ok_x = torch.from_numpy(rng.standard_normal((512, k), dtype=np.float32)).cuda().to(torch.bfloat16)
    ok_out = torch.zeros((512, n), device="cuda")
    assert _noalloc(backend, w, ok_x, ok_out) == 0
    backend.sync()
    ref = backend.project(w, ok_x)
    backend.sync()
    _check(orc, ok_out, ref, orc.matmul_exact(mb.TYPE_Q4_K, packed, n, k, ok_x.float().cpu().numpy()))
