"""GPU parity of the tensor-core prefill route (M > 16) against the CPU oracle.

Tolerance (fixed by the task statement): fp32-accumulated outputs within max relative error 5e-3
for the prefill path, "relative" meaning |err| <= rel * max(|ref|, rms(ref)).  The weights enter
the tensor cores dequantized to fp16, the activations converted to fp16, accumulation is fp32.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
import magnitude_b200 as mb  # noqa: E402
from magnitude_b200 import ggml_quant as gq  # noqa: E402

REL_PREFILL = 5e-3
TYPES = [mb.TYPE_Q4_K, mb.TYPE_Q6_K, mb.TYPE_Q8_0, mb.TYPE_Q5_K, mb.TYPE_Q4_0, mb.TYPE_MXFP4]


def _acts(m, k, seed):
    rng = np.random.default_rng(seed)
    return torch.from_numpy(rng.standard_normal((m, k), dtype=np.float32)).cuda().to(torch.bfloat16)


@pytest.mark.parametrize("qt", TYPES)
@pytest.mark.parametrize("m,n,k", [(24, 128, 256), (20, 128, 512), (64, 256, 1024), (17, 130, 768), (100, 3, 2304),
                                   (300, 260, 5120), (512, 384, 4096)])
def test_prefill_small_shapes(backend, orc, qt, m, n, k):
    rng = np.random.default_rng(m + n + k)
    packed = orc.quantize(qt, rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02))
    w = backend.upload(qt, packed, n, k)
    x = _acts(m, k, seed=m)
    y32 = backend.project(w, x)
    assert backend.last_route()[0] == mb.ROUTE_GEMM
    y16 = backend.project(w, x, out_dtype=torch.bfloat16)
    backend.sync()
    ref = orc.matmul_exact(qt, packed, n, k, x.float().cpu().numpy())
    ok, worst = orc.within_tolerance(y32.cpu().numpy(), ref, REL_PREFILL)
    assert ok, f"fp32 out: worst error {worst:.3f} x tolerance"
    ok, worst = orc.within_tolerance(y16.float().cpu().numpy(), ref, REL_PREFILL)
    assert ok, f"bf16 out: worst error {worst:.3f} x tolerance"


def test_prefill_fp32_activations_and_strided_output(backend, orc):
    m, n, k = 40, 200, 1024
    rng = np.random.default_rng(9)
    packed = orc.quantize(mb.TYPE_Q4_K, rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02))
    w = backend.upload(mb.TYPE_Q4_K, packed, n, k)
    x = torch.from_numpy(rng.standard_normal((m, k), dtype=np.float32)).cuda()
    big = torch.full((m, n + 24), 7.0, device="cuda")
    out = big[:, :n]
    backend.project(w, x, out=out)
    backend.sync()
    xb = x.half().float().cpu().numpy()                  # the route rounds fp32 activations to fp16
    ref = orc.matmul_exact(mb.TYPE_Q4_K, packed, n, k, xb)
    assert orc.within_tolerance(out.cpu().numpy(), ref, REL_PREFILL)[0]
    assert torch.all(big[:, n:] == 7.0)                  # nothing written past the row


def test_prefill_q8_0_ragged_k(backend, orc):
    m, n, k = 33, 140, 288
    rng = np.random.default_rng(3)
    packed = orc.quantize(mb.TYPE_Q8_0, rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02))
    w = backend.upload(mb.TYPE_Q8_0, packed, n, k)
    x = _acts(m, k, 4)
    y = backend.project(w, x)
    backend.sync()
    ref = orc.matmul_exact(mb.TYPE_Q8_0, packed, n, k, x.float().cpu().numpy())
    assert orc.within_tolerance(y.cpu().numpy(), ref, REL_PREFILL)[0]


def test_config4_prefill_with_outlier_channels(backend, orc):
    # M = 2048, K = 4096, N = 14336, 1 % of the channels scaled x20; bf16 output.
    # The full product is checked on a sample of 192 weight rows (the oracle is a CPU loop).
    m, n, k = 2048, 14336, 4096
    packed = gq.synth_weights(mb.TYPE_Q4_K, n, k, seed=0, encoder=orc.quantize)      # the restated reference quantizer
    x = np.random.default_rng(1).standard_normal((m, k), dtype=np.float32)
    ch = np.random.default_rng(2).choice(k, size=41, replace=False)
    x[:, ch] *= 20.0
    xt = torch.from_numpy(x).cuda().to(torch.bfloat16)
    w = backend.upload(mb.TYPE_Q4_K, packed, n, k)
    y = backend.project(w, xt, out_dtype=torch.bfloat16)
    backend.sync()
    rows = np.sort(np.random.default_rng(3).choice(n, size=192, replace=False))
    ref = orc.matmul_exact(mb.TYPE_Q4_K, packed[rows], len(rows), k, xt.float().cpu().numpy())
    got = y[:, torch.from_numpy(rows).cuda()].float().cpu().numpy()
    ok, worst = orc.within_tolerance(got, ref, REL_PREFILL)
    assert ok, f"worst error {worst:.3f} x tolerance"
    # size-independent property on the whole output: linear in the activation
    y2 = backend.project(w, (xt.float() * 0.5).to(torch.bfloat16), out_dtype=torch.bfloat16)
    backend.sync()
    assert torch.allclose(y2.float(), y.float() * 0.5, rtol=2e-2, atol=1e-3)
