"""Second opinion from an independent CUDA implementation: the GGUF kernels of the vllm package in
this image (its own port of llama.cpp's dequantize and Q8_1 mat-vec kernels).  Dequantized weights
must agree to fp16 rounding; the mat-vec product, which quantizes the activation to 8 bits per
32-block as llama.cpp's GPU decode path does, must agree within that quantization's noise.  Skipped
where the package or its compiled ops are missing."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
import magnitude_b200 as mb  # noqa: E402


def _ops():
    try:
        from vllm import _custom_ops as ops
    except Exception as e:  # pragma: no cover - depends on the image
        pytest.skip(f"vllm is not importable: {e!r}"[:200])
    if not hasattr(ops, "ggml_dequantize") or not hasattr(ops, "ggml_mul_mat_vec_a8"):
        pytest.skip("this vllm build has no GGUF ops")
    return ops


def _packed(orc, qt, n, k, seed):
    rng = np.random.default_rng(seed)
    return orc.quantize(qt, rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02))


@pytest.mark.parametrize("qt", [mb.TYPE_Q4_K, mb.TYPE_Q6_K, mb.TYPE_Q8_0])
def test_dequantize_agrees_with_vllm(backend, orc, qt):
    ops = _ops()
    n, k = 256, 2048
    packed = _packed(orc, qt, n, k, seed=qt)
    w = backend.upload(qt, packed, n, k)
    ours = backend.dequantize(w).cpu().numpy()
    wv = torch.from_numpy(np.ascontiguousarray(packed).view(np.uint8).reshape(n, -1)).cuda()
    try:
        theirs = ops.ggml_dequantize(wv, qt, n, k, torch.float16)
    except Exception as e:  # pragma: no cover
        pytest.skip(f"vllm ggml_dequantize is not usable here: {e!r}"[:200])
    torch.cuda.synchronize()
    theirs = theirs.float().cpu().numpy().reshape(n, k)
    # their kernels work in fp16: every term of d * sc * q - dmin * m is rounded to 11 bits at the size of
    # the block's largest values, then the result once more
    block_max = np.abs(ours).reshape(n, k // 32, 32).max(axis=2, keepdims=True).repeat(32, axis=2).reshape(n, k)
    assert np.all(np.abs(theirs - ours) <= 2.0 ** -9 * np.abs(ours) + 2.0 ** -9 * block_max)


@pytest.mark.parametrize("qt", [mb.TYPE_Q4_K, mb.TYPE_Q6_K, mb.TYPE_Q8_0])
def test_matvec_agrees_with_vllm_within_activation_quantization(backend, orc, qt):
    ops = _ops()
    n, k = 1024, 4096
    packed = _packed(orc, qt, n, k, seed=10 + qt)
    w = backend.upload(qt, packed, n, k)
    x = torch.from_numpy(np.random.default_rng(3).standard_normal((1, k), dtype=np.float32)).cuda().to(torch.float16)
    ours = backend.project(w, x.float())
    backend.sync()
    wv = torch.from_numpy(np.ascontiguousarray(packed).view(np.uint8).reshape(n, -1)).cuda()
    try:
        theirs = ops.ggml_mul_mat_vec_a8(wv, x, qt, n)
    except Exception as e:  # pragma: no cover
        pytest.skip(f"vllm ggml_mul_mat_vec_a8 is not usable here: {e!r}"[:200])
    torch.cuda.synchronize()
    a, b = ours.cpu().numpy().astype(np.float64).reshape(-1), theirs.float().cpu().numpy().astype(np.float64).reshape(-1)
    rms = float(np.sqrt(np.mean(a * a)))
    # 8-bit activations per 32-block: relative step 1/127 of the block maximum -> about 0.6 % of the rms per output
    assert np.max(np.abs(a - b)) <= 3e-2 * rms
    assert np.sqrt(np.mean((a - b) ** 2)) <= 1e-2 * rms
    # and our result is the closer one to the exact product
    ref = orc.matmul_exact(qt, packed, n, k, x.float().cpu().numpy()).astype(np.float64).reshape(-1)
    assert np.sqrt(np.mean((a - ref) ** 2)) <= np.sqrt(np.mean((b - ref) ** 2))
