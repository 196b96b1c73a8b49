"""GPU parity: the CUDA path through the C ABI against the CPU oracle and the golden vectors.

Tolerances (fixed by the task statement): dequantized weights bit-exact; fp32-accumulated
outputs within max relative error 1e-3 for M <= 16 (fp32 output) and 5e-3 for bf16 output, where
"relative" is |err| <= rel * max(|ref|, rms(ref)).
"""
from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
import magnitude_b200 as mb  # noqa: E402
from magnitude_b200 import ggml_quant as gq  # noqa: E402

GOLD = Path(__file__).resolve().parent / "golden" / "ggml_blocks.npz"
TYPES = [mb.TYPE_Q4_K, mb.TYPE_Q6_K, mb.TYPE_Q8_0, mb.TYPE_Q5_K, mb.TYPE_Q4_0, mb.TYPE_MXFP4]
REL_DECODE = 1e-3
REL_BF16 = 5e-3


def _weights(orc, qt, n, k, seed, use_oracle_quantizer=True):
    rng = np.random.default_rng(seed)
    w = rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02)
    return orc.quantize(qt, w) if use_oracle_quantizer else gq.quantize(qt, w)


def _acts(m, k, seed, dtype):
    rng = np.random.default_rng(seed)
    x = torch.from_numpy(rng.standard_normal((m, k), dtype=np.float32)).cuda()
    return x.to(dtype)


@pytest.mark.parametrize("qt", TYPES)
def test_dequantize_golden_bit_exact(backend, qt):
    g = np.load(GOLD)
    packed = g[f"packed_{qt}"]
    n, k = packed.shape[0], 768
    w = backend.upload(qt, packed, n, k)
    got = backend.dequantize(w).cpu().numpy()
    assert np.array_equal(got.view(np.uint32), g[f"dequant_{qt}"].view(np.uint32))


@pytest.mark.parametrize("qt", TYPES)
@pytest.mark.parametrize("n,k", [(1, 256), (3, 512), (37, 2304), (64, 5120)])
def test_dequantize_matches_oracle(backend, orc, qt, n, k):
    packed = _weights(orc, qt, n, k, seed=n + k)
    w = backend.upload(qt, packed, n, k)
    got = backend.dequantize(w).cpu().numpy()
    ref = orc.dequantize(qt, packed, k)
    assert np.array_equal(got.view(np.uint32), ref.view(np.uint32))


def test_dequantize_q8_0_ragged_k(backend, orc):
    # Q8_0 rows need only be a multiple of 32 weights; the device layout pads them to 256
    for k in (32, 96, 288):
        packed = _weights(orc, mb.TYPE_Q8_0, 5, k, seed=k)
        w = backend.upload(mb.TYPE_Q8_0, packed, 5, k)
        got = backend.dequantize(w).cpu().numpy()
        assert np.array_equal(got.view(np.uint32), orc.dequantize(mb.TYPE_Q8_0, packed, k).view(np.uint32))


@pytest.mark.parametrize("qt", TYPES)
@pytest.mark.parametrize("m", [1, 2, 3, 4])
@pytest.mark.parametrize("n,k", [(1, 256), (2, 512), (3, 768), (17, 4096), (301, 2304), (130, 5120)])
def test_decode_small_shapes(backend, orc, qt, m, n, k):
    packed = _weights(orc, qt, n, k, seed=7 * n + k + m)
    w = backend.upload(qt, packed, n, k)
    x = _acts(m, k, seed=m, dtype=torch.bfloat16)
    y = backend.project(w, x)
    backend.sync()
    assert backend.last_route()[0] == (mb.ROUTE_GEMV if m <= 2 else mb.ROUTE_SKINNY)
    ref = orc.matmul_exact(qt, packed, n, k, x.float().cpu().numpy())
    ok, worst = orc.within_tolerance(y.cpu().numpy(), ref, REL_DECODE)
    assert ok, f"worst error {worst:.3f} x tolerance"


@pytest.mark.parametrize("qt", TYPES)
def test_decode_fp32_activation_and_bf16_output(backend, orc, qt):
    n, k = 96, 1024
    packed = _weights(orc, qt, n, k, seed=3)
    w = backend.upload(qt, packed, n, k)
    x = _acts(2, k, seed=9, dtype=torch.float32)
    ref = orc.matmul_exact(qt, packed, n, k, x.cpu().numpy())
    y32 = backend.project(w, x)
    y16 = backend.project(w, x, out_dtype=torch.bfloat16)
    backend.sync()
    assert orc.within_tolerance(y32.cpu().numpy(), ref, REL_DECODE)[0]
    assert orc.within_tolerance(y16.float().cpu().numpy(), ref, REL_BF16)[0]


def test_q8_0_ragged_k_product(backend, orc):
    for k in (32, 160, 4128):
        packed = _weights(orc, mb.TYPE_Q8_0, 9, k, seed=k)
        w = backend.upload(mb.TYPE_Q8_0, packed, 9, k)
        x = _acts(1, k, seed=k, dtype=torch.float32)
        y = backend.project(w, x)
        backend.sync()
        ref = orc.matmul_exact(mb.TYPE_Q8_0, packed, 9, k, x.cpu().numpy())
        assert orc.within_tolerance(y.cpu().numpy(), ref, REL_DECODE)[0]


def test_config1_q8_0_reference_cpu_case(backend, orc):
    # 4096 x 4096 Q8_0, fp32 activation, fp32 output
    n = k = 4096
    rng = np.random.default_rng(0)
    packed = orc.quantize(mb.TYPE_Q8_0, rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02))
    x = np.random.default_rng(1).standard_normal((1, k), dtype=np.float32)
    w = backend.upload(mb.TYPE_Q8_0, packed, n, k)
    y = backend.project(w, torch.from_numpy(x).cuda())
    backend.sync()
    ref = orc.matmul_exact(mb.TYPE_Q8_0, packed, n, k, x)
    ok, worst = orc.within_tolerance(y.cpu().numpy(), ref, REL_DECODE)
    assert ok, worst


@pytest.mark.parametrize("n,k", [(14336, 4096), (4096, 14336)])
def test_config2_q4_k_decode_full_size(backend, orc, n, k):
    packed = gq.synth_weights(mb.TYPE_Q4_K, n, k, seed=0, encoder=orc.quantize)      # the restated reference quantizer
    w = backend.upload(mb.TYPE_Q4_K, packed, n, k)
    x = _acts(1, k, seed=1, dtype=torch.bfloat16)
    y = backend.project(w, x)
    backend.sync()
    ref = orc.matmul_exact(mb.TYPE_Q4_K, packed, n, k, x.float().cpu().numpy())
    ok, worst = orc.within_tolerance(y.cpu().numpy(), ref, REL_DECODE)
    assert ok, worst
    # dequantized weights of the full tensor, bit for bit
    got = backend.dequantize(w).cpu().numpy()
    assert np.array_equal(got.view(np.uint32), orc.dequantize(mb.TYPE_Q4_K, packed, k).view(np.uint32))


def test_linearity_full_size(backend, orc):
    # size-independent property: W(a*x1 + x2) = a*W x1 + W x2 (up to the decode tolerance)
    n, k = 4096, 14336
    packed = gq.synth_weights(mb.TYPE_Q6_K, n, k, seed=6, encoder=orc.quantize)
    w = backend.upload(mb.TYPE_Q6_K, packed, n, k)
    x1 = _acts(1, k, seed=11, dtype=torch.float32)
    x2 = _acts(1, k, seed=12, dtype=torch.float32)
    y1, y2 = backend.project(w, x1), backend.project(w, x2)
    y3 = backend.project(w, 2.0 * x1 + x2)
    backend.sync()
    ref = (2.0 * y1 + y2).cpu().numpy()
    err = np.abs(y3.cpu().numpy() - ref)
    rms = np.sqrt(np.mean(ref ** 2))
    assert np.all(err <= 2e-3 * np.maximum(np.abs(ref), rms))


def test_multi_weight_launch_matches_single(backend, orc):
    k = 2048
    ps = [_weights(orc, mb.TYPE_Q4_K, n, k, seed=n) for n in (129, 64, 7)]
    ws = [backend.upload(mb.TYPE_Q4_K, p, p.shape[0], k) for p in ps]
    x = _acts(1, k, seed=5, dtype=torch.bfloat16)
    outs = backend.project_multi(ws, x)
    singles = [backend.project(w, x) for w in ws]
    backend.sync()
    for a, b in zip(outs, singles):
        assert torch.equal(a, b)


def test_host_buffer_path(backend, orc):
    n, k = 200, 1536
    packed = _weights(orc, mb.TYPE_Q6_K, n, k, seed=2)
    w = backend.upload(mb.TYPE_Q6_K, packed, n, k)
    x = np.random.default_rng(3).standard_normal((2, k), dtype=np.float32)
    y = backend.project_host(w, x)
    ref = orc.matmul_exact(mb.TYPE_Q6_K, packed, n, k, x)
    assert orc.within_tolerance(y, ref, REL_DECODE)[0]
    xb = gq.f32_to_bf16_bits(x)
    yb = backend.project_host(w, xb, x_dtype=mb.TYPE_BF16)
    refb = orc.matmul_exact(mb.TYPE_Q6_K, packed, n, k, orc.bf16_to_f32(xb))
    assert orc.within_tolerance(yb, refb, REL_DECODE)[0]


def test_edge_cases_and_errors(backend, orc):
    k = 512
    packed = _weights(orc, mb.TYPE_Q4_K, 8, k, seed=1)
    w = backend.upload(mb.TYPE_Q4_K, packed, 8, k)
    # M = 0 is a no-op
    x0 = torch.empty((0, k), dtype=torch.bfloat16, device="cuda")
    assert backend.project(w, x0).shape == (0, 8)
    # N = 0
    w0 = backend.upload(mb.TYPE_Q4_K, np.zeros((0,), np.uint8), 0, k)
    assert backend.project(w0, _acts(1, k, 0, torch.bfloat16)).shape == (1, 0)
    # all-zero activation -> exact zeros; non-finite activation -> non-finite output, no hang
    z = backend.project(w, torch.zeros((1, k), dtype=torch.bfloat16, device="cuda"))
    backend.sync()
    assert torch.count_nonzero(z) == 0
    bad = _acts(1, k, 4, torch.float32)
    bad[0, 17] = float("inf")
    yb = backend.project(w, bad)
    backend.sync()
    assert not torch.isfinite(yb).all()
    # errors: bad type, K not a block multiple, wrong byte count, wrong dtype
    with pytest.raises(mb.B200QError) as e:
        backend.upload(3, packed, 8, k)      # Q4_1: a ggml type this library does not multiply
    assert e.value.status == 1
    with pytest.raises(mb.B200QError):
        backend.upload(mb.TYPE_Q4_K, packed, 8, k + 32)
    with pytest.raises(mb.B200QError):
        backend.upload(mb.TYPE_Q4_K, packed[:, :-1], 8, k)
    with pytest.raises(mb.B200QError):
        backend.project(w, torch.zeros((1, k), dtype=torch.float16, device="cuda"))
    # the context stays usable after errors
    y = backend.project(w, _acts(1, k, 8, torch.bfloat16))
    backend.sync()
    assert torch.isfinite(y).all()


def test_one_hot_sub_blocks(backend, orc):
    # every sub-block index separately: an activation that is non-zero in one 16-weight slice
    k = 512
    for qt in TYPES:
        packed = _weights(orc, qt, 4, k, seed=qt)
        w = backend.upload(qt, packed, 4, k)
        wf = orc.dequantize(qt, packed, k).astype(np.float64)
        xs = np.zeros((k // 16, k), dtype=np.float32)
        for j in range(k // 16):
            xs[j, 16 * j:16 * j + 16] = 1.0 + 0.25 * (j % 3)
        for j0 in range(0, k // 16, 4):
            x = torch.from_numpy(xs[j0:j0 + 4]).cuda()
            y = backend.project(w, x)
            backend.sync()
            ref = xs[j0:j0 + 4].astype(np.float64) @ wf.T
            assert np.allclose(y.cpu().numpy(), ref, rtol=1e-3, atol=1e-6), (qt, j0)


def test_plan_matches_single_calls_mixed_types(backend, orc):
    k = 2048
    gate = backend.upload(mb.TYPE_Q4_K, _weights(orc, mb.TYPE_Q4_K, 300, k, 1), 300, k)
    up = backend.upload(mb.TYPE_Q4_K, _weights(orc, mb.TYPE_Q4_K, 300, k, 2), 300, k)
    v = backend.upload(mb.TYPE_Q6_K, _weights(orc, mb.TYPE_Q6_K, 65, k, 3), 65, k)
    q8 = backend.upload(mb.TYPE_Q8_0, _weights(orc, mb.TYPE_Q8_0, 33, 1024, 4), 33, 1024)
    x1 = _acts(1, k, 5, torch.bfloat16)
    x2 = _acts(1, 1024, 6, torch.float32)
    outs = [torch.zeros((1, n), device="cuda") for n in (300, 300, 65, 33)]
    plan = backend.plan([([gate, up], x1, outs[0:2]), ([v], x1, outs[2:3]), ([q8], x2, outs[3:4])])
    plan.run()
    backend.sync()
    # one streaming launch for the whole plan, preceded by the small activation-prep launch
    assert backend.last_route() == (mb.ROUTE_GEMV, 2)
    singles = [backend.project(gate, x1), backend.project(up, x1), backend.project(v, x1), backend.project(q8, x2)]
    backend.sync()
    for a, b in zip(outs, singles):
        assert torch.equal(a, b)
    # a second run after rewriting the activation in place
    x1.copy_(_acts(1, k, 7, torch.bfloat16))
    plan.run()
    backend.sync()
    ref = orc.matmul_exact(mb.TYPE_Q6_K, _weights(orc, mb.TYPE_Q6_K, 65, k, 3), 65, k, x1.float().cpu().numpy())
    assert orc.within_tolerance(outs[2].cpu().numpy(), ref, REL_DECODE)[0]


@pytest.mark.parametrize("m", [1, 2])
def test_plan_with_dependent_job(backend, orc, m):
    # job 1 reads what job 0 wrote: every CTA must have stored job 0's rows first
    k0, n0, n1 = 1024, 4096, 512
    p0 = _weights(orc, mb.TYPE_Q4_K, n0, k0, 11)
    p1 = _weights(orc, mb.TYPE_Q4_K, n1, n0, 12)
    w0 = backend.upload(mb.TYPE_Q4_K, p0, n0, k0)
    w1 = backend.upload(mb.TYPE_Q4_K, p1, n1, n0)
    x = _acts(m, k0, 13, torch.bfloat16)
    mid = torch.zeros((m, n0), device="cuda")
    out = torch.zeros((m, n1), device="cuda")
    plan = backend.plan([([w0], x, [mid]), ([w1], mid, [out])], waits=[False, True])
    for _ in range(3):
        mid.zero_()
        out.zero_()
        plan.run()
        backend.sync()
        ref_mid = backend.project(w0, x)
        ref_out = backend.project(w1, ref_mid)
        backend.sync()
        assert torch.equal(mid, ref_mid)
        assert torch.equal(out, ref_out)
    ref = orc.matmul_exact(mb.TYPE_Q4_K, p1, n1, n0, mid.cpu().numpy())
    assert orc.within_tolerance(out.cpu().numpy(), ref, REL_DECODE)[0]


@pytest.mark.parametrize("m", [1, 2])
def test_plan_alternating_independent_and_dependent_jobs(backend, orc, m):
    # six jobs: three layers of gate/up (own input, converted once by the prep launch) and down (reads
    # what gate wrote: converted inside the launch after the grid-wide wait).  The activation areas of
    # consecutive jobs are refilled in lock step with the consumers, whatever the mix.
    k0, n0, n1 = 1024, 2048, 256
    layers = []
    for l in range(3):
        pg, pu = _weights(orc, mb.TYPE_Q4_K, n0, k0, 20 + l), _weights(orc, mb.TYPE_Q4_K, n0, k0, 30 + l)
        pd = _weights(orc, mb.TYPE_Q4_K, n1, n0, 40 + l)
        layers.append((backend.upload(mb.TYPE_Q4_K, pg, n0, k0), backend.upload(mb.TYPE_Q4_K, pu, n0, k0),
                       backend.upload(mb.TYPE_Q4_K, pd, n1, n0)))
    xs = [_acts(m, k0, 50 + l, torch.bfloat16) for l in range(3)]
    ygs = [torch.zeros((m, n0), device="cuda") for _ in range(3)]
    yus = [torch.zeros((m, n0), device="cuda") for _ in range(3)]
    outs = [torch.zeros((m, n1), device="cuda") for _ in range(3)]
    jobs, waits = [], []
    for l, (g, u, d) in enumerate(layers):
        jobs += [([g, u], xs[l], [ygs[l], yus[l]]), ([d], ygs[l], [outs[l]])]
        waits += [False, True]
    plan = backend.plan(jobs, waits=waits)
    for _ in range(3):
        for t in ygs + yus + outs:
            t.zero_()
        plan.run()
        backend.sync()
        for l, (g, u, d) in enumerate(layers):
            rg, ru = backend.project(g, xs[l]), backend.project(u, xs[l])
            rd = backend.project(d, rg)
            backend.sync()
            assert torch.equal(ygs[l], rg) and torch.equal(yus[l], ru)
            assert torch.equal(outs[l], rd)


def test_plan_argument_checks(backend, orc):
    k = 512
    w = backend.upload(mb.TYPE_Q4_K, _weights(orc, mb.TYPE_Q4_K, 8, k, 1), 8, k)
    x = _acts(1, k, 2, torch.bfloat16)
    y = torch.zeros((1, 8), device="cuda")
    with pytest.raises(mb.B200QError):
        backend.plan([([w], _acts(17, k, 2, torch.bfloat16), [torch.zeros((17, 8), device="cuda")])])   # M > 16
    with pytest.raises(mb.B200QError):
        backend.plan([([w], x, [y, y])])
    w6 = backend.upload(mb.TYPE_Q6_K, _weights(orc, mb.TYPE_Q6_K, 8, k, 1), 8, k)
    with pytest.raises(mb.B200QError):
        backend.plan([([w, w6], x, [y, y.clone()])])   # mixed types inside one job


def test_weights_and_plans_may_outlive_their_context(orc):
    # A caller may drop the context first.  Destroying a weight or a plan afterwards must not read the
    # freed context (it used to take the device number from it, and the failed cudaSetDevice it then made
    # was reported by the next launch of another context as its own error).
    import ctypes

    from magnitude_b200 import _binding as B

    n, k = 64, 1024
    rng = np.random.default_rng(5)
    packed = orc.quantize(mb.TYPE_Q4_K, rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02))
    x = torch.from_numpy(rng.standard_normal((2, k), dtype=np.float32)).cuda().to(torch.bfloat16)
    ref = orc.matmul_exact(mb.TYPE_Q4_K, packed, n, k, x.float().cpu().numpy())

    def run_plan(be):
        w = be.upload(mb.TYPE_Q4_K, packed, n, k)
        y = torch.zeros((2, n), device="cuda")
        plan = be.plan([([w], x, [y])])
        plan.run()
        be.sync()
        assert orc.within_tolerance(y.cpu().numpy(), ref, REL_DECODE)[0]
        return w, plan

    be = mb.Backend(0)
    w, plan = run_plan(be)
    hw, hp, hc = w._h, plan._h, be._h
    w._h, plan._h, be._h = ctypes.c_void_p(), ctypes.c_void_p(), ctypes.c_void_p()     # the wrappers let go: raw C order below
    B.lib().b200q_ctx_destroy(hc)
    junk = [np.full(4096, 0x7F, np.uint8) for _ in range(64)]      # reuse the freed host block with a bad device number
    B.lib().b200q_plan_destroy(hp)
    B.lib().b200q_weight_destroy(hw)
    del junk
    be2 = mb.Backend(0)
    w2, plan2 = run_plan(be2)                                      # its activation prep launch checks the last error
    be2.close()                                                    # closes w2 and plan2 first
    assert not w2._h and not plan2._h
