"""Fused epilogues of streaming decode plans: gated MLP (silu(gate x) * (up x)) and the residual
add, alone and as the dependent layer a llama-style MLP is (gate/up -> activation -> down ->
residual), against the same plan without fusion and against the CPU oracle."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
import magnitude_b200 as mb  # noqa: E402


def _weights(orc, qt, n, k, seed):
    rng = np.random.default_rng(seed)
    return orc.quantize(qt, rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.05))


def _silu_mul(g, u):
    g = g.astype(np.float64)
    return g / (1.0 + np.exp(-g)) * u.astype(np.float64)


def _bound(ref, rel):
    return rel * np.maximum(np.abs(ref), np.sqrt(np.mean(ref ** 2)))


@pytest.mark.parametrize("qt", [mb.TYPE_Q4_K, mb.TYPE_Q6_K, mb.TYPE_Q8_0, mb.TYPE_Q5_K, mb.TYPE_Q4_0, mb.TYPE_MXFP4])
@pytest.mark.parametrize("m,n,k,out_dtype", [(1, 1024, 2048, torch.float32), (2, 771, 4096, torch.float32), (1, 5, 256, torch.bfloat16),
                                             (4, 130, 2304, torch.float32)])
def test_swiglu_job(backend, orc, qt, m, n, k, out_dtype):
    pg, pu = _weights(orc, qt, n, k, seed=n), _weights(orc, qt, n, k, seed=n + 1)
    wg, wu = backend.upload(qt, pg, n, k), backend.upload(qt, pu, n, k)
    x = torch.from_numpy(np.random.default_rng(k).standard_normal((m, k), dtype=np.float32)).cuda().to(torch.bfloat16)
    h = torch.full((m, n), 7.0, dtype=out_dtype, device="cuda")
    g, u = torch.empty((m, n), device="cuda"), torch.empty((m, n), device="cuda")
    # a second, unrelated job makes the plan use the activation prep launch and both consumer teams
    other = torch.empty((m, n), device="cuda")
    fused = backend.plan([([wg, wu], x, [h]), ([wu], x, [other])], swiglu=[True, False])
    plain = backend.plan([([wg, wu], x, [g, u]), ([wu], x, [other])])
    fused.run()
    plain.run()
    backend.sync()
    # the same sums go through the same fp32 expression: equal up to the rounding of exp
    want = _silu_mul(g.cpu().numpy(), u.cpu().numpy())
    got = h.float().cpu().numpy().astype(np.float64)
    # (with three or more rows the unfused plan runs on the skinny kernel, whose sums differ in the last bits)
    rel = (1e-5 if m <= 2 else 2e-3) if out_dtype == torch.float32 else 2.0 ** -8
    assert np.all(np.abs(got - want) <= _bound(want, rel))
    # and against the oracle: the two projections carry the decode tolerance each
    xf = x.float().cpu().numpy()
    ref = _silu_mul(orc.matmul_exact(qt, pg, n, k, xf), orc.matmul_exact(qt, pu, n, k, xf))
    assert np.all(np.abs(got - ref) <= _bound(ref, 4e-3 if out_dtype == torch.float32 else 1e-2))
    assert torch.equal(other, u)


@pytest.mark.parametrize("m", [1, 3])
def test_accumulate_job(backend, orc, m):
    n, k = 517, 2048
    p = _weights(orc, mb.TYPE_Q4_K, n, k, seed=3)
    w = backend.upload(mb.TYPE_Q4_K, p, n, k)
    x = torch.from_numpy(np.random.default_rng(4).standard_normal((m, k), dtype=np.float32)).cuda()
    res = torch.from_numpy(np.random.default_rng(5).standard_normal((m, n), dtype=np.float32)).cuda()
    y = res.clone()
    y0 = torch.empty_like(res)
    backend.plan([([w], x, [y])], accumulate=[True]).run()
    backend.plan([([w], x, [y0])]).run()
    backend.sync()
    if m <= 2:
        assert torch.equal(y, res + y0)
    else:       # the unfused plan of three rows runs on the skinny kernel: same sums up to the last bits
        want = (res + y0).cpu().numpy().astype(np.float64)
        assert np.all(np.abs(y.cpu().numpy() - want) <= _bound(y0.cpu().numpy().astype(np.float64), 1e-3))


def _rmsnorm(x, gamma, eps):
    x = x.astype(np.float64)
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps) * gamma.astype(np.float64)


@pytest.mark.parametrize("qt", [mb.TYPE_Q4_K, mb.TYPE_Q6_K, mb.TYPE_Q8_0])
@pytest.mark.parametrize("m,n,k,x_dtype", [(1, 512, 4096, torch.bfloat16), (2, 300, 2304, torch.float32), (4, 64, 256, torch.bfloat16)])
def test_rmsnorm_on_the_activation_load(backend, orc, qt, m, n, k, x_dtype):
    p = _weights(orc, qt, n, k, seed=n)
    w = backend.upload(qt, p, n, k)
    rng = np.random.default_rng(k + m)
    x = (torch.from_numpy(rng.standard_normal((m, k), dtype=np.float32)) * 3.0).cuda().to(x_dtype)
    gamma = torch.from_numpy(rng.uniform(0.5, 1.5, k).astype(np.float32)).cuda()
    eps = 1e-5
    ref = orc.matmul_exact(qt, p, n, k, _rmsnorm(x.float().cpu().numpy(), gamma.cpu().numpy(), eps).astype(np.float32))
    y_img, y_in, mid, other = (torch.empty((m, n), device="cuda") for _ in range(4))
    # two independent jobs: the activation prep launch normalises; a job that waits converts inside the kernel
    backend.plan([([w], x, [y_img]), ([w], x, [other])], norms=[gamma, None], norm_eps=eps).run()
    backend.plan([([w], x, [mid]), ([w], x, [y_in])], waits=[False, True], norms=[None, gamma], norm_eps=eps).run()
    backend.sync()
    for got in (y_img, y_in):
        g = got.cpu().numpy().astype(np.float64)
        assert np.all(np.abs(g - ref) <= _bound(ref, 1e-3))
    assert torch.equal(other, mid)            # the job without a norm weight is untouched by its neighbour's


@pytest.mark.parametrize("m", [1, 2])
def test_dependent_mlp_layer(backend, orc, m):
    """gate/up -> silu * -> down -> residual, two layers chained through the residual stream."""
    hdim, idim = 1024, 2816
    layers = []
    for l in range(2):
        layers.append((_weights(orc, mb.TYPE_Q4_K, idim, hdim, seed=10 + l), _weights(orc, mb.TYPE_Q4_K, idim, hdim, seed=20 + l),
                       _weights(orc, mb.TYPE_Q6_K, hdim, idim, seed=30 + l)))
    ws = [(backend.upload(mb.TYPE_Q4_K, g, idim, hdim), backend.upload(mb.TYPE_Q4_K, u, idim, hdim), backend.upload(mb.TYPE_Q6_K, d, hdim, idim))
          for g, u, d in layers]
    x0 = np.random.default_rng(9).standard_normal((m, hdim), dtype=np.float32)
    xs = torch.from_numpy(x0).cuda()            # the residual stream, updated in place
    hs = [torch.empty((m, idim), device="cuda") for _ in layers]
    jobs, waits, glu, acc = [], [], [], []
    for (wg, wu, wd), h in zip(ws, hs):
        jobs += [([wg, wu], xs, [h]), ([wd], h, [xs])]
        waits += [len(jobs) > 2, True]          # the next layer reads the stream the previous down wrote
        glu += [True, False]
        acc += [False, True]
    gammas = [torch.from_numpy(np.random.default_rng(40 + l).uniform(0.5, 1.5, hdim).astype(np.float32)).cuda() for l in range(2)]
    norms = [gammas[i // 2] if i % 2 == 0 else None for i in range(len(jobs))]      # pre-norm before gate/up
    plan = backend.plan(jobs, waits=waits, swiglu=glu, accumulate=acc, norms=norms, norm_eps=1e-6)
    plan.run()
    backend.sync()
    ref = x0.astype(np.float64)
    for l, (g, u, d) in enumerate(layers):
        xin = _rmsnorm(ref, gammas[l].cpu().numpy(), 1e-6).astype(np.float32)
        h = _silu_mul(orc.matmul_exact(mb.TYPE_Q4_K, g, idim, hdim, xin), orc.matmul_exact(mb.TYPE_Q4_K, u, idim, hdim, xin))
        ref = ref + orc.matmul_exact(mb.TYPE_Q6_K, d, hdim, idim, h.astype(np.float32))
    got = xs.cpu().numpy().astype(np.float64)
    assert np.all(np.abs(got - ref) <= _bound(ref, 5e-3))


def test_fused_flags_argument_checks(backend, orc):
    n, k = 64, 256
    p = _weights(orc, mb.TYPE_Q4_K, n, k, seed=1)
    w = backend.upload(mb.TYPE_Q4_K, p, n, k)
    w2 = backend.upload(mb.TYPE_Q4_K, _weights(orc, mb.TYPE_Q4_K, n + 4, k, seed=2), n + 4, k)
    x = torch.zeros((1, k), device="cuda")
    y = torch.zeros((1, n), device="cuda")
    with pytest.raises(mb.B200QError):      # one weight
        backend.plan([([w], x, [y])], swiglu=[True])
    with pytest.raises(mb.B200QError):      # unequal shapes
        backend.plan([([w, w2], x, [y])], swiglu=[True])
    x8 = torch.zeros((8, k), device="cuda", dtype=torch.bfloat16)
    y8 = torch.zeros((8, n), device="cuda")
    with pytest.raises(mb.B200QError):      # beyond the streaming plans
        backend.plan([([w, w], x8, [y8])], swiglu=[True])
    with pytest.raises(mb.B200QError):
        backend.plan([([w], x8, [y8])], accumulate=[True])
