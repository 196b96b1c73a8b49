"""GPU parity of the skinny-batch route (3 <= M <= 16, and M = 2 when asked for) against the CPU
oracle, through the C ABI.

Tolerance (fixed by the task statement): fp32-accumulated outputs of a decode-sized batch (M <= 16,
fp32 output) within max relative error 1e-3, "relative" meaning |err| <= rel * max(|ref|, rms(ref)).
The route multiplies exact integer weights by the exact bf16 activations and scales in fp32, so it
sits far inside that bound; bf16 outputs are held to the 5e-3 of a rounded output.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
import magnitude_b200 as mb  # noqa: E402
from magnitude_b200 import _binding as B  # noqa: E402

REL_DECODE = 1e-3
REL_BF16 = 5e-3
TYPES = [mb.TYPE_Q4_K, mb.TYPE_Q6_K, mb.TYPE_Q8_0, mb.TYPE_Q5_K, mb.TYPE_Q4_0, mb.TYPE_MXFP4]


def _acts(m, k, seed, dtype=None):
    rng = np.random.default_rng(seed)
    return torch.from_numpy(rng.standard_normal((m, k), dtype=np.float32)).cuda().to(dtype or torch.bfloat16)


def _weights(orc, qt, n, k, seed):
    rng = np.random.default_rng(seed)
    return orc.quantize(qt, rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02))


@pytest.mark.parametrize("qt", TYPES)
@pytest.mark.parametrize("m", [5, 8, 9, 16])
@pytest.mark.parametrize("n,k", [(1, 256), (16, 512), (19, 2048), (130, 2304), (301, 5120), (64, 4096), (40, 16640)])
def test_skinny_small_shapes(backend, orc, qt, m, n, k):
    # one chunk, whole chunks, a short last chunk (2304 = 9 records, 5120 = 20), many chunks; rows that
    # do not fill a 16-row block or a 4-row group
    packed = _weights(orc, qt, n, k, seed=3 * n + k + m)
    w = backend.upload(qt, packed, n, k)
    x = _acts(m, k, seed=m)
    y = backend.project(w, x)
    assert backend.last_route()[0] == mb.ROUTE_SKINNY
    y16 = backend.project(w, x, out_dtype=torch.bfloat16)
    backend.sync()
    ref = orc.matmul_exact(qt, packed, n, k, x.float().cpu().numpy())
    ok, worst = orc.within_tolerance(y.cpu().numpy(), ref, REL_DECODE)
    assert ok, f"fp32 out: worst error {worst:.3f} x tolerance"
    ok, worst = orc.within_tolerance(y16.float().cpu().numpy(), ref, REL_BF16)
    assert ok, f"bf16 out: worst error {worst:.3f} x tolerance"


@pytest.mark.parametrize("qt", TYPES)
@pytest.mark.parametrize("m", [5, 8, 11, 16])
def test_skinny_fp32_activations_and_strided_buffers(backend, orc, qt, m):
    # fp32 rows enter as two bf16 halves (two token slots each, at most 8 rows per launch)
    n, k = 200, 1280
    packed = _weights(orc, qt, n, k, seed=m)
    w = backend.upload(qt, packed, n, k)
    xbig = _acts(m, k + 40, seed=17, dtype=torch.float32)
    x = xbig[:, :k]
    big = torch.full((m, n + 24), 7.0, device="cuda")
    out = big[:, :n]
    backend.project(w, x, out=out)
    assert backend.last_route()[0] == mb.ROUTE_SKINNY
    backend.sync()
    ref = orc.matmul_exact(qt, packed, n, k, x.contiguous().cpu().numpy())
    ok, worst = orc.within_tolerance(out.cpu().numpy(), ref, REL_DECODE)
    assert ok, f"worst error {worst:.3f} x tolerance"
    assert torch.all(big[:, n:] == 7.0)                  # nothing written past the row


def test_skinny_q8_0_ragged_k(backend, orc):
    for k in (32, 288, 4128):
        packed = _weights(orc, mb.TYPE_Q8_0, 37, k, seed=k)
        w = backend.upload(mb.TYPE_Q8_0, packed, 37, k)
        x = _acts(7, k, seed=k)
        y = backend.project(w, x)
        backend.sync()
        ref = orc.matmul_exact(mb.TYPE_Q8_0, packed, 37, k, x.float().cpu().numpy())
        assert orc.within_tolerance(y.cpu().numpy(), ref, REL_DECODE)[0], k


@pytest.mark.parametrize("qt", TYPES)
def test_skinny_small_m_when_selected(backend, orc, qt):
    # M = 2 normally takes the dp4a kernel; the context option moves it to this route (and back)
    n, k = 150, 3072
    packed = _weights(orc, qt, n, k, seed=5)
    w = backend.upload(qt, packed, n, k)
    backend.set_option(B.OPT_SKINNY_MIN_M, 2)
    try:
        for m in (2, 3, 4):
            x = _acts(m, k, seed=m)
            y = backend.project(w, x)
            assert backend.last_route()[0] == mb.ROUTE_SKINNY
            backend.sync()
            ref = orc.matmul_exact(qt, packed, n, k, x.float().cpu().numpy())
            assert orc.within_tolerance(y.cpu().numpy(), ref, REL_DECODE)[0], m
    finally:
        backend.set_option(B.OPT_SKINNY_MIN_M, 3)
    with pytest.raises(mb.B200QError):
        backend.set_option(B.OPT_SKINNY_MIN_M, 1)
    with pytest.raises(mb.B200QError):
        backend.set_option(99, 1)


def test_skinny_multi_weights_share_the_activation(backend, orc):
    k, m = 2048, 6
    ws, packs = [], []
    for i, n in enumerate((96, 200, 33)):
        packs.append(_weights(orc, mb.TYPE_Q4_K, n, k, seed=i))
        ws.append(backend.upload(mb.TYPE_Q4_K, packs[-1], n, k))
    x = _acts(m, k, seed=2)
    outs = backend.project_multi(ws, x)
    assert backend.last_route()[0] == mb.ROUTE_SKINNY
    backend.sync()
    for o, p, w in zip(outs, packs, ws):
        ref = orc.matmul_exact(mb.TYPE_Q4_K, p, w.n, k, x.float().cpu().numpy())
        assert orc.within_tolerance(o.cpu().numpy(), ref, REL_DECODE)[0]
        assert torch.equal(o, backend.project(w, x))      # same kernel, same order of additions
    backend.sync()


def test_skinny_repeated_calls_are_bit_identical(backend, orc):
    # the chunk sums meet through a workspace and arrival counters that every launch must leave clean
    n, k, m = 333, 6144, 16
    w = backend.upload(mb.TYPE_Q6_K, _weights(orc, mb.TYPE_Q6_K, n, k, seed=1), n, k)
    x = _acts(m, k, seed=3)
    first = backend.project(w, x).clone()
    for _ in range(5):
        assert torch.equal(backend.project(w, x), first)
    backend.sync()


@pytest.mark.parametrize("qt", [mb.TYPE_Q4_K, mb.TYPE_Q6_K])
@pytest.mark.parametrize("m", [3, 8, 16])
def test_skinny_plan_of_many_products(backend, orc, qt, m):
    # more products than travel in the kernel parameters: the job table lives in device memory and the
    # chunk-sum launch shares its grid among the products.  One, two, three and seven chunks (a
    # one-chunk product needs no chunk sum and is skipped there), rows that fill no 16-row block, a bf16 output.
    shapes = [(301, 4096), (64, 2048), (19, 6144), (130, 2304), (40, 14336), (257, 4096), (16, 512)]
    x = {k: _acts(m, k, seed=k + m) for k in {k for _, k in shapes}}
    packed, ws, ys = [], [], []
    for i, (n, k) in enumerate(shapes):
        packed.append(_weights(orc, qt, n, k, seed=100 + i))
        ws.append(backend.upload(qt, packed[-1], n, k))
        ys.append(torch.full((m, n), 7.0, dtype=torch.bfloat16 if i == 2 else torch.float32, device="cuda"))
    plan = backend.plan([([w], x[k], [y]) for w, (n, k), y in zip(ws, shapes, ys)])
    for _ in range(2):
        plan.run()
        backend.sync()
        assert backend.last_route()[0] == mb.ROUTE_SKINNY
        for i, (n, k) in enumerate(shapes):
            ref = orc.matmul_exact(qt, packed[i], n, k, x[k].float().cpu().numpy())
            ok, worst = orc.within_tolerance(ys[i].float().cpu().numpy(), ref, REL_BF16 if i == 2 else REL_DECODE)
            assert ok, f"product {i} ({n}x{k}): worst error {worst:.3f} x tolerance"
            assert torch.equal(ys[i], backend.project(ws[i], x[k], out_dtype=ys[i].dtype)), f"product {i}: plan and single call differ"


@pytest.mark.parametrize("m", [5, 16])
def test_skinny_plan_with_dependent_job(backend, orc, m):
    # gate/up share x; down reads what they wrote (a new launch, so stream order is the dependency)
    k0, n0, n1 = 1024, 2048, 300
    pg, pu = _weights(orc, mb.TYPE_Q4_K, n0, k0, 1), _weights(orc, mb.TYPE_Q4_K, n0, k0, 2)
    pd = _weights(orc, mb.TYPE_Q6_K, n1, n0, 3)
    g, u = backend.upload(mb.TYPE_Q4_K, pg, n0, k0), backend.upload(mb.TYPE_Q4_K, pu, n0, k0)
    d = backend.upload(mb.TYPE_Q6_K, pd, n1, n0)
    x = _acts(m, k0, seed=4)
    yg = torch.zeros((m, n0), dtype=torch.bfloat16, device="cuda")
    yu = torch.zeros((m, n0), dtype=torch.bfloat16, device="cuda")
    out = torch.zeros((m, n1), device="cuda")
    plan = backend.plan([([g, u], x, [yg, yu]), ([d], yg, [out])], waits=[False, True])
    for _ in range(3):
        out.zero_()
        plan.run()
        backend.sync()
        assert backend.last_route()[0] == mb.ROUTE_SKINNY
        ref = orc.matmul_exact(mb.TYPE_Q6_K, pd, n1, n0, yg.float().cpu().numpy())
        assert orc.within_tolerance(out.cpu().numpy(), ref, REL_DECODE)[0]
    ref_g = orc.matmul_exact(mb.TYPE_Q4_K, pg, n0, k0, x.float().cpu().numpy())
    assert orc.within_tolerance(yg.float().cpu().numpy(), ref_g, REL_BF16)[0]
    with pytest.raises(mb.B200QError):
        backend.plan([([g], _acts(17, k0, 1), [torch.zeros((17, n0), device="cuda")])])    # more than 16 rows


@pytest.mark.parametrize("qt,n,k", [(mb.TYPE_Q4_K, 6144, 4096), (mb.TYPE_Q6_K, 4096, 14336)])
def test_config3_verify_batches_full_size(backend, orc, qt, n, k):
    # configs[2]: fused QKV Q4_K 6144 x 4096 and down Q6_K 4096 x 14336, M in {2, 4, 8, 16}, weights from
    # the restated reference quantizer on N(0, 0.02), bf16 N(0, 1) tokens, fp32 out, 1e-3
    rng = np.random.default_rng(0)
    packed = orc.quantize(qt, rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02))
    w = backend.upload(qt, packed, n, k)
    xs = _acts(16, k, seed=1)
    ref = orc.matmul_exact(qt, packed, n, k, xs.float().cpu().numpy())
    for m in (2, 4, 8, 16):
        y = backend.project(w, xs[:m])
        backend.sync()
        ok, worst = orc.within_tolerance(y.cpu().numpy(), ref[:m], REL_DECODE)
        assert ok, f"M={m} (route {backend.last_route()[0]}): worst error {worst:.3f} x tolerance"
    backend.set_option(B.OPT_SKINNY_MIN_M, 2)
    try:
        for m in (2, 4):
            y = backend.project(w, xs[:m])
            backend.sync()
            ok, worst = orc.within_tolerance(y.cpu().numpy(), ref[:m], REL_DECODE)
            assert ok, f"M={m} on the skinny route: worst error {worst:.3f} x tolerance"
    finally:
        backend.set_option(B.OPT_SKINNY_MIN_M, 3)
