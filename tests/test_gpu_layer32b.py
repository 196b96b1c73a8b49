"""configs[4]: every projection of one decoder layer of a 32B-class dense model (Q4_K_M mix: Q4_K for
q, k, o, gate, up; Q6_K for v and down; hidden 5120, intermediate 25600, 64 q / 8 kv heads of 128),
against the CPU oracle at M = 1 (1e-3) and on sampled weight rows at M = 4096 (bf16 out, 5e-3), plus the
tensor-parallel cuts at 8 ranks (13,13,13,13,12,12,12,12 superblocks) emulated on one GPU.
Weights: N(0, 0.02) from seeds 0..6 (q, k, v, o, gate, up, down) through the restated reference quantizer."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
import magnitude_b200 as mb  # noqa: E402
from magnitude_b200 import ggml_quant as gq  # noqa: E402

H, I = 5120, 25600
LAYER = [("q", mb.TYPE_Q4_K, 8192, H), ("k", mb.TYPE_Q4_K, 1024, H), ("v", mb.TYPE_Q6_K, 1024, H), ("o", mb.TYPE_Q4_K, H, 8192),
         ("gate", mb.TYPE_Q4_K, I, H), ("up", mb.TYPE_Q4_K, I, H), ("down", mb.TYPE_Q6_K, H, I)]


@pytest.fixture(scope="module")
def layer(orc):
    return {name: gq.synth_weights(qt, n, k, seed, encoder=orc.quantize) for seed, (name, qt, n, k) in enumerate(LAYER)}


def _x(m, k, seed=1):
    return torch.from_numpy(np.random.default_rng(seed).standard_normal((m, k), dtype=np.float32)).cuda().to(torch.bfloat16)


@pytest.mark.parametrize("name,qt,n,k", LAYER)
def test_layer_projection_decode(backend, orc, layer, name, qt, n, k):
    w = backend.upload(qt, layer[name], n, k)
    x = _x(1, k)
    y = backend.project(w, x)
    backend.sync()
    ref = orc.matmul_exact(qt, layer[name], n, k, x.float().cpu().numpy())
    ok, worst = orc.within_tolerance(y.cpu().numpy(), ref, 1e-3)
    assert ok, f"{name}: worst error {worst:.3f} x tolerance"


@pytest.mark.parametrize("name,qt,n,k", LAYER)
def test_layer_projection_prefill_sampled_rows(backend, orc, layer, name, qt, n, k):
    m = 4096
    w = backend.upload(qt, layer[name], n, k)
    x = _x(m, k)
    y = backend.project(w, x, out_dtype=torch.bfloat16)
    assert backend.last_route()[0] == mb.ROUTE_GEMM
    backend.sync()
    rows = np.sort(np.random.default_rng(3).choice(n, size=32 if k > 8192 else 96, replace=False))
    ref = orc.matmul_exact(qt, layer[name][rows], len(rows), k, x.float().cpu().numpy())
    got = y[:, torch.from_numpy(rows).cuda()].float().cpu().numpy()
    ok, worst = orc.within_tolerance(got, ref, 5e-3)
    assert ok, f"{name}: worst error {worst:.3f} x tolerance"


def test_layer_cuts_for_eight_ranks(backend, orc, layer):
    # down: 100 superblocks along K -> 13,13,13,13,12,12,12,12; the partial products of the eight shards add
    # up to the full product.  gate: the same cut of the intermediate dimension taken by rows.
    name, qt, n, k = LAYER[6]
    x = _x(1, k)
    total = torch.zeros((1, n), device="cuda")
    sizes = []
    for r in range(8):
        lo, hi = mb.shard_range(qt, n, k, mb.SPLIT_ROW, r, 8)
        sizes.append((hi - lo) // 256)
        w = backend.upload_shard(qt, layer[name], n, k, mb.SPLIT_ROW, r, 8)
        total += backend.project(w, x[:, lo:hi].contiguous())
        backend.sync()
        w.close()
    assert sizes == [13, 13, 13, 13, 12, 12, 12, 12]
    ref = orc.matmul_exact(qt, layer[name], n, k, x.float().cpu().numpy())
    assert orc.within_tolerance(total.cpu().numpy(), ref, 1e-3)[0]
    name, qt, n, k = LAYER[4]
    xg = _x(1, k, seed=2)
    refg = orc.matmul_exact(qt, layer[name], n, k, xg.float().cpu().numpy())
    for r in (0, 3, 4, 7):
        lo, hi = mb.shard_range(qt, n, k, mb.SPLIT_COLUMN, r, 8, 256)
        assert (hi - lo) // 256 == sizes[r]
        w = backend.upload_shard(qt, layer[name], n, k, mb.SPLIT_COLUMN, r, 8, 256)
        y = backend.project(w, xg)
        backend.sync()
        assert orc.within_tolerance(y.cpu().numpy(), refg[:, lo:hi], 1e-3)[0]
        w.close()
    # head-aligned attention cuts: 8 query heads and 1 kv head per rank
    assert mb.shard_range(mb.TYPE_Q4_K, 8192, H, mb.SPLIT_COLUMN, 5, 8, 128) == (5120, 6144)
    assert mb.shard_range(mb.TYPE_Q6_K, 1024, H, mb.SPLIT_COLUMN, 5, 8, 128) == (640, 768)
    assert mb.shard_range(mb.TYPE_Q4_K, H, 8192, mb.SPLIT_ROW, 5, 8) == (5120, 6144)
