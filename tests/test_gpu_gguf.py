"""GGUF file -> GPU weights: the tensors of a small file written with the `gguf` package are uploaded
through b200q_gguf_upload, and their device copies decode bit for bit to what the package's own
dequantizer gives for the same bytes; a row shard of a file tensor multiplies like the oracle says."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
gguf = pytest.importorskip("gguf")
import magnitude_b200 as mb  # noqa: E402


def _file(tmp_path, orc):
    rng = np.random.default_rng(3)
    specs = (("blk.0.ffn_gate.weight", mb.TYPE_Q4_K, 40, 1024), ("blk.0.ffn_down.weight", mb.TYPE_Q6_K, 24, 2048),
             ("blk.0.attn_q.weight", mb.TYPE_Q8_0, 33, 160))
    packed = {n: orc.quantize(qt, rng.standard_normal((r, k), dtype=np.float32) * np.float32(0.02)) for n, qt, r, k in specs}
    path = tmp_path / "w.gguf"
    w = gguf.GGUFWriter(str(path), "llama")
    for n, qt, r, k in specs:
        w.add_tensor(n, packed[n].reshape(r, -1), raw_dtype=gguf.GGMLQuantizationType(qt))
    w.add_tensor("blk.0.attn_norm.weight", rng.standard_normal(1024, dtype=np.float32))
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()
    return path, specs, packed


def test_uploaded_file_tensors_decode_like_the_gguf_package(backend, orc, tmp_path):
    path, specs, packed = _file(tmp_path, orc)
    f = mb.GgufFile(path)
    for name, qt, r, k in specs:
        w = f.upload(backend, name)
        assert (w.qtype, w.n, w.k) == (qt, r, k)
        got = backend.dequantize(w).cpu().numpy()
        ref = gguf.quants.dequantize(packed[name].reshape(r, -1), gguf.GGMLQuantizationType(qt)).astype(np.float32)
        assert np.array_equal(got.view(np.uint32), ref.view(np.uint32)), name
    with pytest.raises(mb.B200QError) as e:
        f.upload(backend, "blk.0.attn_norm.weight")          # fp32 vector: not a projection weight
    assert "ggml type 0" in str(e.value)


def test_sharded_upload_from_a_file(backend, orc, tmp_path):
    path, specs, packed = _file(tmp_path, orc)
    f = mb.GgufFile(path)
    name, qt, r, k = specs[1]                                  # down: row-parallel, cut along K at superblocks
    x = torch.from_numpy(np.random.default_rng(1).standard_normal((2, k), dtype=np.float32)).cuda().to(torch.bfloat16)
    total = torch.zeros((2, r), device="cuda")
    for rank in range(2):
        w = f.upload(backend, name, split=mb.SPLIT_ROW, rank=rank, world=2)
        lo, hi = mb.shard_range(qt, r, k, mb.SPLIT_ROW, rank, 2)
        assert w.k == hi - lo
        total += backend.project(w, x[:, lo:hi].contiguous())
    backend.sync()
    ref = orc.matmul_exact(qt, packed[name], r, k, x.float().cpu().numpy())
    assert orc.within_tolerance(total.cpu().numpy(), ref, 1e-3)[0]
