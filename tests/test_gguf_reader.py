"""The GGUF tensor reader on the CPU: files written with the `gguf` package's writer (import only) are
walked the way the reference inspector walks them (inference/crates/icn-models/src/gguf.rs:75-149), and
hand-made malformed headers are rejected with the reference's messages (its own tests: gguf.rs:477-572)."""
import struct

import numpy as np
import pytest

import magnitude_b200 as mb

gguf = pytest.importorskip("gguf")


def _s(text):
    b = text.encode()
    return struct.pack("<Q", len(b)) + b


def _header(version=3, tensors=0, kvs=0):
    return b"GGUF" + struct.pack("<IQQ", version, tensors, kvs)


def _write(tmp_path, name, data):
    p = tmp_path / name
    p.write_bytes(data)
    return p


def _model_file(tmp_path, orc, alignment=None):
    rng = np.random.default_rng(0)
    tensors = {}
    for name, qt, n, k in (("blk.0.ffn_gate.weight", mb.TYPE_Q4_K, 24, 512), ("blk.0.ffn_down.weight", mb.TYPE_Q6_K, 16, 768),
                           ("blk.0.attn_q.weight", mb.TYPE_Q8_0, 10, 96)):
        tensors[name] = (qt, n, k, orc.quantize(qt, rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02)))
    norm = rng.standard_normal(512, dtype=np.float32)
    path = tmp_path / "tiny.gguf"
    w = gguf.GGUFWriter(str(path), "llama")
    if alignment:
        w.add_custom_alignment(alignment)
    w.add_name("tiny")
    w.add_context_length(4096)
    w.add_uint64("general.parameter_count", 123456)
    w.add_array("tokenizer.ggml.tokens", ["<bos>", "<eos>", "a"])
    w.add_float32("llama.rope.freq_base", 10000.0)
    w.add_bool("general.some_flag", True)
    for name, (qt, n, k, packed) in tensors.items():
        w.add_tensor(name, packed.reshape(n, -1), raw_shape=None, raw_dtype=gguf.GGMLQuantizationType(qt))
    w.add_tensor("blk.0.attn_norm.weight", norm)
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()
    return path, tensors, norm


def test_reads_what_the_gguf_package_wrote(tmp_path, orc):
    path, tensors, norm = _model_file(tmp_path, orc)
    f = mb.GgufFile(path)
    rd = gguf.GGUFReader(str(path))
    assert f.version == 3 and f.tensor_count == 4 and f.alignment == 32
    assert f.metadata_string("general.architecture") == "llama"
    assert f.metadata_string("general.name") == "tiny"
    assert f.metadata_u64("llama.context_length") == 4096
    assert f.parameter_count == 123456
    assert f.metadata_string("no.such.key") is None and f.metadata_u64("general.name") is None
    assert f.header_bytes == rd.data_offset
    assert f.file_bytes == path.stat().st_size
    by_name = {t.name: t for t in rd.tensors}
    total = 0
    for t in f.tensors():
        ref = by_name[t["name"]]
        assert t["type"] == int(ref.tensor_type)
        assert t["dims"] == [int(d) for d in ref.shape]          # GGUF order: row length first
        assert t["bytes"] == int(ref.n_bytes) and t["file_offset"] == int(ref.data_offset)
        assert t["bytes"] == mb.tensor_storage_bytes_shape(t["type"], t["dims"])
        assert np.array_equal(f.read(t["name"]), np.asarray(ref.data).reshape(-1).view(np.uint8))
        total += t["bytes"]
    assert f.tensor_storage_bytes == total
    for name, (qt, n, k, packed) in tensors.items():
        t = f.tensor(name)
        assert t["dims"] == [k, n] and t["type"] == qt
        assert np.array_equal(f.read(name), packed.reshape(-1))
    with pytest.raises(mb.B200QError):
        f.tensor("missing.weight")
    f.close()


def test_custom_alignment_moves_the_data_section(tmp_path, orc):
    path, tensors, _ = _model_file(tmp_path, orc, alignment=128)
    f = mb.GgufFile(path)
    assert f.alignment == 128 and f.header_bytes % 128 == 0
    assert f.header_bytes == gguf.GGUFReader(str(path)).data_offset
    name = "blk.0.ffn_down.weight"
    assert f.tensor(name)["file_offset"] % 128 == 0
    assert np.array_equal(f.read(name), tensors[name][3].reshape(-1))


def test_storage_bytes_table_matches_the_gguf_package():
    for t, (elems, nbytes) in gguf.GGML_QUANT_SIZES.items():
        assert mb.tensor_storage_bytes_shape(int(t), [elems * 3, 5]) == 3 * nbytes * 5, t
        if elems > 1:
            assert mb.tensor_storage_bytes_shape(int(t), [elems * 3 + 1, 5]) == -1     # row is not a block multiple
    assert mb.tensor_storage_bytes_shape(12, [512, 7, 3]) == 2 * 144 * 21
    assert mb.tensor_storage_bytes_shape(1234, [256]) == -1
    assert mb.tensor_storage_bytes_shape(12, []) == -1


@pytest.mark.parametrize("data,text", [
    (b"not a gguf", "file is not GGUF"),
    (b"GG", "file is not GGUF"),
    (_header(version=1), "unsupported GGUF version 1"),
    (_header(version=4), "unsupported GGUF version 4"),
    (_header(tensors=10_000_001), "tensor count exceeds inspection bound"),
    (_header(kvs=1_000_001), "metadata count exceeds inspection bound"),
    (_header(kvs=1), "header extends beyond end of file"),                                   # truncated key
    (_header(kvs=1) + _s("k") + struct.pack("<I", 99), "unknown metadata value type"),
    (_header(kvs=1) + struct.pack("<Q", (16 << 20) + 1), "metadata string exceeds inspection bound"),
    (_header(kvs=1) + _s("general.alignment") + struct.pack("<II", 4, 48), "GGUF alignment is invalid"),
    (_header(kvs=1) + _s("general.alignment") + struct.pack("<II", 4, 0), "GGUF alignment is invalid"),
    (_header(tensors=1) + _s("t") + struct.pack("<I", 0), "tensor dimension count is invalid"),
    (_header(tensors=1) + _s("t") + struct.pack("<I", 9), "tensor dimension count is invalid"),
    (_header(tensors=1) + _s("t") + struct.pack("<IQQ", 2, 1 << 40, 1 << 40), "tensor element count overflow"),
    (_header(tensors=1) + _s("t") + struct.pack("<IQII", 1, 100, 12, 0) + struct.pack("<I", 0), "tensor storage shape or type is invalid"),
    (_header(tensors=1) + _s("t") + struct.pack("<IQI", 1, 256, 777) + struct.pack("<Q", 0), "tensor storage shape or type is invalid"),
    (_header(kvs=1) + _s("k") + struct.pack("<IIQ", 9, 4, 1_000_001), "metadata array exceeds inspection bound"),
])
def test_malformed_headers_are_rejected(tmp_path, data, text):
    p = _write(tmp_path, "bad.gguf", data)
    with pytest.raises(mb.B200QError) as e:
        mb.GgufFile(p)
    assert e.value.status == mb._binding.ERR_INVALID_CONFIG
    assert text in str(e.value)


def test_missing_file_and_padding_rule(tmp_path):
    with pytest.raises(mb.B200QError) as e:
        mb.GgufFile(tmp_path / "nope.gguf")
    assert e.value.status == mb._binding.ERR_BACKEND
    # a header that ends off the alignment must be followed by padding inside the file (gguf.rs:147-149)
    body = _header(kvs=1) + _s("general.name") + struct.pack("<I", 8) + _s("x")
    with pytest.raises(mb.B200QError) as e:
        mb.GgufFile(_write(tmp_path, "short.gguf", body))
    assert "GGUF header extends beyond end of file" in str(e.value)
    padded = body + b"\0" * (-len(body) % 32)
    f = mb.GgufFile(_write(tmp_path, "ok.gguf", padded))
    assert f.header_bytes == len(padded) and f.tensor_count == 0 and f.metadata_string("general.name") == "x"


def test_tensor_data_beyond_the_file_is_refused(tmp_path):
    # one Q4_K tensor of 2 rows x 256 whose offset points past the end of the file
    body = _header(tensors=1) + _s("w") + struct.pack("<IQQI", 2, 256, 2, 12) + struct.pack("<Q", 64)
    body += b"\0" * (-len(body) % 32) + b"\0" * 100
    f = mb.GgufFile(_write(tmp_path, "cut.gguf", body))
    assert f.tensor(0)["bytes"] == 288
    with pytest.raises(mb.B200QError) as e:
        f.read(0)
    assert "beyond end of file" in str(e.value)
