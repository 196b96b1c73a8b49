"""The C-ABI library on a machine without a GPU: it loads, exports every declared symbol, and its
host-only logic (sizes, shard ranges, layout conversion, argument checks) behaves."""
import ctypes
import re
from ctypes import byref, c_int64, c_void_p
from pathlib import Path

import numpy as np
import pytest

import magnitude_b200 as mb
from magnitude_b200 import _binding as B

ROOT = Path(__file__).resolve().parent.parent
HEADER = (ROOT / "include" / "b200q.h").read_text()


def declared_symbols():
    code = re.sub(r"/\*.*?\*/", "", HEADER, flags=re.S)      # drop comments
    return sorted(set(re.findall(r"\b(b200q_[a-z0-9_]+)\s*\(", code)))


def test_header_and_library_agree():
    names = declared_symbols()
    assert len(names) >= 20
    lib = ctypes.CDLL(str(B.LIB_PATH))
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/b200q.h but not exported"
    assert sorted(B.SIGNATURES) == names, "the ctypes table and the header list different entry points"


def test_integration_notes_bind_every_entry_point():
    # the reference-side binding shown to a maintainer (the Rust extern block) lists exactly the header's functions
    notes = (ROOT / "INTEGRATION.md").read_text()
    bound = sorted(set(re.findall(r"pub fn (b200q_[a-z0-9_]+)\s*\(", notes)))
    assert bound == declared_symbols()


def test_version_and_storage_bytes():
    assert re.fullmatch(r"\d+\.\d+\.\d+", mb.__version__)
    assert mb.tensor_storage_bytes(mb.TYPE_Q8_0, 4096 * 4096) == 17825792
    assert mb.tensor_storage_bytes(mb.TYPE_Q4_K, 14336 * 4096) == 33030144
    assert mb.tensor_storage_bytes(mb.TYPE_Q6_K, 4096 * 14336) == 48168960
    assert mb.tensor_storage_bytes(mb.TYPE_Q4_K, 100) == -1      # not a block multiple
    assert mb.tensor_storage_bytes(99, 256) == -1                # unknown type


def test_shard_ranges():
    # row split at 256-weight superblocks, remainders to the low ranks: 100 superblocks over 8 ranks
    sizes = [mb.shard_range(mb.TYPE_Q6_K, 5120, 25600, mb.SPLIT_ROW, r, 8) for r in range(8)]
    assert [(e - b) // 256 for b, e in sizes] == [13, 13, 13, 13, 12, 12, 12, 12]
    assert sizes[0][0] == 0 and sizes[-1][1] == 25600
    assert all(sizes[i][1] == sizes[i + 1][0] for i in range(7))
    # column split aligned to 256 rows reproduces the same cut of the intermediate dimension
    cols = [mb.shard_range(mb.TYPE_Q4_K, 25600, 5120, mb.SPLIT_COLUMN, r, 8, 256) for r in range(8)]
    assert cols == sizes
    # head-aligned QKV: 64 query heads of 128 rows over 8 ranks
    assert mb.shard_range(mb.TYPE_Q4_K, 8192, 5120, mb.SPLIT_COLUMN, 3, 8, 128) == (3072, 4096)
    # llama-3-8b down projection: 56 superblocks, 7 per rank
    assert mb.shard_range(mb.TYPE_Q4_K, 4096, 14336, mb.SPLIT_ROW, 7, 8) == (12544, 14336)
    # more ranks than units: trailing ranks own nothing
    assert mb.shard_range(mb.TYPE_Q4_K, 8, 512, mb.SPLIT_ROW, 3, 4) == (512, 512)
    for bad in [dict(rank=8, world=8), dict(rank=-1, world=2), dict(rank=0, world=0)]:
        with pytest.raises(mb.B200QError):
            mb.shard_range(mb.TYPE_Q4_K, 8, 512, mb.SPLIT_ROW, bad["rank"], bad["world"])
    with pytest.raises(mb.B200QError):
        mb.shard_range(mb.TYPE_Q4_K, 100, 512, mb.SPLIT_COLUMN, 0, 2, 64)   # N not a multiple of the alignment


def _pack(qt, packed, n, k):
    rb = B.lib().b200q_layout_row_bytes(qt, k)
    out = np.zeros(((n + 3) // 4 * 4, rb), np.uint8)     # the layout pads to whole 4-row groups
    st = B.lib().b200q_layout_pack(qt, n, k, packed.ctypes.data, packed.size, out.ctypes.data, out.size)
    assert st == 0
    return out


REC = {12: 144, 8: 272, 14: 208}


def _rec_off(qt, sb):
    return (sb >> 3) * 1680 + (sb & 7) * 208 if qt == 14 else sb * REC[qt]


def _row_bytes(qt, nsb):
    if qt == 14:
        return (nsb >> 3) * 1680 + ((nsb & 7) * 208 + 16 if nsb & 7 else 0)
    return nsb * REC[qt]


def _record_off(qt, row, sb, n, nsb):
    """Tile-major layout: groups of 4 rows, chunks of 8 records, rows of a group adjacent inside a chunk."""
    g, c = row // 4, sb // 8
    nr = 4                                # groups are whole: missing rows are zero padding
    end = _row_bytes(qt, nsb) if (c + 1) * 8 >= nsb else _rec_off(qt, (c + 1) * 8)
    chunk_row = end - _rec_off(qt, c * 8)
    return 4 * g * _row_bytes(qt, nsb) + nr * _rec_off(qt, c * 8) + (row - 4 * g) * chunk_row + _rec_off(qt, sb) - _rec_off(qt, c * 8)


def test_streaming_layout_is_a_permutation_of_the_gguf_bytes(orc):
    rng = np.random.default_rng(0)
    # Q4_K: native 144-byte blocks, tile order; 6 rows = one full row group + a group of 2
    n, nsb = 6, 11
    p = rng.integers(0, 256, size=(n, nsb * 144), dtype=np.uint8)
    s = _pack(12, p, n, nsb * 256).reshape(-1)
    assert s.size == 8 * nsb * 144        # 6 rows padded to 8
    for r in range(n):
        for sb in range(nsb):
            o = _record_off(12, r, sb, n, nsb)
            assert np.array_equal(s[o:o + 144], p[r, sb * 144:(sb + 1) * 144])
    # a tile (4 rows x 8 records) is one contiguous range
    assert _record_off(12, 1, 0, n, nsb) - _record_off(12, 0, 0, n, nsb) == 8 * 144
    assert _record_off(12, 0, 8, n, nsb) == 4 * 8 * 144
    # Q8_0: per 8 blocks [8 x 32 quants][8 x d]; ragged K padded with zero blocks
    n, k = 5, 11 * 32
    p = rng.integers(0, 256, size=(n, 11 * 34), dtype=np.uint8)
    s = _pack(8, p, n, k).reshape(-1)
    assert s.size == 8 * 2 * 272          # 5 rows padded to 8
    for r in range(n):
        for b in range(16):
            o = _record_off(8, r, b // 8, n, 2)
            rec = s[o:o + 272]
            q, d = rec[32 * (b % 8):32 * (b % 8) + 32], rec[256 + 2 * (b % 8):258 + 2 * (b % 8)]
            if b < 11:
                assert np.array_equal(q, p[r, 34 * b + 2:34 * b + 34]) and np.array_equal(d, p[r, 34 * b:34 * b + 2])
            else:
                assert not q.any() and not d.any()
    # Q6_K: 208-byte records, the eight d of an octet after it; 11 superblocks = one octet + 3
    n, nsb = 7, 11
    p = rng.integers(0, 256, size=(n, nsb * 210), dtype=np.uint8)
    s = _pack(14, p, n, nsb * 256).reshape(-1)
    assert s.size == 8 * (1680 + 3 * 208 + 16) and s.size % 16 == 0
    for r in range(n):
        for sb in range(nsb):
            o = _record_off(14, r, sb, n, nsb)
            in_octet = min(8, nsb - (sb // 8) * 8)
            od = _record_off(14, r, (sb // 8) * 8, n, nsb) + in_octet * 208 + 2 * (sb % 8)
            assert np.array_equal(s[o:o + 208], p[r, sb * 210: sb * 210 + 208])
            assert np.array_equal(s[od:od + 2], p[r, sb * 210 + 208: sb * 210 + 210])


def test_layout_argument_checks():
    L = B.lib()
    assert L.b200q_layout_row_bytes(12, 4096) == 2304
    assert L.b200q_layout_row_bytes(14, 14336) == 11760
    assert L.b200q_layout_row_bytes(14, 5120) == 4208      # 4200 GGUF bytes + 8 of padding
    assert L.b200q_layout_row_bytes(8, 4096) == 4352
    assert L.b200q_layout_row_bytes(12, 100) == -1
    assert L.b200q_layout_row_bytes(3, 256) == -1
    buf = np.zeros(144, np.uint8)
    out = np.zeros(4 * 144, np.uint8)
    assert L.b200q_layout_pack(12, 1, 256, buf.ctypes.data, 143, out.ctypes.data, 576) == B.ERR_INVALID_CONFIG
    assert L.b200q_layout_pack(12, 1, 256, buf.ctypes.data, 144, out.ctypes.data, 100) == B.ERR_INVALID_CONFIG
    assert L.b200q_layout_pack(12, 1, 256, None, 144, out.ctypes.data, 576) == B.ERR_INVALID_CONFIG
    assert L.b200q_layout_pack(12, 0, 256, None, 0, None, 0) == B.OK


def test_null_handles_are_rejected_not_dereferenced():
    L = B.lib()
    assert L.b200q_ctx_create(0, None) == B.ERR_INVALID_CONFIG
    assert L.b200q_last_error(None, None, 0) == B.ERR_INVALID_CONFIG
    assert L.b200q_sync(None, None, 1) == B.ERR_INVALID_CONFIG
    assert L.b200q_matmul(None, None, None, 0, 1, 1, None, 0, 1, None) == B.ERR_INVALID_CONFIG
    assert L.b200q_weight_info(None, None, None, None, None, None) == B.ERR_INVALID_CONFIG
    assert L.b200q_tp_unique_id(None) == B.ERR_INVALID_CONFIG
    L.b200q_weight_destroy(None)
    L.b200q_ctx_destroy(None)
    b, e = c_int64(), c_int64()
    assert L.b200q_shard_range(12, 8, 512, 5, 0, 1, 0, byref(b), byref(e)) == B.ERR_INVALID_CONFIG


def test_no_cpu_fallback_without_a_device():
    torch = pytest.importorskip("torch")
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    h = c_void_p()
    assert B.lib().b200q_ctx_create(0, byref(h)) == B.ERR_BACKEND
    with pytest.raises(mb.B200QError) as e:
        mb.Backend(0)
    assert e.value.kind == "Backend"


def test_missing_library_fails_loudly(tmp_path):
    with pytest.raises(ImportError):
        B.load_library(tmp_path / "libb200q.so")
