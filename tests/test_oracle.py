"""CPU tests of the oracle against the golden vectors and against itself (no GPU)."""
from pathlib import Path

import numpy as np
import pytest

from magnitude_b200 import ggml_quant as gq

GOLD = Path(__file__).resolve().parent / "golden" / "ggml_blocks.npz"
TYPES = [2, 8, 12, 13, 14, 39]
SIZES = {39: (32, 17), 2: (32, 18), 8: (32, 34), 12: (256, 144), 13: (256, 176), 14: (256, 210)}


@pytest.mark.parametrize("qt", TYPES)
def test_block_sizes(orc, qt):
    be, bb = SIZES[qt]
    assert orc.lib().ggq_block_elems(qt) == be
    assert orc.lib().ggq_block_bytes(qt) == bb
    assert orc.row_bytes(qt, 4096) == 4096 // be * bb
    with pytest.raises(ValueError):
        orc.row_bytes(qt, be + 1)


@pytest.mark.parametrize("qt", TYPES)
def test_dequantize_matches_golden_bit_for_bit(orc, qt):
    g = np.load(GOLD)
    got = orc.dequantize(qt, g[f"packed_{qt}"], 768)
    assert np.array_equal(got.view(np.uint32), g[f"dequant_{qt}"].view(np.uint32))


def test_q8_0_quantizer_matches_golden(orc):
    g = np.load(GOLD)
    assert np.array_equal(orc.quantize(8, g["q8_0_src"]), g["q8_0_packed"])
    assert np.array_equal(gq.quantize_q8_0(g["q8_0_src"]), g["q8_0_packed"])


@pytest.mark.parametrize("qt,bound", [(8, 0.01), (12, 0.09), (14, 0.025)])
def test_quantize_round_trip_error(orc, qt, bound):
    rng = np.random.default_rng(0)
    w = rng.standard_normal((32, 2048), dtype=np.float32) * np.float32(0.02)
    for enc in (orc.quantize, gq.quantize):
        d = orc.dequantize(qt, enc(qt, w), 2048)
        assert np.sqrt(np.mean((d - w) ** 2)) / 0.02 < bound


@pytest.mark.parametrize("qt", TYPES)
def test_quantizer_edge_blocks(orc, qt):
    k = 512
    w = np.zeros((3, k), dtype=np.float32)
    w[1] = 1e-3                      # constant block
    w[2, ::7] = np.linspace(-1, 1, len(w[2, ::7]))
    d = orc.dequantize(qt, orc.quantize(qt, w), k)
    assert np.all(d[0] == 0)
    assert np.all(np.isfinite(d))
    assert np.max(np.abs(d[1] - w[1])) < 2e-4
    assert np.max(np.abs(d[2] - w[2])) < (0.13 if qt == 39 else 0.08)      # MXFP4's top levels are 8 and 12 scale units apart


@pytest.mark.parametrize("qt", TYPES)
def test_exact_matmul_is_fp64_dot_of_dequantized(orc, qt):
    rng = np.random.default_rng(qt)
    n, k, m = 19, 1024, 3
    p = orc.quantize(qt, rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02))
    x = rng.standard_normal((m, k), dtype=np.float32)
    ref = (x.astype(np.float64) @ orc.dequantize(qt, p, k).astype(np.float64).T).astype(np.float32)
    got = orc.matmul_exact(qt, p, n, k, x)
    assert np.allclose(got, ref, rtol=2e-7, atol=1e-9)


@pytest.mark.parametrize("qt", TYPES)
def test_cpu_style_path_tracks_exact(orc, qt):
    # the reference-style CPU path quantizes activations to 8 bit: close, not equal
    rng = np.random.default_rng(100 + qt)
    n, k = 64, 4096
    p = orc.quantize(qt, rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02))
    x = rng.standard_normal((2, k), dtype=np.float32)
    exact = orc.matmul_exact(qt, p, n, k, x)
    cpu = orc.matmul_cpu(qt, p, n, k, x)
    rms = np.sqrt(np.mean(exact ** 2))
    assert np.max(np.abs(cpu - exact)) < 0.06 * rms
    assert np.array_equal(cpu, orc.matmul_cpu(qt, p, n, k, x, threads=1))   # thread count does not change results


def test_one_hot_sub_block_decode(orc):
    # each 6-bit scale/min slot of Q4_K and each int8 scale slot of Q6_K decodes to its own sub-block
    blk = np.zeros((1, 144), dtype=np.uint8)
    blk[0, 0:2] = np.array([1.0], np.float16).view(np.uint8)       # d = 1
    blk[0, 2:4] = np.array([1.0], np.float16).view(np.uint8)       # dmin = 1
    blk[0, 16:] = 0x11                                             # every quant = 1
    for j in range(8):
        b = blk.copy()
        sc, mn = 5 + 7 * j, 3 + 6 * j                              # distinct 6-bit values, some > 15 and > 31
        if j < 4:
            b[0, 4 + j] = sc
            b[0, 8 + j] = mn
        else:
            b[0, 4 + j + 4] = (sc & 0xF) | ((mn & 0xF) << 4)
            b[0, 4 + j - 4] |= (sc >> 4) << 6
            b[0, 4 + j] |= (mn >> 4) << 6
        d = orc.dequantize(12, b, 256)[0]
        want = np.zeros(256, np.float32)
        want[32 * j:32 * j + 32] = sc - mn
        assert np.array_equal(d, want), j
    blk6 = np.zeros((1, 210), dtype=np.uint8)
    blk6[0, 208:210] = np.array([1.0], np.float16).view(np.uint8)
    blk6[0, 0:128] = 0x11                                          # low nibbles 1
    blk6[0, 128:192] = 0xAA                                        # high bits 2 -> q = 33 - 32 = 1
    for j in range(16):
        b = blk6.copy()
        b[0, 192 + j] = np.int8(-3 - j).view(np.uint8)
        d = orc.dequantize(14, b, 256)[0]
        want = np.zeros(256, np.float32)
        want[16 * j:16 * j + 16] = -3 - j
        assert np.array_equal(d, want), j


def test_bf16_and_f16_conversions(orc):
    rng = np.random.default_rng(3)
    a = np.concatenate([rng.standard_normal(1000).astype(np.float32) * 10, np.array([0, -0.0, 1e-8, 65504, 65520, 1e6, np.inf, -np.inf], np.float32)])
    assert np.array_equal(orc.f32_to_f16(a), a.astype(np.float16).view(np.uint16))
    h = np.arange(0, 65536, dtype=np.uint32).astype(np.uint16)
    f = orc.f16_to_f32(h)
    ref = h.view(np.float16).astype(np.float32)
    assert np.array_equal(f.view(np.uint32)[~np.isnan(ref)], ref.view(np.uint32)[~np.isnan(ref)])
    assert np.array_equal(orc.f32_to_bf16(a), gq.f32_to_bf16_bits(a))
    assert np.array_equal(orc.bf16_to_f32(orc.f32_to_bf16(a)).view(np.uint32) & 0xFFFF, np.zeros(a.shape, np.uint32))


def test_tolerance_rule(orc):
    ref = np.array([1.0, 0.0, -2.0], np.float32)
    assert orc.within_tolerance(ref * (1 + 5e-4), ref, 1e-3)[0]
    assert not orc.within_tolerance(ref * (1 + 5e-3), ref, 1e-3)[0]
    assert not orc.within_tolerance(np.array([1.0, np.nan, -2.0]), ref, 1e-3)[0]


def test_library_quantizer_is_the_oracles_quantizer_byte_for_byte(orc):
    # the product ships the same reference quantizer (b200q_quantize, used to make benchmark tensors):
    # identical bytes on random, constant, tiny, huge and all-zero rows
    import magnitude_b200 as mb

    rng = np.random.default_rng(11)
    for qt in (orc.Q4_0, orc.Q8_0, orc.Q4_K, orc.Q5_K, orc.Q6_K, orc.MXFP4):
        for n, k, scale in ((33, 1024, 0.02), (5, 256, 1.0), (4, 512, 1e-9), (6, 768, 300.0)):
            w = (rng.standard_normal((n, k)) * scale).astype(np.float32)
            w[0] = 0.0
            w[-1] = w[-1, 0]
            assert np.array_equal(mb.quantize(qt, w), orc.quantize(qt, w)), (qt, n, k, scale)
    with pytest.raises(mb.B200QError):
        mb.quantize(orc.Q4_K, np.zeros((2, 100), np.float32))
