"""Generates tests/golden/ggml_blocks.npz from the third-party `gguf` Python package.

The package is an independent statement of the GGUF block formats (not the reference engine and
not this repository's oracle).  Run from the repository root:  python tests/golden/make_golden.py
Each case stores packed blocks and what gguf.quants.dequantize() decodes them to; the Q8_0 case
also stores gguf.quants.quantize() output for a seeded fp32 tensor.
"""
from pathlib import Path

import gguf
import numpy as np
from gguf import quants

OUT = Path(__file__).resolve().parent / "ggml_blocks.npz"
T = {2: gguf.GGMLQuantizationType.Q4_0, 8: gguf.GGMLQuantizationType.Q8_0, 12: gguf.GGMLQuantizationType.Q4_K, 13: gguf.GGMLQuantizationType.Q5_K,
     14: gguf.GGMLQuantizationType.Q6_K, 39: gguf.GGMLQuantizationType.MXFP4}
BLK = {39: (32, 17), 2: (32, 18), 8: (32, 34), 12: (256, 144), 13: (256, 176), 14: (256, 210)}
# byte offsets of the fp16 fields inside a block (kept finite so decoded values are comparable)
F16_AT = {39: [], 2: [0], 8: [0], 12: [0, 2], 13: [0, 2], 14: [208]}


def random_blocks(rng, qt, rows, k):
    be, bb = BLK[qt]
    nblk = rows * k // be
    raw = rng.integers(0, 256, size=(nblk, bb), dtype=np.uint8)
    for off in F16_AT[qt]:
        scale = (rng.standard_normal(nblk) * 0.01).astype(np.float16)
        # a few exact zeros, negative values and fp16 subnormals exercise the widening
        scale[::7] = np.float16(0)
        scale[3::11] = np.float16(6e-8) * rng.integers(1, 100, size=scale[3::11].shape).astype(np.float16)
        raw[:, off:off + 2] = scale.view(np.uint8).reshape(nblk, 2)
    return raw.reshape(rows, -1)


def main():
    rng = np.random.default_rng(1234)
    out = {}
    def case(qt):
        rows, k = 6, 768
        packed = random_blocks(rng, qt, rows, k)
        out[f"packed_{qt}"] = packed
        out[f"dequant_{qt}"] = quants.dequantize(packed, T[qt]).astype(np.float32)

    for qt in (8, 12, 14):
        case(qt)
    w = (rng.standard_normal((4, 512)) * 0.02).astype(np.float32)
    w[0, :32] = 0.0          # an all-zero block
    w[1, 5] = 0.5            # an outlier
    out["q8_0_src"] = w
    out["q8_0_packed"] = quants.quantize(w, T[8])
    case(13)      # drawn last: the cases above keep the bytes they had before Q5_K was added
    case(2)       # ... and before Q4_0 was
    out["q4_0_packed"] = quants.quantize(w, T[2])       # of the same source as the Q8_0 case
    case(39)      # MXFP4: every byte random, the whole range of e8m0 scales included
    out["mxfp4_packed"] = quants.quantize(w, T[39])
    np.savez_compressed(OUT, **out)
    print("wrote", OUT, OUT.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
