"""Plain round-to-nearest encoders for the three GGUF block formats (numpy, vectorised).

These produce *valid* Q8_0 / Q4_K / Q6_K blocks from fp32 weights so benchmarks and examples can
make seeded synthetic tensors without a model file.  Q8_0 follows the format's one obvious rule
(d = max|w| / 127).  For Q4_K and Q6_K this is a direct min/max fit per sub-block, not the
search-based quantizer of the GGUF reference implementation: the bytes differ from what that
tool would write, but any valid block is a legal input to the projection, whose results depend
only on what the blocks decode to.
"""
from __future__ import annotations

import numpy as np

Q4_0, Q8_0, Q4_K, Q5_K, Q6_K, MXFP4 = 2, 8, 12, 13, 14, 39
BLOCK = {MXFP4: (32, 17), Q4_0: (32, 18), Q8_0: (32, 34), Q4_K: (256, 144), Q5_K: (256, 176), Q6_K: (256, 210)}


def _check(w: np.ndarray, blk: int) -> np.ndarray:
    w = np.ascontiguousarray(w, dtype=np.float32)
    if w.ndim != 2 or w.shape[1] % blk:
        raise ValueError(f"expected [N, K] with K a multiple of {blk}, got {w.shape}")
    return w


def quantize_q8_0(w: np.ndarray) -> np.ndarray:
    w = _check(w, 32)
    n, k = w.shape
    b = w.reshape(n, k // 32, 32)
    d = np.abs(b).max(axis=2) / np.float32(127.0)
    with np.errstate(divide="ignore"):
        inv = np.where(d > 0, np.float32(1.0) / d, np.float32(0.0)).astype(np.float32)
    q = np.round(b * inv[..., None]).astype(np.int8)  # np.round is half-even; ties are measure-zero for random input
    out = np.empty((n, k // 32, 34), dtype=np.uint8)
    out[..., 0:2] = d.astype(np.float16)[..., None].view(np.uint8)
    out[..., 2:] = q.view(np.uint8)
    return out.reshape(n, -1)


def quantize_q4_k(w: np.ndarray) -> np.ndarray:
    w = _check(w, 256)
    n, k = w.shape
    nb = k // 256
    b = w.reshape(n, nb, 8, 32)
    mn = np.minimum(b.min(axis=3), 0.0)
    mx = np.maximum(b.max(axis=3), mn)
    scale = (mx - mn) / np.float32(15.0)            # per 32-weight sub-block
    mins = -mn
    d = (scale.max(axis=2) / np.float32(63.0)).astype(np.float16)
    dmin = (mins.max(axis=2) / np.float32(63.0)).astype(np.float16)
    df, dminf = d.astype(np.float32), dmin.astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        ls = np.where(df[..., None] > 0, np.round(scale / df[..., None]), 0).clip(0, 63).astype(np.uint8)
        lm = np.where(dminf[..., None] > 0, np.round(mins / dminf[..., None]), 0).clip(0, 63).astype(np.uint8)
        dl = df[..., None] * ls
        ml = dminf[..., None] * lm
        q = np.where(dl[..., None] > 0, np.round((b + ml[..., None]) / dl[..., None]), 0).clip(0, 15).astype(np.uint8)
    out = np.zeros((n, nb, 144), dtype=np.uint8)
    out[..., 0:2] = d[..., None].view(np.uint8)
    out[..., 2:4] = dmin[..., None].view(np.uint8)
    sc = out[..., 4:16]
    sc[..., 0:4] = ls[..., 0:4] | ((ls[..., 4:8] >> 4) << 6)
    sc[..., 4:8] = lm[..., 0:4] | ((lm[..., 4:8] >> 4) << 6)
    sc[..., 8:12] = (ls[..., 4:8] & 0xF) | ((lm[..., 4:8] & 0xF) << 4)
    qg = q.reshape(n, nb, 4, 2, 32)                  # 64-weight groups: low nibbles then high nibbles
    out[..., 16:] = (qg[..., 0, :] | (qg[..., 1, :] << 4)).reshape(n, nb, 128)
    return out.reshape(n, -1)


def quantize_q6_k(w: np.ndarray) -> np.ndarray:
    w = _check(w, 256)
    n, k = w.shape
    nb = k // 256
    b = w.reshape(n, nb, 16, 16)
    scale = np.abs(b).max(axis=3) / np.float32(31.0)  # per 16-weight sub-block
    d = (scale.max(axis=2) / np.float32(127.0)).astype(np.float16)
    df = d.astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        ls = np.where(df[..., None] > 0, np.round(scale / df[..., None]), 0).clip(0, 127).astype(np.int8)
        dl = df[..., None] * ls.astype(np.float32)
        q = (np.where(dl[..., None] > 0, np.round(b / dl[..., None]), 0).clip(-32, 31) + 32).astype(np.uint8)
    L = q.reshape(n, nb, 2, 4, 32)                    # halves of 128, quadrants of 32
    out = np.zeros((n, nb, 210), dtype=np.uint8)
    ql = out[..., 0:128].reshape(n, nb, 2, 64)
    qh = out[..., 128:192].reshape(n, nb, 2, 32)
    ql[..., 0:32] = (L[..., 0, :] & 0xF) | ((L[..., 2, :] & 0xF) << 4)
    ql[..., 32:64] = (L[..., 1, :] & 0xF) | ((L[..., 3, :] & 0xF) << 4)
    qh[...] = (L[..., 0, :] >> 4) | ((L[..., 1, :] >> 4) << 2) | ((L[..., 2, :] >> 4) << 4) | ((L[..., 3, :] >> 4) << 6)
    out[..., 192:208] = ls.view(np.uint8)
    out[..., 208:210] = d[..., None].view(np.uint8)
    return out.reshape(n, -1)


def quantize(qtype: int, w: np.ndarray) -> np.ndarray:
    """fp32 [N, K] -> packed uint8 [N, K / blk * block_bytes] in GGUF order."""
    if qtype == Q8_0:
        return quantize_q8_0(w)
    if qtype == Q4_K:
        return quantize_q4_k(w)
    if qtype == Q6_K:
        return quantize_q6_k(w)
    raise ValueError(f"unsupported ggml type id {qtype}")


def dequantize_q4_k(packed: np.ndarray, k: int) -> np.ndarray:
    """fp32 [N, K] of Q4_K blocks: w = (d * sc) * q - (dmin * m), each product rounded to fp32 (the format's rule)."""
    rows = np.ascontiguousarray(packed, dtype=np.uint8).reshape(-1, k // 256, 144)
    n, nb = rows.shape[:2]
    d = rows[..., 0:2].copy().view(np.float16).astype(np.float32)[..., 0]
    dmin = rows[..., 2:4].copy().view(np.float16).astype(np.float32)[..., 0]
    sc = rows[..., 4:16]
    ls = np.empty((n, nb, 8), np.uint8)
    lm = np.empty((n, nb, 8), np.uint8)
    ls[..., 0:4] = sc[..., 0:4] & 63
    lm[..., 0:4] = sc[..., 4:8] & 63
    ls[..., 4:8] = (sc[..., 8:12] & 0xF) | ((sc[..., 0:4] >> 6) << 4)
    lm[..., 4:8] = (sc[..., 8:12] >> 4) | ((sc[..., 4:8] >> 6) << 4)
    qs = rows[..., 16:].reshape(n, nb, 4, 32)
    q = np.stack([qs & 0xF, qs >> 4], axis=3).reshape(n, nb, 8, 32).astype(np.float32)
    dl = (d[..., None] * ls.astype(np.float32)).astype(np.float32)
    ml = (dmin[..., None] * lm.astype(np.float32)).astype(np.float32)
    return ((dl[..., None] * q).astype(np.float32) - ml[..., None]).astype(np.float32).reshape(n, k)


def dequantize_q4_0(packed: np.ndarray, k: int) -> np.ndarray:
    """fp32 [N, K] of Q4_0 blocks: w = (q - 8) * d, weights 0..15 in the low nibbles, 16..31 in the high ones."""
    rows = np.ascontiguousarray(packed, dtype=np.uint8).reshape(-1, k // 32, 18)
    d = rows[..., 0:2].copy().view(np.float16).astype(np.float32)
    qs = rows[..., 2:]
    q = np.concatenate([qs & 0xF, qs >> 4], axis=-1).astype(np.float32) - np.float32(8)
    return (q * d).astype(np.float32).reshape(rows.shape[0], k)


def dequantize_q5_k(packed: np.ndarray, k: int) -> np.ndarray:
    """fp32 [N, K] of Q5_K blocks: the Q4_K rule with levels nibble + 16 * (bit s of qh[l]) for sub-block s."""
    rows = np.ascontiguousarray(packed, dtype=np.uint8).reshape(-1, k // 256, 176)
    n, nb = rows.shape[:2]
    d = rows[..., 0:2].copy().view(np.float16).astype(np.float32)[..., 0]
    dmin = rows[..., 2:4].copy().view(np.float16).astype(np.float32)[..., 0]
    sc = rows[..., 4:16]
    ls = np.empty((n, nb, 8), np.uint8)
    lm = np.empty((n, nb, 8), np.uint8)
    ls[..., 0:4] = sc[..., 0:4] & 63
    lm[..., 0:4] = sc[..., 4:8] & 63
    ls[..., 4:8] = (sc[..., 8:12] & 0xF) | ((sc[..., 0:4] >> 6) << 4)
    lm[..., 4:8] = (sc[..., 8:12] >> 4) | ((sc[..., 4:8] >> 6) << 4)
    qh = rows[..., 16:48]                                       # [n, nb, 32]
    qs = rows[..., 48:].reshape(n, nb, 4, 32)
    nib = np.stack([qs & 0xF, qs >> 4], axis=3).reshape(n, nb, 8, 32)
    hb = (qh[:, :, None, :] >> np.arange(8, dtype=np.uint8)[None, None, :, None]) & 1
    q = (nib + 16 * hb).astype(np.float32)
    dl = (d[..., None] * ls.astype(np.float32)).astype(np.float32)
    ml = (dmin[..., None] * lm.astype(np.float32)).astype(np.float32)
    return ((dl[..., None] * q).astype(np.float32) - ml[..., None]).astype(np.float32).reshape(n, k)


def dequantize_q6_k(packed: np.ndarray, k: int) -> np.ndarray:
    """fp32 [N, K] of Q6_K blocks: w = (d * sc) * (q - 32), the product d * sc rounded to fp32 first."""
    rows = np.ascontiguousarray(packed, dtype=np.uint8).reshape(-1, k // 256, 210)
    n, nb = rows.shape[:2]
    ql = rows[..., 0:128].reshape(n, nb, 2, 2, 32)            # half, (l | l + 32), l
    qh = rows[..., 128:192].reshape(n, nb, 2, 32)
    sc = rows[..., 192:208].copy().view(np.int8).astype(np.float32)
    d = rows[..., 208:210].copy().view(np.float16).astype(np.float32)[..., 0]
    q = np.empty((n, nb, 2, 4, 32), np.int16)
    q[:, :, :, 0] = (ql[:, :, :, 0] & 0xF) | ((qh & 3) << 4)
    q[:, :, :, 1] = (ql[:, :, :, 1] & 0xF) | (((qh >> 2) & 3) << 4)
    q[:, :, :, 2] = (ql[:, :, :, 0] >> 4) | (((qh >> 4) & 3) << 4)
    q[:, :, :, 3] = (ql[:, :, :, 1] >> 4) | (((qh >> 6) & 3) << 4)
    dl = (d[..., None] * sc).astype(np.float32)                # [n, nb, 16]
    w = (q.reshape(n, nb, 16, 16).astype(np.float32) - np.float32(32.0)) * dl[..., None]
    return w.astype(np.float32).reshape(n, k)


def dequantize(qtype: int, packed: np.ndarray, k: int) -> np.ndarray:
    if qtype == Q4_K:
        return dequantize_q4_k(packed, k)
    if qtype == Q4_0:
        return dequantize_q4_0(packed, k)
    if qtype == Q5_K:
        return dequantize_q5_k(packed, k)
    if qtype == Q6_K:
        return dequantize_q6_k(packed, k)
    raise ValueError(f"no numpy decoder for ggml type id {qtype}")


def f32_to_bf16_bits(a: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even bf16 bit patterns (uint16) of an fp32 array."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    r = (u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)
    return r.astype(np.uint16)


def synth_weights(qtype: int, n: int, k: int, seed: int, std: float = 0.02, encoder=None) -> np.ndarray:
    """Packed blocks of W ~ N(0, std) drawn with numpy.random.default_rng(seed).

    `encoder(qtype, w)` turns fp32 rows into packed rows; the default is this module's plain min/max
    encoder, the benchmark passes the format's reference quantizer (magnitude_b200.quantize)."""
    rng = np.random.default_rng(seed)
    enc = encoder or quantize
    out = []
    step = max(1, (1 << 24) // max(k, 1))             # bound the fp32 scratch to ~64 MB
    for r0 in range(0, n, step):
        w = rng.standard_normal((min(step, n - r0), k), dtype=np.float32) * np.float32(std)
        out.append(enc(qtype, w))
    return np.concatenate(out, axis=0) if out else np.zeros((0, k // BLOCK[qtype][0] * BLOCK[qtype][1]), np.uint8)
