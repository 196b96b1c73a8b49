"""Tensor-parallel helpers for the projection path (host side).

The reference only *declares* how weights spread over devices (`SplitMode::{Row, Tensor}` and
`tensor_split`, inference/crates/icn-contracts/src/lib.rs:122-124,200-205) and leaves the work to
its native dependency.  Here the cut is explicit: QKV / gate / up are split by output rows (no
exchange), O / down by 256-weight superblocks along K (outputs are partial sums, one all-reduce).
"""
from __future__ import annotations

import numpy as np

from . import _binding as B
from .projection import shard_range

BLOCK = {B.TYPE_MXFP4: (32, 17), B.TYPE_Q4_0: (32, 18), B.TYPE_Q8_0: (32, 34), B.TYPE_Q4_K: (256, 144), B.TYPE_Q5_K: (256, 176), B.TYPE_Q6_K: (256, 210)}


def shard_gguf(qtype: int, packed: np.ndarray, n: int, k: int, split: int, rank: int, world: int,
               align_rows: int = 0) -> tuple[np.ndarray, int, int]:
    """The GGUF bytes of one rank's shard of W[N][K] plus the shard's (N, K).

    Column split keeps whole rows; row split keeps a range of blocks of every row.  The device
    path does the same cut inside b200q_weight_upload_shard; this host version exists for tools and
    for checking shards on the CPU.
    """
    be, bb = BLOCK[qtype]
    rows = np.ascontiguousarray(packed, dtype=np.uint8).reshape(n, k // be * bb)
    lo, hi = shard_range(qtype, n, k, split, rank, world, align_rows)
    if split == B.SPLIT_COLUMN:
        return rows[lo:hi].copy(), hi - lo, k
    return rows[:, lo // be * bb: hi // be * bb].copy(), n, hi - lo


def activation_slice(qtype: int, n: int, k: int, rank: int, world: int) -> tuple[int, int]:
    """Columns of the activation a row-parallel rank multiplies (its K range)."""
    return shard_range(qtype, n, k, B.SPLIT_ROW, rank, world)
