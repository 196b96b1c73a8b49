"""Tensor-parallel cut on CPU: two gloo ranks, shards computed with the oracle.

Column-parallel shards gathered = the full product; row-parallel partial sums all-reduced = the
full product.  No GPU: this covers the host logic (shard ranges, byte cuts, the exchange step).
"""
import os
import socket

import numpy as np
import pytest

torch = pytest.importorskip("torch")
import torch.distributed as dist  # noqa: E402
import torch.multiprocessing as mp  # noqa: E402


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, qtype, n, k, out_dir):
    import sys
    from pathlib import Path

    sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import magnitude_b200 as mb
    from magnitude_b200 import ggml_quant as gq
    from magnitude_b200 import tp
    from oracle import oracle as orc

    rng = np.random.default_rng(0)                       # every rank draws the same full tensors
    w = rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02)
    x = rng.standard_normal((2, k), dtype=np.float32)
    packed = gq.quantize(qtype, w)
    full = orc.matmul_exact(qtype, packed, n, k, x)

    # column parallel: own rows, gather
    shard, sn, sk = tp.shard_gguf(qtype, packed, n, k, mb.SPLIT_COLUMN, rank, world, 4)
    part = torch.from_numpy(orc.matmul_exact(qtype, shard, sn, sk, x))
    sizes = [mb.shard_range(qtype, n, k, mb.SPLIT_COLUMN, r, world, 4) for r in range(world)]
    bufs = [torch.empty((2, e - b)) for b, e in sizes]
    dist.all_gather(bufs, part) if len({e - b for b, e in sizes}) == 1 else None
    if len({e - b for b, e in sizes}) != 1:              # ragged: exchange one by one
        for r in range(world):
            t = part.clone() if r == rank else torch.empty((2, sizes[r][1] - sizes[r][0]))
            dist.broadcast(t, src=r)
            bufs[r] = t
    col = torch.cat(bufs, dim=1).numpy()

    # row parallel: own K range of every row, partial sums, one all-reduce
    shard, sn, sk = tp.shard_gguf(qtype, packed, n, k, mb.SPLIT_ROW, rank, world)
    lo, hi = tp.activation_slice(qtype, n, k, rank, world)
    partial = np.zeros((2, n), np.float32) if sk == 0 else orc.matmul_exact(qtype, shard, sn, sk, np.ascontiguousarray(x[:, lo:hi]))
    t = torch.from_numpy(partial.copy())
    dist.all_reduce(t)
    row = t.numpy()

    if rank == 0:
        np.savez(os.path.join(out_dir, "res.npz"), full=full, col=col, row=row)
    dist.destroy_process_group()


@pytest.mark.parametrize("qtype,n,k", [(12, 24, 1280), (14, 16, 768), (8, 12, 512)])
def test_two_rank_column_and_row_parallel(tmp_path, qtype, n, k):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), qtype, n, k, str(tmp_path)), nprocs=world, join=True)
    r = np.load(tmp_path / "res.npz")
    assert np.array_equal(r["col"], r["full"])                           # same rows, same arithmetic
    assert np.allclose(r["row"], r["full"], rtol=1e-5, atol=1e-6)        # fp32 sum of two fp64-accumulated partials


def test_shard_bytes_cover_the_tensor_exactly():
    import magnitude_b200 as mb
    from magnitude_b200 import tp

    rng = np.random.default_rng(1)
    for qtype, (be, bb) in tp.BLOCK.items():
        n, k = 20, 5 * 256
        packed = rng.integers(0, 256, size=(n, k // be * bb), dtype=np.uint8)
        for world in (1, 2, 3, 8):
            cols = [tp.shard_gguf(qtype, packed, n, k, mb.SPLIT_COLUMN, r, world, 4)[0] for r in range(world)]
            assert np.array_equal(np.concatenate(cols, axis=0), packed)
            rows = [tp.shard_gguf(qtype, packed, n, k, mb.SPLIT_ROW, r, world)[0] for r in range(world)]
            assert np.array_equal(np.concatenate(rows, axis=1), packed)
