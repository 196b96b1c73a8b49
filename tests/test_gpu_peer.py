"""Peer-memory all-reduce on 2, 4 and 8 GPUs (skipped where the box has fewer): sums equal the
rank-ordered fp32 sum bit for bit on every rank, for aligned, ragged and tiny vectors whose length
changes from call to call, eagerly and replayed from a CUDA graph; and the sums over ranks inside a
decode plan."""
import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
import torch.distributed as dist  # noqa: E402
import torch.multiprocessing as mp  # noqa: E402


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    import sys
    from pathlib import Path

    sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import magnitude_b200 as mb

    be = mb.Backend(rank)
    be.peer_setup(dist)
    failed = []      # names of the checks that failed on this rank
    stream = torch.cuda.Stream()
    for it, count in enumerate([4096, 1000, 16384, 5, 4096, 4096, 14336, 3, 3584, 7168, 10752, 1000, 10752, 7168]):
        gens = [torch.Generator().manual_seed(100 * it + r) for r in range(world)]
        parts = [torch.randn(count, generator=g) for g in gens]          # every rank knows all partial vectors
        want = parts[0].clone()
        for r in range(1, world):
            want += parts[r]                                               # rank order, fp32
        y = parts[rank].cuda()
        be.allreduce(y, stream=stream)
        be.sync(stream)
        if not torch.equal(y.cpu(), want):
            failed.append(f"allreduce[{it}:{count}]")
    # replay from a graph: the call number lives on the device, so replays stay in step
    y = torch.empty(4096, device="cuda")
    src = torch.randn(4096, generator=torch.Generator().manual_seed(7 + rank)).cuda()
    others = [torch.randn(4096, generator=torch.Generator().manual_seed(7 + r)) for r in range(world)]
    want = others[0].clone()
    for r in range(1, world):
        want += others[r]
    with torch.cuda.stream(stream):
        y.copy_(src)
        be.allreduce(y, stream=stream)
    stream.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=stream):
        y.copy_(src)
        be.allreduce(y, stream=stream)
    for _ in range(20):
        with torch.cuda.stream(stream):
            g.replay()
    be.sync(stream)
    if not torch.equal(y.cpu(), want):
        failed.append("allreduce graph replay")
    # rank sums inside a decode plan: a row-parallel down projection per layer, three layers, run
    # twice and replayed from a graph; every rank must end with the full product
    from magnitude_b200 import ggml_quant as gq
    from oracle import oracle as orc

    n, k = 1024, 2048
    rngw = np.random.default_rng(5)
    ws_host = [gq.quantize(mb.TYPE_Q4_K, rngw.standard_normal((n, k), dtype=np.float32) * np.float32(0.02)) for _ in range(3)]
    x32 = rngw.standard_normal((1, k), dtype=np.float32)
    xb = torch.from_numpy(x32).to(torch.bfloat16)
    lo, hi = mb.shard_range(mb.TYPE_Q4_K, n, k, mb.SPLIT_ROW, rank, world)
    shards = [be.upload_shard(mb.TYPE_Q4_K, w, n, k, mb.SPLIT_ROW, rank, world) for w in ws_host]
    xs = xb[:, lo:hi].contiguous().cuda()
    outs = [torch.zeros(1, n, device="cuda") for _ in range(3)]
    plan = be.plan([([shards[i]], xs, [outs[i]]) for i in range(3)], sum_ranks=[True] * 3)
    refs = [orc.matmul_exact(mb.TYPE_Q4_K, ws_host[i], n, k, xb.float().numpy()) for i in range(3)]

    def check_outs():
        good = True
        for i in range(3):
            good &= bool(orc.within_tolerance(outs[i].cpu().numpy(), refs[i], 1e-3)[0])
        return good

    for _ in range(2):
        for o in outs:
            o.zero_()
        plan.run(stream=stream)
        be.sync(stream)
        if not check_outs():
            failed.append("plan sums")
    all_out = [torch.empty_like(outs[0]) for _ in range(world)]
    gathered = [t.cpu() for t in all_out]
    dist.all_gather(gathered, outs[0].cpu())
    if not all(bool(torch.equal(g_, gathered[0])) for g_ in gathered):      # bit-identical on every rank
        failed.append("plan sums differ between ranks")
    g2 = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g2, stream=stream):
        plan.run(stream=stream)
    for o in outs:
        o.zero_()
    for _ in range(5):
        with torch.cuda.stream(stream):
            g2.replay()
    be.sync(stream)
    if not check_outs():
        failed.append("plan sums, graph replay")
    del g2
    dist.barrier()
    # the NCCL path: joined with a host deadline, used for bf16 and for vectors beyond the peer limit
    uid = [mb.tp_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(uid, src=0)
    be.tp_init(rank, world, uid[0])
    for count, dtype in ((40000, torch.float32), (8192, torch.bfloat16)):
        parts = [torch.randn(count, generator=torch.Generator().manual_seed(900 + r)).to(dtype) for r in range(world)]
        want = torch.stack([p.float() for p in parts]).sum(0)
        yv = parts[rank].cuda()
        be.allreduce(yv, stream=stream)
        be.sync(stream)
        # bf16: every addition of the library's reduction rounds to 8 bits, at the size of the running sum
        bound = 2.0 ** -8 * world * torch.stack([p.float().abs() for p in parts]).sum(0) if dtype == torch.bfloat16 else 1e-5 * (1 + want.abs())
        if not bool(((yv.float().cpu() - want).abs() <= bound).all()):
            failed.append(f"nccl allreduce {dtype}")
    be.tp_finalize()
    dist.barrier()
    with open(os.path.join(out_dir, f"ok{rank}"), "w") as f:
        f.write("1" if not failed else "failed: " + ", ".join(failed))
    del g
    be.peer_detach()
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_peer_allreduce_and_plan_sums(tmp_path, world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert (tmp_path / f"ok{r}").read_text() == "1"
