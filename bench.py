#!/usr/bin/env python
"""Benchmark of the quantized projection path.

Workload (N = 1): Q4_K decode GEMV, batch 1, Llama-3-8B MLP shapes — per layer gate and up
(14336 x 4096) and down (4096 x 14336), 32 layers, activations bf16, outputs fp32.  A step is one
pass over all 32 layers' projections: 96 weight matrices, 3.17 GB of packed blocks, so every step
streams far more than the 126 MB L2.  Inputs are seeded synthetic tensors (N(0, 0.02) weights
encoded to Q4_K, N(0, 1) activations); layers reuse one encoded gate/up/down set at distinct HBM
addresses.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

For N > 1 launch under torchrun; weights are split tensor-parallel (gate/up by rows, down by K
superblocks with one all-reduce per down projection).  Rank 0 prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "q4_k_decode_gemv_weight_bandwidth"
UNIT = "GB/s"
LAYERS = 32
HIDDEN, INTER = 4096, 14336
Q4_K = 12
FALLBACK_HBM_GBS = 6650.0
FALLBACK_TFLOPS = 1400.0
# DRAM traffic of the dominant kernels from one ncu capture each (dram__bytes_read.sum +
# dram__bytes_write.sum per launch; summaries under profiles/).  The decode figure was captured on a
# 4-layer launch and is proportional to the layers a launch streams, so it is kept as a ratio to
# the algorithmic bytes; a prefill launch is one whole product whatever the number of copies.
NCU_DECODE_TRAFFIC_PER_ALGORITHMIC_BYTE = 1.012
NCU_PREFILL_TRAFFIC_BYTES_PER_LAUNCH = 73.9e6


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            return float(d["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


def algorithmic_bytes(n, k, m=1, x_bytes=2, y_bytes=4):
    return n * (k // 256) * 144 + m * k * x_bytes + m * n * y_bytes


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.samples = []
        self._stop = threading.Event()
        self._t = threading.Thread(target=self._run, daemon=True)

    def _run(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(
                    ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-i", str(self.index)],
                    capture_output=True, text=True, timeout=5).stdout.strip()
                if out:
                    self.samples.append([c.strip() for c in out.splitlines()[0].split(",")])
            except Exception:
                pass
            self._stop.wait(0.1)

    def __enter__(self):
        self._t.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        self._t.join(timeout=10)

    def summary(self):
        mhz, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            try:
                mhz.append(float(s[0]))
                mx.append(float(s[1]))
            except Exception:
                continue
            for nme, v in zip(names, s[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(nme)
        return {
            "sm_mhz": float(np.median(mhz)) if mhz else None,
            "sm_max_mhz": max(mx) if mx else None,
            "reasons": sorted(reasons),
            "samples": len(mhz),
        }


def dist_env():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


# ------------------------------------------------------------------------------------------------
# reference arm: the CPU path (integer block dots on re-quantized activations), all host threads
# ------------------------------------------------------------------------------------------------

def cpu_reference_pass(orc, mats, xs, reps):
    """Times `reps` passes over the given (packed, n, k) matrices; returns seconds per pass."""
    t0 = time.perf_counter()
    for _ in range(reps):
        for (p, n, k), x in zip(mats, xs):
            orc.matmul_cpu(Q4_K, p, n, k, x)
    return (time.perf_counter() - t0) / reps


def make_host_layer(seed=0):
    from magnitude_b200 import ggml_quant as gq

    gate = gq.synth_weights(Q4_K, INTER, HIDDEN, seed)
    up = gq.synth_weights(Q4_K, INTER, HIDDEN, seed + 1)
    down = gq.synth_weights(Q4_K, HIDDEN, INTER, seed + 2)
    return gate, up, down


def run_reference(args):
    rank, _, world = dist_env()
    if rank != 0:
        return
    # torchrun pins OMP_NUM_THREADS to 1 for its workers; this arm is the CPU path on all host cores
    os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)
    from oracle import oracle as orc  # the CPU restatement of the reference's path, timed here

    orc.build()
    from magnitude_b200 import ggml_quant as gq

    gate, up, down = make_host_layer()
    rng = np.random.default_rng(1)
    xh = gq.f32_to_bf16_bits(rng.standard_normal((1, HIDDEN), dtype=np.float32)).astype(np.uint32) << 16
    xi = gq.f32_to_bf16_bits(rng.standard_normal((1, INTER), dtype=np.float32)).astype(np.uint32) << 16
    xh, xi = xh.view(np.float32), xi.view(np.float32)
    # distinct copies per layer so the host caches do not hold the weights between layers
    layers = min(LAYERS, 8)
    mats, xs = [], []
    for l in range(layers):
        mats += [(gate.copy(), INTER, HIDDEN), (up.copy(), INTER, HIDDEN), (down.copy(), HIDDEN, INTER)]
        xs += [xh, xh, xi]
    bytes_pass = sum(algorithmic_bytes(n, k) for _, n, k in mats)
    for _ in range(max(args.warmup, 1)):
        cpu_reference_pass(orc, mats, xs, 1)
    per = []
    for _ in range(args.steps):
        per.append(cpu_reference_pass(orc, mats, xs, 1))
    sec = float(np.sum(per)) / len(per)
    value = bytes_pass / sec / 1e9
    cores = orc.num_threads()
    sample = f"{layers} of {LAYERS} layers per step (gate, up, down each), all {cores} host threads"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3 * (LAYERS / layers),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "u8/int32 block dots, fp32 accumulate",
        "data": "synthetic", "config": workload_config(args.gpus),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def workload_config(n_gpus):
    return {
        "workload": f"configs[1]: Q4_K decode GEMV, batch 1, Llama-3-8B MLP shapes, {LAYERS} layers per step"
                    + ("" if LAYERS == 32 else " (reduced profiling case, not the benchmark)"),
        "shapes": "gate/up 14336x4096, down 4096x14336, x bf16 1xK, y fp32",
        "layers": LAYERS,
        "weight_bytes_per_step": LAYERS * 3 * (INTER * HIDDEN // 256 * 144),
        "l2": f"inputs larger than L2 ({LAYERS * 3 * (INTER * HIDDEN // 256 * 144) / 1e9:.2f} GB of distinct weight buffers per step)",
        "parallelism": f"tp{n_gpus}" if n_gpus > 1 else "single",
    }


def mark_diagnostic(line, args):
    if getattr(args, "no_exchange", False) and line.get("n_gpus", 1) > 1:
        line["invalid"] = "diagnostic run without the all-reduce: partial sums only"
    return line


# ------------------------------------------------------------------------------------------------
# the CUDA arm
# ------------------------------------------------------------------------------------------------

def run_b200(args):
    import torch

    rank, local_rank, world = dist_env()
    if world != args.gpus and world != 1:
        raise SystemExit(f"--gpus {args.gpus} does not match WORLD_SIZE {world}")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the projection path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod

        dist = dist_mod
        dist.init_process_group("nccl", device_id=dev)

    import magnitude_b200 as mb
    from magnitude_b200 import ggml_quant as gq

    be = mb.Backend(local_rank)
    # row-parallel sums: the library's one-kernel peer-memory all-reduce (NVLink stores and loads);
    # --nccl times torch.distributed's NCCL all-reduce in its place
    use_peer = world > 1 and not args.nccl
    if use_peer:
        be.peer_setup(dist)
    gate_h, up_h, down_h = make_host_layer()
    if world > 1:
        g0 = be.upload_shard(Q4_K, gate_h, INTER, HIDDEN, mb.SPLIT_COLUMN, rank, world, 256)
        u0 = be.upload_shard(Q4_K, up_h, INTER, HIDDEN, mb.SPLIT_COLUMN, rank, world, 256)
        d0 = be.upload_shard(Q4_K, down_h, HIDDEN, INTER, mb.SPLIT_ROW, rank, world)
    else:
        g0 = be.upload(Q4_K, gate_h, INTER, HIDDEN)
        u0 = be.upload(Q4_K, up_h, INTER, HIDDEN)
        d0 = be.upload(Q4_K, down_h, HIDDEN, INTER)
    gates, ups, downs = [g0], [u0], [d0]
    for _ in range(LAYERS - 1):
        gates.append(g0.clone())
        ups.append(u0.clone())
        downs.append(d0.clone())
    n_gu, k_d = g0.n, d0.k

    rng = np.random.default_rng(1)
    x_h = torch.from_numpy(rng.standard_normal((1, HIDDEN), dtype=np.float32)).to(torch.bfloat16)
    x_i = torch.from_numpy(rng.standard_normal((1, INTER), dtype=np.float32)).to(torch.bfloat16)
    x_hd = x_h.to(dev)
    lo, hi = mb.shard_range(Q4_K, HIDDEN, INTER, mb.SPLIT_ROW, rank, world) if world > 1 else (0, INTER)
    x_id = x_i[:, lo:hi].contiguous().to(dev)
    y_g = torch.empty((1, n_gu), dtype=torch.float32, device=dev)
    y_u = torch.empty((1, n_gu), dtype=torch.float32, device=dev)
    y_d = torch.empty((1, HIDDEN), dtype=torch.float32, device=dev)

    stream = torch.cuda.Stream(device=dev)

    # One decode plan holds the whole step: 64 projection jobs run by one persistent launch, the
    # weights of job i+1 streaming while job i is reduced and stored.  Under tensor parallelism the
    # all-reduce after every down projection cuts the step into one two-job plan per layer.
    fused = use_peer and not args.unfused and not args.per_launch and not args.no_exchange
    if args.per_launch:
        plans = None
        launches_per_step = 2 * LAYERS
    elif world == 1 or fused:
        jobs = []
        for l in range(LAYERS):
            jobs.append(([gates[l], ups[l]], x_hd, [y_g, y_u]))
            jobs.append(([downs[l]], x_id, [y_d]))
        # tensor parallel: the down projections' partial sums are added up over the ranks inside the launch
        plans = [be.plan(jobs, sum_ranks=[fused and (i % 2 == 1) for i in range(len(jobs))])]
        launches_per_step = 1
    else:
        plans = [be.plan([([gates[l], ups[l]], x_hd, [y_g, y_u]), ([downs[l]], x_id, [y_d])]) for l in range(LAYERS)]
        launches_per_step = LAYERS

    def sum_ranks():
        if args.no_exchange or fused:
            return
        if use_peer:
            be.allreduce(y_d, stream=stream)
        else:
            with torch.cuda.stream(stream):
                dist.all_reduce(y_d)

    def step_device():
        if plans is None:
            for l in range(LAYERS):
                be.project_multi([gates[l], ups[l]], x_hd, outs=[y_g, y_u], stream=stream)
                be.project(downs[l], x_id, out=y_d, stream=stream)
                if world > 1:
                    sum_ranks()
        else:
            for pl in plans:
                pl.run(stream=stream)
                if world > 1:
                    sum_ranks()

    # capture one step in a CUDA graph (launch-bound inner loop); fall back to direct launches
    graph = None
    with torch.cuda.stream(stream):
        step_device()
    stream.synchronize()
    be.sync(stream)
    if not args.no_graph:
        try:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                step_device()
            graph = g
        except Exception as exc:  # pragma: no cover - depends on driver behaviour
            if rank == 0:
                print(f"# graph capture unavailable ({type(exc).__name__}: {exc}); timing direct launches", file=sys.stderr)
            graph = None
            torch.cuda.synchronize()

    def run_step():
        if graph is not None:
            with torch.cuda.stream(stream):
                graph.replay()
        else:
            step_device()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        run_step()
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clocks:
        barrier()
        with torch.cuda.stream(stream):
            ev0.record(stream)
        for _ in range(args.steps):
            run_step()
        with torch.cuda.stream(stream):
            ev1.record(stream)
        barrier()
        ms_total = ev0.elapsed_time(ev1)
        # keep sampling clocks under the same load for a moment so short runs still get samples
        t_end = time.time() + 0.6
        while time.time() < t_end:
            run_step()
        torch.cuda.synchronize()
    be.sync(stream)
    if world > 1:
        t = torch.tensor([ms_total], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    ms_step = ms_total / args.steps

    # whole-job algorithmic bytes per step (all ranks): weights + activations + outputs
    per_layer = 2 * algorithmic_bytes(INTER, HIDDEN) + algorithmic_bytes(HIDDEN, INTER)
    bytes_step = LAYERS * per_layer
    value = bytes_step / (ms_step * 1e-3) / 1e9

    # ---- end to end through the host-buffer entry point (pinned host in, pinned host out) ----
    xh_pin = x_h.clone().pin_memory()
    xi_pin = x_i[:, lo:hi].contiguous().pin_memory()
    yg_pin = torch.empty((1, n_gu), dtype=torch.float32).pin_memory()
    yu_pin = torch.empty((1, n_gu), dtype=torch.float32).pin_memory()
    yd_pin = torch.empty((1, HIDDEN), dtype=torch.float32).pin_memory()
    yd_dev = torch.empty((1, HIDDEN), dtype=torch.float32, device=dev)

    xhd_e2e = torch.empty_like(x_hd)
    xid_e2e = torch.empty_like(x_id)
    if plans is not None:
        if world == 1 or fused:
            e2e_plans = [be.plan([j for l in range(LAYERS) for j in (([gates[l], ups[l]], xhd_e2e, [y_g, y_u]), ([downs[l]], xid_e2e, [y_d]))],
                                 sum_ranks=[fused and (i % 2 == 1) for i in range(2 * LAYERS)])]
        else:
            e2e_plans = [be.plan([([gates[l], ups[l]], xhd_e2e, [y_g, y_u]), ([downs[l]], xid_e2e, [y_d])]) for l in range(LAYERS)]

    def step_e2e():
        if plans is None:
            for l in range(LAYERS):
                be.project_host_ptr([gates[l], ups[l]], xh_pin.data_ptr(), mb.TYPE_BF16, 1, HIDDEN,
                                    [yg_pin.data_ptr(), yu_pin.data_ptr()], mb.TYPE_F32, [n_gu, n_gu])
                be.project_host_ptr([downs[l]], xi_pin.data_ptr(), mb.TYPE_BF16, 1, k_d,
                                    [yd_pin.data_ptr()], mb.TYPE_F32, [HIDDEN])
            return
        # host activations in, one plan launch (per layer under TP), host results out
        with torch.cuda.stream(stream):
            xhd_e2e.copy_(xh_pin, non_blocking=True)
            xid_e2e.copy_(xi_pin, non_blocking=True)
        for pl in e2e_plans:
            pl.run(stream=stream)
            if world > 1:
                sum_ranks()
        with torch.cuda.stream(stream):
            yg_pin.copy_(y_g, non_blocking=True)
            yu_pin.copy_(y_u, non_blocking=True)
            yd_pin.copy_(y_d, non_blocking=True)
        stream.synchronize()

    e2e_steps = max(3, min(args.steps, 10))
    for _ in range(2):
        step_e2e()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        step_e2e()
    barrier()
    e2e_s = (time.perf_counter() - t0) / e2e_steps
    if world > 1:
        t = torch.tensor([e2e_s], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e = {
        "value": bytes_step / e2e_s / 1e9, "unit": UNIT,
        "h2d_bytes_per_step": (LAYERS if plans is None else 1) * (HIDDEN * 2 + k_d * 2) * world,
        "d2h_bytes_per_step": (LAYERS if plans is None else 1) * (2 * n_gu * 4 + HIDDEN * 4) * world,
        "ms_per_step": e2e_s * 1e3,
        "api": ("b200q_matmul_multi_host per projection group" if plans is None else
                "pinned host activations -> device, b200q_plan_run (whole step), results -> pinned host, synchronize"),
    }

    # Teardown: the captured graph holds NCCL kernels, so it goes before anything of the process
    # group does; ranks leave together, and they leave through os._exit so that no destructor can
    # wait on a peer that has already gone.
    used_graph = graph is not None
    graph = None
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    if rank != 0:
        sys.stdout.flush()
        os._exit(0)

    peak, peak_src = peaks()
    # dominant kernel: stream_kernel<M=1, Q4_K> running the step's 64 projection jobs (the
    # activation-prep launch before it takes about 1 % of the step);
    # achieved = algorithmic bytes of this rank's launches / their device time
    rank_bytes = bytes_step / world
    achieved = rank_bytes / (ms_step * 1e-3) / 1e9
    roofline = {
        "bound": "hbm", "kernel": "stream_kernel<M=1,Q4_K>", "achieved": achieved, "peak": peak, "unit": "GB/s",
        "frac": achieved / peak, "peak_source": f"of {peak_src}",
        "traffic": NCU_DECODE_TRAFFIC_PER_ALGORITHMIC_BYTE * rank_bytes / launches_per_step,
        "traffic_source": "ncu capture of a 4-layer launch, scaled by the bytes a launch streams",
        "bytes_per_launch": rank_bytes / launches_per_step,
        "us_per_launch": ms_step * 1e3 / launches_per_step,
        "note": "per-rank algorithmic bytes per step / per-step device time (CUDA events on the launch stream)"
                + (("; includes the sum over ranks of each down projection ("
                    + ("peer-memory stores and loads inside the launch" if fused else "peer-memory kernel" if use_peer else "NCCL") + ")")
                   if world > 1 else ""),
    }

    cpu_baseline = None
    if world == 1 and not args.no_cpu_baseline:
        from oracle import oracle as orc  # CPU-baseline leg only

        orc.build()
        xh32 = x_h.float().numpy()
        xi32 = x_i.float().numpy()
        mats = [(gate_h, INTER, HIDDEN), (up_h, INTER, HIDDEN), (down_h, HIDDEN, INTER)]
        xs = [xh32, xh32, xi32]
        cpu_reference_pass(orc, mats, xs, 1)
        reps, spent, t_start = 0, [], time.perf_counter()
        while time.perf_counter() - t_start < 10.0 and reps < 400:
            spent.append(cpu_reference_pass(orc, mats, xs, 1))
            reps += 1
        sec = float(np.median(spent))
        cpu_baseline = {
            "value": per_layer / sec / 1e9, "unit": UNIT, "cores": orc.num_threads(), "kind": "port",
            "sample": f"one layer (gate, up, down) x {reps} passes, median; integer block-dot CPU path, OpenMP over rows",
        }

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "u8 x s16 integer block dots (dp4a), fp32 accumulate", "data": "synthetic",
        "config": workload_config(world), "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e,
        # a plan run = the activation-prep launch + the streaming launch; the unfused TP mode adds the all-reduce kernel
        "gpu_launches": launches_per_step * ((2 if plans is not None else 1) + (1 if (use_peer and not fused) else 0)) * args.steps,
        "cuda_graph": used_graph,
        "clocks": clocks.summary(),
    }
    print(json.dumps(mark_diagnostic(line, args)))
    sys.stdout.flush()
    if dist is not None:
        os._exit(0)


# ------------------------------------------------------------------------------------------------
# secondary line: the prefill GEMM (configs[3]) — tcgen05 route, reported in TFLOP/s
# ------------------------------------------------------------------------------------------------

def run_prefill(args):
    """M=2048 tokens x Q4_K 14336x4096, bf16 activations (1% of channels x20), bf16 output.

    A step multiplies the same activations by `copies` distinct weight buffers (default 8, 264 MB,
    larger than L2).  The reference arm of this line is the CPU path on a bounded token sample.
    """
    M, N, K = 2048, INTER, HIDDEN
    copies = max(1, min(args.layers, 8)) if args.layers != 32 else 8
    rank, local_rank, world = dist_env()
    if world > 1:
        if rank == 0:
            print(json.dumps({"metric": "q4_k_prefill_gemm_tflops", "unavailable": "the prefill line is single-GPU"}))
        return
    from magnitude_b200 import ggml_quant as gq

    w_h = gq.synth_weights(Q4_K, N, K, 0)
    rng = np.random.default_rng(3)
    x32 = rng.standard_normal((M, K), dtype=np.float32)
    x32[:, rng.choice(K, K // 100, replace=False)] *= np.float32(20.0)
    flops_one = 2.0 * M * N * K
    cfg = {"workload": "configs[3]: Q4_K prefill GEMM, M=2048 K=4096 N=14336, bf16 activations with 1% outlier channels, bf16 output",
           "weight_copies_per_step": copies, "l2": f"{copies} distinct weight buffers ({copies * N * K // 256 * 144 / 1e6:.0f} MB) per step",
           "parallelism": "single"}

    if args.impl == "reference":
        os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)
        from oracle import oracle as orc

        orc.build()
        rows = 8                                         # bounded sample: 8 of the 2048 token rows
        xs = np.ascontiguousarray((gq.f32_to_bf16_bits(x32[:rows]).astype(np.uint32) << 16).view(np.float32))
        for _ in range(max(args.warmup, 1)):
            orc.matmul_cpu(Q4_K, w_h, N, K, xs)
        t0 = time.perf_counter()
        for _ in range(args.steps):
            orc.matmul_cpu(Q4_K, w_h, N, K, xs)
        sec = (time.perf_counter() - t0) / args.steps
        val = 2.0 * rows * N * K / sec / 1e12
        cores = orc.num_threads()
        print(json.dumps({"impl": "reference", "metric": "q4_k_prefill_gemm_tflops", "value": val, "unit": "TFLOP/s", "n_gpus": 1,
                          "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3 * (M / rows) * copies,
                          "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "u8/int32 block dots",
                          "data": "synthetic", "config": cfg,
                          "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                                           "sample": f"{rows} of {M} token rows against one weight, all {cores} host threads"},
                          "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))
        return

    import torch

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the projection path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    import magnitude_b200 as mb

    be = mb.Backend(local_rank)
    w0 = be.upload(Q4_K, w_h, N, K)
    ws = [w0] + [w0.clone() for _ in range(copies - 1)]
    x_host = torch.from_numpy(x32).to(torch.bfloat16)
    x = x_host.to(dev)
    y = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
    stream = torch.cuda.Stream(device=dev)

    def step():
        for w in ws:
            be.project(w, x, out=y, stream=stream)

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    if be.last_route()[0] != mb.ROUTE_GEMM:
        raise SystemExit("prefill did not take the tcgen05 route")
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clocks:
        torch.cuda.synchronize()
        ev0.record(stream)
        for _ in range(args.steps):
            step()
        ev1.record(stream)
        torch.cuda.synchronize()
        ms_step = ev0.elapsed_time(ev1) / args.steps
        t_end = time.time() + 0.6
        while time.time() < t_end:
            step()
        torch.cuda.synchronize()
    be.sync(stream)
    value = flops_one * copies / (ms_step * 1e-3) / 1e12

    x_pin = x_host.clone().pin_memory()
    y_pin = torch.empty((M, N), dtype=torch.bfloat16).pin_memory()
    x_e = torch.empty_like(x)

    def step_e2e():
        with torch.cuda.stream(stream):
            x_e.copy_(x_pin, non_blocking=True)
        for w in ws:
            be.project(w, x_e, out=y, stream=stream)
        with torch.cuda.stream(stream):
            y_pin.copy_(y, non_blocking=True)
        stream.synchronize()

    step_e2e()
    t0 = time.perf_counter()
    n_e2e = max(3, min(args.steps, 10))
    for _ in range(n_e2e):
        step_e2e()
    e2e_s = (time.perf_counter() - t0) / n_e2e

    peak, src, burst = FALLBACK_TFLOPS, "fallback", None
    pk = ROOT / "MEASURED_PEAKS.json"
    if pk.exists():
        try:
            d = json.loads(pk.read_text())
            peak, src = float(d["bf16_tflops_sustained"]), "measured (sustained: the step is a run of products back to back)"
            burst = float(d["bf16_tflops"])
        except Exception:
            pass
    line = {
        "metric": "q4_k_prefill_gemm_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "fp16 x fp16 tcgen05.mma, fp32 accumulate in TMEM (weights dequantized exactly to fp16, activations bf16 -> fp16)",
        "data": "synthetic", "config": cfg,
        "roofline": {"bound": "tensor", "kernel": "gemm_tc_pair_kernel<Q4_K> (+ convert_x_vec8_kernel per product)", "achieved": value, "peak": peak,
                     "unit": "TFLOP/s", "frac": value / peak, "peak_source": f"of {src}", "peak_burst": burst,
                     "frac_of_burst": (value / burst) if burst else None, "traffic": NCU_PREFILL_TRAFFIC_BYTES_PER_LAUNCH,
                     "us_per_launch": ms_step * 1e3 / copies,
                     "note": "2*M*N*K per product / device time per product, activation conversion launch included"},
        "cpu_baseline": None,
        "e2e": {"value": flops_one * copies / e2e_s / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": M * K * 2,
                "d2h_bytes_per_step": M * N * 2, "ms_per_step": e2e_s * 1e3,
                "api": "pinned host activations -> device, b200q_matmul per weight, last result -> pinned host, synchronize"},
        "gpu_launches": 2 * copies * args.steps, "clocks": clocks.summary(),
    }
    print(json.dumps(line))

# ------------------------------------------------------------------------------------------------
# secondary line: skinny batches (configs[2]) — speculative-decode verify, M in {2, 4, 8, 16}
# ------------------------------------------------------------------------------------------------

def run_skinny(args):
    """Fused-QKV Q4_K 6144x4096 and down Q6_K 4096x14336 against M = 2, 4, 8, 16 bf16 tokens.

    Every case multiplies the tokens by 16 distinct copies of the weight (more than L2 for both
    shapes) inside one CUDA graph, so the time is the device's, not the launching host's.
    """
    import torch

    rank, local_rank, world = dist_env()
    if world > 1 or args.impl == "reference":
        if rank == 0:
            print(json.dumps({"metric": "skinny_gemm_weight_bandwidth", "unavailable": "the skinny line is single-GPU and has no CPU arm"}))
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the projection path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    import magnitude_b200 as mb
    from magnitude_b200 import ggml_quant as gq

    be = mb.Backend(local_rank)
    if args.skinny_min_m:
        be.set_option(1, args.skinny_min_m)
    peak, src = peaks()
    copies = 16
    stream = torch.cuda.Stream(device=dev)
    cases, tot_bytes, tot_s = [], 0.0, 0.0
    with ClockSampler(local_rank) as clocks:
        for qt, name, n, k, blk in ((Q4_K, "Q4_K qkv", 6144, 4096, 144), (14, "Q6_K down", 4096, 14336, 210)):
            w0 = be.upload(qt, gq.synth_weights(qt, n, k, 0), n, k)
            ws = [w0] + [w0.clone() for _ in range(copies - 1)]
            wbytes = n * (k // 256) * blk
            for m in (2, 4, 8, 16):
                x = torch.randn(m, k, device=dev).to(torch.bfloat16)
                y = torch.empty((m, n), dtype=torch.float32, device=dev)

                plan = be.plan([([w], x, [y]) for w in ws]) if args.skinny_plan else None

                def step():
                    if plan is not None:       # the 16 independent products as one decode plan
                        plan.run(stream=stream)
                        return
                    for w in ws:
                        be.project(w, x, out=y, stream=stream)

                for _ in range(max(args.warmup, 3)):
                    step()
                stream.synchronize()
                route = be.last_route()[0]
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=stream):
                    step()
                ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                with torch.cuda.stream(stream):
                    g.replay()
                    ev0.record(stream)
                    for _ in range(args.steps):
                        g.replay()
                    ev1.record(stream)
                stream.synchronize()
                be.sync(stream)
                us = ev0.elapsed_time(ev1) * 1e3 / (args.steps * copies)
                algo = wbytes + m * k * 2 + m * n * 4
                cases.append({"weight": name, "N": n, "K": k, "M": m, "us_per_product": us, "GB/s": algo / us / 1e3,
                              "frac_of_hbm_peak": algo / us / 1e3 / peak,
                              "route": {mb.ROUTE_GEMV: "dp4a stream kernel", mb.ROUTE_SKINNY: "skinny kernel (mma.sync, exact bf16)",
                                        mb.ROUTE_GEMM: "tcgen05 GEMM, K split"}.get(route, str(route))})
                tot_bytes += algo
                tot_s += us * 1e-6
                del g, plan
            del ws, w0
    value = tot_bytes / tot_s / 1e9
    print(json.dumps({
        "metric": "skinny_gemm_weight_bandwidth", "value": value, "unit": UNIT, "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": tot_s * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "M <= 4: u8 x s16 dp4a; M >= 5: exact integer weights x bf16 in mma.sync, fp32 accumulate", "data": "synthetic",
        "config": {"workload": "configs[2]: skinny verify batches, Q4_K 6144x4096 and Q6_K 4096x14336, M in {2,4,8,16}, bf16 tokens, fp32 out",
                   "l2": f"{copies} distinct weight copies per case", "parallelism": "single"},
        "roofline": {"bound": "hbm", "achieved": value, "peak": peak, "unit": UNIT, "frac": value / peak, "peak_source": f"of {src}",
                     "traffic": None, "note": "algorithmic bytes of all eight cases / their device time"},
        "cases": cases, "cpu_baseline": None, "e2e": None, "gpu_launches": None, "clocks": clocks.summary(),
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["b200", "reference"], default="b200")
    ap.add_argument("--no-graph", action="store_true", help="time direct launches instead of a CUDA graph replay")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--per-launch", action="store_true", help="one launch per projection group instead of a decode plan")
    ap.add_argument("--nccl", action="store_true", help="N > 1: NCCL all-reduce instead of the peer-memory kernel")
    ap.add_argument("--unfused", action="store_true",
                    help="N > 1: one plan per layer followed by the peer-memory all-reduce kernel, instead of sums inside one launch")
    ap.add_argument("--no-exchange", action="store_true",
                    help="N > 1 diagnostic: skip the all-reduce (partial sums only; the line is marked invalid)")
    ap.add_argument("--layers", type=int, default=32,
                    help="layers per step (default 32 = the benchmark; a smaller count is a profiling case, named as such in config)")
    ap.add_argument("--skinny-plan", action="store_true",
                    help="skinny workload: run the 16 weight copies of a case as one decode plan instead of 16 calls")
    ap.add_argument("--skinny-min-m", type=int, default=0,
                    help="skinny workload: smallest M sent to the skinny kernel (default: the library's, 5)")
    ap.add_argument("--workload", choices=["decode", "prefill", "skinny"], default="decode",
                    help="decode = the headline Q4_K GEMV step; prefill = the M=2048 Q4_K GEMM (secondary line, TFLOP/s)")
    args = ap.parse_args()
    # last resort against a stuck collective or teardown: never hold a GPU box for more than 20 minutes
    wd = threading.Timer(1200.0, lambda: os._exit(3))
    wd.daemon = True
    wd.start()
    global LAYERS
    LAYERS = max(1, min(args.layers, 32))
    if args.workload == "prefill":
        run_prefill(args)
    elif args.workload == "skinny":
        run_skinny(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
