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
superblocks with the rank sums taken inside the launch).  Rank 0 prints one JSON line.  Beside the
headline figure the N = 1 line carries: the host check of the step's results, the step with its real
dependencies (plain and as chained fused MLP blocks), a seconds-long replay, the prefill (TFLOP/s),
skinny-batch (one product per call, and as plans) and per-type calibration figures, a library arm (the vllm package's GGUF kernels) and the
CPU baseline.  --workload prefill | skinny | calibration | layer32b | library print those lines alone.
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
NCU_DECODE_TRAFFIC_PER_ALGORITHMIC_BYTE = 1.014
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


def sample_stats(samples_ms):
    """Median, median absolute deviation and spread of per-step device times (the reference keeps raw
    repetitions: inference/parity/cases/performance/backend-ops/native-perf-qualification.json:37-43)."""
    a = np.asarray(samples_ms, dtype=np.float64)
    med = float(np.median(a))
    mad = float(np.median(np.abs(a - med)))
    return {"median_ms": med, "mad_ms": mad, "min_ms": float(a.min()), "max_ms": float(a.max()),
            "relative_spread": float((a.max() - a.min()) / med) if med > 0 else None,
            "samples_ms": [round(float(v), 6) for v in a]}


def physical_cores():
    """Distinct (physical id, core id) pairs of /proc/cpuinfo; falls back to the logical count."""
    try:
        seen, phys, core = set(), None, None
        for line in open("/proc/cpuinfo"):
            if line.startswith("physical id"):
                phys = line.split(":")[1].strip()
            elif line.startswith("core id"):
                core = line.split(":")[1].strip()
            elif not line.strip():
                if phys is not None and core is not None:
                    seen.add((phys, core))
                phys = core = None
        if seen:
            return len(seen)
    except Exception:
        pass
    return os.cpu_count() or 1


def load_quant_module():
    """magnitude_b200/ggml_quant.py by file path: the CPU arm needs the synthetic-weight encoders but must
    not load the CUDA library that importing the package would."""
    import importlib.util

    spec = importlib.util.spec_from_file_location("b200q_ggml_quant", ROOT / "magnitude_b200" / "ggml_quant.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def calibration_row(tensor_type, bytes_per_second, launch_us, spread, count):
    """One row in the shape of the reference's hardware-calibration metric
    (inference/crates/icn-hardware/src/lib.rs:4043-4055; consumed at :1380-1382)."""
    return {"tensor_type": tensor_type, "routed": False, "bytes_per_second": bytes_per_second,
            "launch_microseconds": launch_us, "relative_spread": spread, "sample_count": count,
            "stable": bool(spread is not None and spread < 0.05)}


def p0_row(time_us, flops, bytes_moved, memory_bytes, n_runs):
    """The reference's backend-op performance row (inference/crates/icn-parity/src/decode.rs:548-562)."""
    return {"time_us": time_us, "flops": flops, "bandwidth_gb_s": bytes_moved / (time_us * 1e-6) / 1e9,
            "memory_kb": memory_bytes / 1024.0, "n_runs": n_runs}


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


def make_host_layer(seed=0, gq=None, encoder=None):
    """gate, up, down of one layer: N(0, 0.02) from seeds 0, 1, 2, encoded with the format's reference
    quantizer (the CUDA arm passes the library's, the CPU arm the oracle's: the same bytes)."""
    if gq is None:
        from magnitude_b200 import ggml_quant as gq

    gate = gq.synth_weights(Q4_K, INTER, HIDDEN, seed, encoder=encoder)
    up = gq.synth_weights(Q4_K, INTER, HIDDEN, seed + 1, encoder=encoder)
    down = gq.synth_weights(Q4_K, HIDDEN, INTER, seed + 2, encoder=encoder)
    return gate, up, down


def run_reference(args):
    rank, _, world = dist_env()
    if rank != 0:
        return
    # torchrun pins OMP_NUM_THREADS to 1 for its workers; this arm is the CPU path on all host cores
    os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)
    from oracle import oracle as orc  # the CPU restatement of the reference's path, timed here

    orc.build()
    gq = load_quant_module()

    gate, up, down = make_host_layer(gq=gq, encoder=orc.quantize)
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
    # the reference's CPU-resident parity cases run one thread (single-batch-logits.json:24-25): same pass, one layer
    one = []
    for _ in range(3):
        t0 = time.perf_counter()
        for (pk, n, k), x in zip(mats[:3], xs[:3]):
            orc.matmul_cpu(Q4_K, pk, n, k, x, threads=1)
        one.append(time.perf_counter() - t0)
    one_thread = sum(algorithmic_bytes(n, k) for _, n, k in mats[:3]) / float(np.median(one)) / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3 * (LAYERS / layers),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "u8/int32 block dots, fp32 accumulate",
        "data": "synthetic", "config": workload_config(args.gpus),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample,
                         "physical_cores": physical_cores(), "one_thread_value": one_thread,
                         "stats": sample_stats([p_ * 1e3 for p_ in per])},
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
    gate_h, up_h, down_h = make_host_layer(encoder=mb.quantize)
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
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    with ClockSampler(local_rank) as clocks:
        barrier()
        with torch.cuda.stream(stream):
            evs[0].record(stream)
        for i in range(args.steps):
            run_step()
            with torch.cuda.stream(stream):
                evs[i + 1].record(stream)
        barrier()
        ms_total = evs[0].elapsed_time(evs[-1])
        step_samples = [evs[i].elapsed_time(evs[i + 1]) for i in range(args.steps)]
        # keep sampling clocks under the same load for a moment so short runs still get samples
        t_end = time.time() + 0.6
        while time.time() < t_end:
            run_step()
        torch.cuda.synchronize()
    be.sync(stream)

    # ---- result check on the box that was timed (outside the timed region) -------------------------
    # every layer holds the same encoded matrices, so after a step y_d is the full down product
    # (summed over the ranks) and y_g this rank's rows of the gate product: compare with the exact
    # host product of the decoded blocks (numpy, fp64 accumulation).
    check = None
    if not args.no_exchange and not args.no_check:
        run_step()
        torch.cuda.synchronize()
        wd = gq.dequantize_q4_k(down_h, INTER).astype(np.float64)
        ref_d = (wd @ x_i.float().numpy().astype(np.float64).T).T
        r0, r1 = mb.shard_range(Q4_K, INTER, HIDDEN, mb.SPLIT_COLUMN, rank, world, 256) if world > 1 else (0, INTER)
        wg = gq.dequantize_q4_k(gate_h[r0:r1], HIDDEN).astype(np.float64)
        ref_g = (wg @ x_h.float().numpy().astype(np.float64).T).T

        def worst(got, ref):
            rms = float(np.sqrt(np.mean(ref * ref)))
            return float(np.max(np.abs(got - ref) / (1e-3 * np.maximum(np.abs(ref), rms))))

        w_d, w_g = worst(y_d.cpu().numpy().astype(np.float64), ref_d), worst(y_g.cpu().numpy().astype(np.float64), ref_g)
        check = {"max_err_over_tol": max(w_d, w_g), "down_summed_over_ranks": w_d, "gate_rows_of_this_rank": w_g,
                 "tolerance": "|err| <= 1e-3 * max(|ref|, rms(ref))", "ok": bool(max(w_d, w_g) <= 1.0)}
        if world > 1:
            t = torch.tensor([check["max_err_over_tol"]], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            check["max_err_over_tol"] = float(t.item())
            check["ok"] = bool(check["max_err_over_tol"] <= 1.0)
            check["ranks_checked"] = world

    # ---- two figures beside the headline (N = 1): the step with its real dependency, and a long run ----
    dependent = sustained = None
    if world == 1 and plans is not None and not args.quick:
        dep_plan = be.plan(jobs, waits=[i % 2 == 1 for i in range(len(jobs))])     # down waits for gate/up
        with torch.cuda.stream(stream):
            for _ in range(3):
                dep_plan.run(stream=stream)
        stream.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = max(5, min(args.steps, 20))
        with torch.cuda.stream(stream):
            e0.record(stream)
            for _ in range(reps):
                dep_plan.run(stream=stream)
            e1.record(stream)
        stream.synchronize()
        be.sync(stream)
        ms_dep = e0.elapsed_time(e1) / reps
        dependent = {"ms_per_step": ms_dep, "value": LAYERS * (2 * algorithmic_bytes(INTER, HIDDEN) + algorithmic_bytes(HIDDEN, INTER)) / (ms_dep * 1e-3) / 1e9,
                     "unit": UNIT, "note": "same step, every down projection flagged as reading what gate/up wrote (one consumer team, grid counter between jobs)"}
        dep_plan.close()
        # The MLP block as a model runs it: h = silu(gate x) * (up x) in the gate/up job's epilogue, down
        # reads h and adds into the residual stream x, the next layer's gate/up reads that stream.
        x_res = torch.empty((1, HIDDEN), dtype=torch.float32, device=dev)
        h_mid = torch.empty((1, INTER), dtype=torch.float32, device=dev)
        x0_res = x_h.float()
        gamma = torch.from_numpy(np.random.default_rng(7).uniform(0.5, 1.5, HIDDEN).astype(np.float32)).to(dev)
        norm_eps = 1e-5

        def fused_plan(n_layers):
            fj, fw, fg, fa, fn = [], [], [], [], []
            for l in range(n_layers):
                fj += [([gates[l], ups[l]], x_res, [h_mid]), ([downs[l]], h_mid, [x_res])]
                fw += [l > 0, True]
                fg += [True, False]
                fa += [False, True]
                fn += [gamma, None]                       # RMSNorm of the stream on the gate/up job's load
            return be.plan(fj, waits=fw, swiglu=fg, accumulate=fa, norms=fn, norm_eps=norm_eps)

        fcheck = None
        if not args.no_check:
            two = fused_plan(2)
            x_res.copy_(x0_res)
            two.run(stream=torch.cuda.current_stream())
            torch.cuda.synchronize()
            be.sync()
            wg_f = gq.dequantize_q4_k(gate_h, HIDDEN).astype(np.float64)
            wu_f = gq.dequantize_q4_k(up_h, HIDDEN).astype(np.float64)
            wd_f = gq.dequantize_q4_k(down_h, INTER).astype(np.float64)
            xr = x0_res.cpu().numpy().astype(np.float64)[0]
            gam = gamma.cpu().numpy().astype(np.float64)
            for _ in range(2):
                xn = xr / np.sqrt(np.mean(xr * xr) + norm_eps) * gam
                gv, uv = wg_f @ xn, wu_f @ xn
                xr = xr + wd_f @ (gv / (1.0 + np.exp(-gv)) * uv)
            del wg_f, wu_f, wd_f
            got = x_res.cpu().numpy().astype(np.float64)[0]
            rms = float(np.sqrt(np.mean(xr * xr)))
            werr = float(np.max(np.abs(got - xr) / (5e-3 * np.maximum(np.abs(xr), rms))))
            fcheck = {"max_err_over_tol": werr, "ok": bool(werr <= 1.0), "what": "residual stream after two fused layers", "tolerance": "5e-3 (two chained layers)"}
            two.close()
        fplan = fused_plan(LAYERS)
        with torch.cuda.stream(stream):
            for _ in range(3):
                fplan.run(stream=stream)
        stream.synchronize()
        with torch.cuda.stream(stream):
            e0.record(stream)
            for _ in range(reps):
                fplan.run(stream=stream)
            e1.record(stream)
        stream.synchronize()
        be.sync(stream)
        ms_f = e0.elapsed_time(e1) / reps
        dependent["fused_layer"] = {"ms_per_step": ms_f, "value": LAYERS * (2 * algorithmic_bytes(INTER, HIDDEN) + algorithmic_bytes(HIDDEN, INTER)) / (ms_f * 1e-3) / 1e9,
                                    "unit": UNIT, "check": fcheck,
                                    "note": "32 chained MLP blocks: RMSNorm on the gate/up job's activation load, SwiGLU in its epilogue, down adds into the "
                                            "residual stream, every job waits for the one before"}
        fplan.close()
        with ClockSampler(local_rank) as long_clocks:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            n_long = 0
            with torch.cuda.stream(stream):
                e0.record(stream)
            t_end = time.time() + 2.5
            while time.time() < t_end:
                for _ in range(50):
                    run_step()
                n_long += 50
                stream.synchronize()
            with torch.cuda.stream(stream):
                e1.record(stream)
            stream.synchronize()
        ms_long = e0.elapsed_time(e1) / n_long
        lc = long_clocks.summary()
        sustained = {"ms_per_step": ms_long, "steps": n_long, "seconds": e0.elapsed_time(e1) / 1e3, "sm_mhz": lc["sm_mhz"], "reasons": lc["reasons"],
                     "ms_x_mhz": ms_long * lc["sm_mhz"] if lc["sm_mhz"] else None,
                     "value": LAYERS * (2 * algorithmic_bytes(INTER, HIDDEN) + algorithmic_bytes(HIDDEN, INTER)) / (ms_long * 1e-3) / 1e9, "unit": UNIT}
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
        # the CPU path is timed by this script's own reference arm in a process of its own, so that this
        # figure and the reference arm's are taken in the same process state (no CUDA runtime, one OpenMP pool)
        try:
            env = dict(os.environ)
            env.pop("OMP_NUM_THREADS", None)
            out = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "20", "--warmup", "2"],
                                 capture_output=True, text=True, timeout=600, env=env).stdout.strip().splitlines()
            cpu_baseline = json.loads(out[-1])["cpu_baseline"]
        except Exception as exc:  # pragma: no cover
            cpu_baseline = {"value": None, "unit": UNIT, "cores": os.cpu_count(), "kind": "port", "sample": f"failed: {exc}"}

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "u8 x s16 integer block dots (dp4a), fp32 accumulate", "data": "synthetic",
        "config": workload_config(world), "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e,
        # a plan run = the activation-prep launch + the streaming launch; the unfused TP mode adds the all-reduce kernel
        "gpu_launches": launches_per_step * ((2 if plans is not None else 1) + (1 if (use_peer and not fused) else 0)) * args.steps,
        "cuda_graph": used_graph,
        "clocks": clocks.summary(),
        "stats": sample_stats(step_samples),
        "check": check,
        "dependent": dependent,
        "sustained": sustained,
    }
    st = line["stats"]
    launch_us = None
    line["p0"] = p0_row(st["median_ms"] * 1e3 / (3 * LAYERS), 2.0 * INTER * HIDDEN, rank_bytes / (3 * LAYERS),
                        LAYERS * 3 * (INTER * HIDDEN // 256 * 144) / world, args.steps)
    line["p0"]["note"] = "per projection (MUL_MAT, Q4_K, M = 1): median step time / 96 projections"
    line["calibration"] = [calibration_row("Q4_K", rank_bytes / (st["median_ms"] * 1e-3), launch_us, st["relative_spread"], args.steps)]
    if world == 1 and not args.quick and args.workload == "decode":
        # the other two halves of the metric, measured after the headline region on the same box
        sec_args = argparse.Namespace(**vars(args))
        sec_args.steps, sec_args.warmup = min(args.steps, 10), 3
        line["secondary"] = {}
        for name, fn in (("prefill", run_prefill), ("skinny", run_skinny), ("calibration", run_calibration)):
            try:
                line["secondary"][name] = fn(sec_args, emit=False)
            except Exception as exc:  # pragma: no cover
                line["secondary"][name] = {"unavailable": f"{type(exc).__name__}: {exc}"}
        try:      # the same verify batches as the engine would issue them inside a step: one plan per case
            plan_args = argparse.Namespace(**vars(sec_args))
            plan_args.skinny_plan = True
            line["secondary"]["skinny_plan"] = run_skinny(plan_args, emit=False)
        except Exception as exc:  # pragma: no cover
            line["secondary"]["skinny_plan"] = {"unavailable": f"{type(exc).__name__}: {exc}"}
        cal = line["secondary"].get("calibration")
        if isinstance(cal, dict) and "rows" in cal:
            line["calibration"] = cal["rows"]
        # a second GPU baseline: the same projections through the vllm package's GGUF mat-vec kernel, in a
        # process of its own (the package's import is heavy and must not disturb this one)
        try:
            out = subprocess.run([sys.executable, os.path.abspath(__file__), "--workload", "library", "--steps", "10", "--warmup", "3"],
                                 capture_output=True, text=True, timeout=240)
            rows = [json.loads(l) for l in out.stdout.splitlines() if l.startswith("{")]
            line["secondary"]["library_arm"] = rows[-1] if rows else {"unavailable": (out.stderr or "no output")[-300:]}
        except Exception as exc:  # pragma: no cover
            line["secondary"]["library_arm"] = {"unavailable": f"{type(exc).__name__}: {exc}"[:300]}
    print(json.dumps(mark_diagnostic(line, args)))
    sys.stdout.flush()
    if dist is not None:
        os._exit(0)


# ------------------------------------------------------------------------------------------------
# secondary line: the prefill GEMM (configs[3]) — tcgen05 route, reported in TFLOP/s
# ------------------------------------------------------------------------------------------------

def run_prefill(args, emit=True):
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

    w_h = None       # encoded below by whichever arm runs
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
        w_h = load_quant_module().synth_weights(Q4_K, N, K, 0, encoder=orc.quantize)
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
    w_h = gq.synth_weights(Q4_K, N, K, 0, encoder=mb.quantize)
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
        "roofline": {"bound": "tensor", "kernel": "gemm_tc_pair_kernel<Q4_K> (+ convert_x_vec8_kernel per product)", "achieved": value,
                     "peak": burst or peak, "unit": "TFLOP/s", "frac": value / (burst or peak),
                     "peak_source": f"of {'measured (burst: the timed region lasts tens of milliseconds)' if burst else src}",
                     "peak_sustained": peak, "frac_of_sustained": value / peak, "traffic": NCU_PREFILL_TRAFFIC_BYTES_PER_LAUNCH,
                     "us_per_launch": ms_step * 1e3 / copies,
                     "note": "2*M*N*K per product / device time per product, activation conversion launch included"},
        "cpu_baseline": None,
        "e2e": {"value": flops_one * copies / e2e_s / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": M * K * 2,
                "d2h_bytes_per_step": M * N * 2, "ms_per_step": e2e_s * 1e3,
                "api": "pinned host activations -> device, b200q_matmul per weight, last result -> pinned host, synchronize"},
        "gpu_launches": 2 * copies * args.steps, "clocks": clocks.summary(),
        "p0": p0_row(ms_step * 1e3 / copies, flops_one, N * K // 256 * 144 + M * K * 2 + M * N * 2, N * K // 256 * 144 + M * K * 2 + M * N * 2, args.steps * copies),
    }
    del ws, w0, x, y
    be.close()
    if not emit:
        return line
    print(json.dumps(line))

# ------------------------------------------------------------------------------------------------
# secondary line: skinny batches (configs[2]) — speculative-decode verify, M in {2, 4, 8, 16}
# ------------------------------------------------------------------------------------------------

def run_skinny(args, emit=True):
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
            w0 = be.upload(qt, gq.synth_weights(qt, n, k, 0, encoder=mb.quantize), n, k)
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
    be.close()
    line = {
        "metric": "skinny_gemm_weight_bandwidth", "value": value, "unit": UNIT, "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": tot_s * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "M <= 2: u8 x s16 dp4a; M >= 3: exact integer weights x bf16 in mma.sync, fp32 accumulate", "data": "synthetic",
        "config": {"workload": "configs[2]: skinny verify batches, Q4_K 6144x4096 and Q6_K 4096x14336, M in {2,4,8,16}, bf16 tokens, fp32 out",
                   "l2": f"{copies} distinct weight copies per case", "parallelism": "single",
                   "form": "the 16 products of a case as one decode plan" if args.skinny_plan else "one product per call"},
        "roofline": {"bound": "hbm", "achieved": value, "peak": peak, "unit": UNIT, "frac": value / peak, "peak_source": f"of {src}",
                     "traffic": None, "note": "algorithmic bytes of all eight cases / their device time"},
        "cases": cases, "cpu_baseline": None, "e2e": None, "gpu_launches": None, "clocks": clocks.summary(),
    }
    if not emit:
        return line
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------------
# configs[4]: one decoder layer of a 32B-class dense model under tensor parallelism, M = 1 and M = 4096
# ------------------------------------------------------------------------------------------------

L32_H, L32_I = 5120, 25600
L32 = [("q", Q4_K, 8192, L32_H), ("k", Q4_K, 1024, L32_H), ("v", 14, 1024, L32_H), ("o", Q4_K, L32_H, 8192),
       ("gate", Q4_K, L32_I, L32_H), ("up", Q4_K, L32_I, L32_H), ("down", 14, L32_H, L32_I)]
BLK_BYTES = {Q4_K: 144, 14: 210}


def run_layer32b(args, emit=True):
    """All seven projections of one layer (Q4_K_M mix), split tensor-parallel: q / k / v by heads and
    gate / up by rows in the 256-row units that match down's cut (no exchange); o and down along K at
    superblocks, their partial results added over the ranks.  Decode (M = 1): one plan per rank, the sums
    made inside the launch (peer memory).  Prefill (M = 4096): tcgen05 GEMMs, the row-parallel partials
    (bf16) summed by one NCCL all-reduce per projection, issued per M-chunk on a second stream so that it
    overlaps the next chunk's GEMM.  `--layers L` distinct copies of the layer per step (default 4: 1.24 GB)."""
    import torch

    rank, local_rank, world = dist_env()
    if args.impl == "reference":
        if rank == 0:
            print(json.dumps({"impl": "reference", "metric": "layer32b", "unavailable": "the layer workload has no CPU arm (see the decode line)"}))
        return None
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
    if world > 1:
        be.peer_setup(dist)
        uid = [mb.tp_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(uid, src=0)
        be.tp_init(rank, world, uid[0])
    layers = max(1, min(args.layers if args.layers != 32 else 4, 8))
    host = {name: gq.synth_weights(qt, n, k, seed, encoder=mb.quantize) for seed, (name, qt, n, k) in enumerate(L32)}
    split = {"q": (mb.SPLIT_COLUMN, 128), "k": (mb.SPLIT_COLUMN, 128), "v": (mb.SPLIT_COLUMN, 128), "o": (mb.SPLIT_ROW, 0),
             "gate": (mb.SPLIT_COLUMN, 256), "up": (mb.SPLIT_COLUMN, 256), "down": (mb.SPLIT_ROW, 0)}
    shards = []
    for _ in range(layers):
        if not shards:
            shards.append({name: be.upload_shard(qt, host[name], n, k, split[name][0], rank, world, split[name][1]) for name, qt, n, k in L32})
        else:
            shards.append({name: w.clone() for name, w in shards[0].items()})
    w0 = shards[0]
    weight_bytes = sum(n * (k // 256) * BLK_BYTES[qt] for _, qt, n, k in L32)
    stream = torch.cuda.Stream(device=dev)
    rng = np.random.default_rng(1)
    result = {}

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, warm=3):
        for _ in range(warm):
            fn()
        barrier()
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
        with torch.cuda.stream(stream):
            evs[0].record(stream)
        for i in range(steps):
            fn()
            with torch.cuda.stream(stream):
                evs[i + 1].record(stream)
        barrier()
        be.sync(stream)
        total = evs[0].elapsed_time(evs[-1])
        if world > 1:
            t = torch.tensor([total], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            total = float(t.item())
        return total / steps, [evs[i].elapsed_time(evs[i + 1]) for i in range(steps)]

    def worst(got, ref, rel):
        rms = float(np.sqrt(np.mean(ref * ref)))
        return float(np.max(np.abs(got - ref) / (rel * np.maximum(np.abs(ref), rms))))

    with ClockSampler(local_rank) as clocks:
        # ---------------- decode, M = 1 ----------------
        xh = torch.from_numpy(rng.standard_normal((1, L32_H), dtype=np.float32)).to(torch.bfloat16)
        xo = torch.from_numpy(rng.standard_normal((1, 8192), dtype=np.float32)).to(torch.bfloat16)
        xd = torch.from_numpy(rng.standard_normal((1, L32_I), dtype=np.float32)).to(torch.bfloat16)
        lo_o, hi_o = mb.shard_range(Q4_K, L32_H, 8192, mb.SPLIT_ROW, rank, world) if world > 1 else (0, 8192)
        lo_d, hi_d = mb.shard_range(14, L32_H, L32_I, mb.SPLIT_ROW, rank, world) if world > 1 else (0, L32_I)
        xh_d, xo_d, xd_d = xh.to(dev), xo[:, lo_o:hi_o].contiguous().to(dev), xd[:, lo_d:hi_d].contiguous().to(dev)
        yq = torch.empty((1, w0["q"].n), device=dev)
        yk = torch.empty((1, w0["k"].n), device=dev)
        yv = torch.empty((1, w0["v"].n), device=dev)
        yo = torch.empty((1, L32_H), device=dev)
        yg = torch.empty((1, w0["gate"].n), device=dev)
        yu = torch.empty((1, w0["up"].n), device=dev)
        yd = torch.empty((1, L32_H), device=dev)
        jobs, sums = [], []
        for s in shards:
            jobs += [([s["q"], s["k"]], xh_d, [yq, yk]), ([s["v"]], xh_d, [yv]), ([s["o"]], xo_d, [yo]),
                     ([s["gate"], s["up"]], xh_d, [yg, yu]), ([s["down"]], xd_d, [yd])]
            sums += [False, False, world > 1, False, world > 1]
        plan = be.plan(jobs, sum_ranks=sums)
        graph = None
        with torch.cuda.stream(stream):
            plan.run(stream=stream)
        stream.synchronize()
        try:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                plan.run(stream=stream)
            graph = g
        except Exception:
            torch.cuda.synchronize()

        def step_decode():
            if graph is not None:
                with torch.cuda.stream(stream):
                    graph.replay()
            else:
                plan.run(stream=stream)

        ms, samples = timed(step_decode, args.steps)
        step_decode()
        torch.cuda.synchronize()
        ref_o = (gq.dequantize(Q4_K, host["o"], 8192).astype(np.float64) @ xo.float().numpy().astype(np.float64).T).T
        ref_d = (gq.dequantize(14, host["down"], L32_I).astype(np.float64) @ xd.float().numpy().astype(np.float64).T).T
        chk = max(worst(yo.cpu().numpy().astype(np.float64), ref_o, 1e-3), worst(yd.cpu().numpy().astype(np.float64), ref_d, 1e-3))
        bytes_step = layers * (weight_bytes + 2 * (3 * L32_H + 8192 + L32_I) + 4 * (8192 + 2 * 1024 + 2 * L32_H + 2 * L32_I))
        peak, src = peaks()
        result["decode"] = {"ms_per_step": ms, "value": bytes_step / (ms * 1e-3) / 1e9, "unit": UNIT,
                            "roofline": {"bound": "hbm", "achieved": bytes_step / world / (ms * 1e-3) / 1e9, "peak": peak,
                                         "frac": bytes_step / world / (ms * 1e-3) / 1e9 / peak, "peak_source": f"of {src}",
                                         "note": "per-rank algorithmic bytes / device time, rank sums of o and down inside the launch"},
                            "stats": sample_stats(samples), "check": {"max_err_over_tol": chk, "ok": bool(chk <= 1.0)},
                            "jobs_per_launch": len(jobs), "cuda_graph": graph is not None}
        graph = None
        plan.close()

        # ---------------- prefill, M = 4096 ----------------
        M, chunks = 4096, 4
        mc = M // chunks
        X = torch.from_numpy(rng.standard_normal((M, L32_H), dtype=np.float32)).to(torch.bfloat16).to(dev)
        Xo = torch.from_numpy(rng.standard_normal((M, 8192), dtype=np.float32)).to(torch.bfloat16)
        Xd = torch.from_numpy(rng.standard_normal((M, 512), dtype=np.float32)).to(torch.bfloat16).repeat(1, L32_I // 512)
        Xo_d, Xd_d = Xo[:, lo_o:hi_o].contiguous().to(dev), Xd[:, lo_d:hi_d].contiguous().to(dev)
        Yq = torch.empty((M, w0["q"].n), dtype=torch.bfloat16, device=dev)
        Yk = torch.empty((M, w0["k"].n), dtype=torch.bfloat16, device=dev)
        Yv = torch.empty((M, w0["v"].n), dtype=torch.bfloat16, device=dev)
        Yg = torch.empty((M, w0["gate"].n), dtype=torch.bfloat16, device=dev)
        Yu = torch.empty((M, w0["up"].n), dtype=torch.bfloat16, device=dev)
        # row-parallel partial products are summed over the ranks in fp32: bf16 partials (2^-9 each, and
        # again at every addition of the reduction) leave the 5e-3 bound at 2 and 4 ranks
        part_dtype = torch.float32 if world > 1 else torch.bfloat16
        Yo = torch.empty((M, L32_H), dtype=part_dtype, device=dev)
        Yd = torch.empty((M, L32_H), dtype=part_dtype, device=dev)
        comm = torch.cuda.Stream(device=dev)

        def row_parallel(w, x, y):
            # partial products chunk by chunk; each chunk's sum over the ranks runs on the second stream
            # while the next chunk multiplies
            for c in range(chunks):
                be.project(w, x[c * mc:(c + 1) * mc], out=y[c * mc:(c + 1) * mc], stream=stream)
                if world > 1:
                    ev = torch.cuda.Event()
                    ev.record(stream)
                    comm.wait_event(ev)
                    be.allreduce(y[c * mc:(c + 1) * mc], stream=comm)
            if world > 1:
                ev = torch.cuda.Event()
                ev.record(comm)
                stream.wait_event(ev)

        def step_prefill():
            for s in shards:
                be.project(s["q"], X, out=Yq, stream=stream)
                be.project(s["k"], X, out=Yk, stream=stream)
                be.project(s["v"], X, out=Yv, stream=stream)
                row_parallel(s["o"], Xo_d, Yo)
                be.project(s["gate"], X, out=Yg, stream=stream)
                be.project(s["up"], X, out=Yu, stream=stream)
                row_parallel(s["down"], Xd_d, Yd)

        ms, samples = timed(step_prefill, max(3, min(args.steps, 5)), warm=2)
        torch.cuda.synchronize()
        rows = np.sort(np.random.default_rng(4).choice(L32_H, size=16, replace=False))
        wd = gq.dequantize(14, host["down"][rows], L32_I).astype(np.float64)
        ref = (Xd.float().numpy().astype(np.float64)[:256] @ wd.T)
        chk = worst(Yd[:256][:, torch.from_numpy(rows).to(dev)].float().cpu().numpy().astype(np.float64), ref, 5e-3)
        flops = layers * 2.0 * M * sum(n * k for _, _, n, k in L32)
        tpeak, tsrc = FALLBACK_TFLOPS, "fallback"
        pk = ROOT / "MEASURED_PEAKS.json"
        if pk.exists():
            try:
                tpeak, tsrc = float(json.loads(pk.read_text())["bf16_tflops"]), "measured (burst)"
            except Exception:
                pass
        result["prefill"] = {"ms_per_step": ms, "value": flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                             "roofline": {"bound": "tensor", "achieved": flops / world / (ms * 1e-3) / 1e12, "peak": tpeak,
                                          "frac": flops / world / (ms * 1e-3) / 1e12 / tpeak, "peak_source": f"of {tsrc}",
                                          "note": "per-rank 2 M N K / device time; includes activation conversions and, for N > 1, "
                                                  f"{2 * chunks} NCCL all-reduces per layer ({M * L32_H * 2} bytes per projection) on a second stream"},
                             "stats": sample_stats(samples),
                             "check": {"max_err_over_tol": chk, "ok": bool(chk <= 1.0), "what": "16 sampled rows of down, 256 tokens" + (", fp32 partials summed over the ranks" if world > 1 else "")},
                             "allreduce_bytes_per_projection": M * L32_H * 4 if world > 1 else 0, "m_chunks": chunks}
    used = clocks.summary()
    if world > 1:
        be.tp_finalize()
        dist.barrier()
    line = {"metric": "layer32b_projection_throughput", "value": result["decode"]["value"], "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": 3, "ms_per_step": result["decode"]["ms_per_step"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "decode: u8 x s16 dp4a; prefill: fp16 tcgen05.mma; fp32 accumulate", "data": "synthetic",
            "config": {"workload": "configs[4]: all projections of one decoder layer of a 32B-class dense model (Q4_K_M mix), M = 1 and M = 4096",
                       "layers_per_step": layers, "weight_bytes_per_layer": weight_bytes, "parallelism": f"tp{world}" if world > 1 else "single",
                       "l2": f"{layers} distinct copies of the layer per step ({layers * weight_bytes / world / 1e6:.0f} MB per rank)"},
            "decode": result["decode"], "prefill": result["prefill"], "clocks": used, "cpu_baseline": None, "e2e": None}
    if rank == 0 and emit:
        print(json.dumps(line))
        sys.stdout.flush()
    if dist is not None:
        sys.stdout.flush()
        os._exit(0)
    return line


# ------------------------------------------------------------------------------------------------
# library arm: the same decode projections through the GGUF mat-vec kernel of the vllm package in the
# image (its port of llama.cpp's mmvq kernel: activation re-quantized to Q8_1, integer block dots).
# Not this repository's code and not the product path: a second GPU baseline beside the CPU arm.
# ------------------------------------------------------------------------------------------------

def run_library_arm(args, emit=True):
    import torch

    rank, local_rank, world = dist_env()
    if world > 1:
        if rank == 0 and emit:
            print(json.dumps({"metric": METRIC, "impl": "library", "unavailable": "the library arm is single-GPU"}))
        return None
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device")
    try:
        from vllm import _custom_ops as ops
        ops.ggml_mul_mat_vec_a8  # noqa: B018
    except Exception as exc:
        line = {"metric": METRIC, "impl": "library", "unavailable": f"vllm GGUF ops not usable: {type(exc).__name__}: {exc}"[:300]}
        if emit:
            print(json.dumps(line))
        return line
    import magnitude_b200 as mb

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    gate_h, up_h, down_h = make_host_layer(encoder=mb.quantize)
    copies = 8          # 8 x 99 MB of packed weights: more than L2

    def dev_bytes(a):
        return torch.from_numpy(np.ascontiguousarray(a).view(np.uint8).reshape(a.shape[0], -1)).to(dev)

    layers = [(dev_bytes(gate_h), dev_bytes(up_h), dev_bytes(down_h)) for _ in range(copies)]
    rng = np.random.default_rng(1)
    x_h = torch.from_numpy(rng.standard_normal((1, HIDDEN), dtype=np.float32)).to(dev).to(torch.float16)
    x_i = torch.from_numpy(rng.standard_normal((1, INTER), dtype=np.float32)).to(dev).to(torch.float16)
    stream = torch.cuda.Stream(device=dev)

    def step():
        outs = None
        for g, u, d in layers:
            outs = (ops.ggml_mul_mat_vec_a8(g, x_h, Q4_K, INTER), ops.ggml_mul_mat_vec_a8(u, x_h, Q4_K, INTER),
                    ops.ggml_mul_mat_vec_a8(d, x_i, Q4_K, HIDDEN))
        return outs

    with torch.cuda.stream(stream):
        for _ in range(max(args.warmup, 3)):
            outs = step()
    stream.synchronize()
    # agreement with the product's own result on one projection, within the 8-bit activation's noise
    be = mb.Backend(local_rank)
    w = be.upload(Q4_K, down_h, HIDDEN, INTER)
    ours = be.project(w, x_i.float())
    be.sync()
    a, b = ours.float().cpu().numpy().reshape(-1).astype(np.float64), outs[2].float().cpu().numpy().reshape(-1).astype(np.float64)
    agree = float(np.sqrt(np.mean((a - b) ** 2)) / np.sqrt(np.mean(a * a)))
    be.close()
    graph = torch.cuda.CUDAGraph()
    try:
        with torch.cuda.graph(graph, stream=stream):
            step()
    except Exception:
        graph = None
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clocks:
        with torch.cuda.stream(stream):
            ev0.record(stream)
            for _ in range(args.steps):
                if graph is not None:
                    graph.replay()
                else:
                    step()
            ev1.record(stream)
        stream.synchronize()
    ms = ev0.elapsed_time(ev1) / args.steps
    bytes_step = copies * (2 * algorithmic_bytes(INTER, HIDDEN, x_bytes=2, y_bytes=2) + algorithmic_bytes(HIDDEN, INTER, x_bytes=2, y_bytes=2))
    peak, src = peaks()
    line = {"metric": METRIC, "impl": "library", "value": bytes_step / (ms * 1e-3) / 1e9, "unit": UNIT, "n_gpus": 1, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
            "kernel": "vllm _custom_ops.ggml_mul_mat_vec_a8 (llama.cpp mmvq port; activation re-quantized to Q8_1, fp16 in and out)",
            "config": {"workload": f"configs[1] shapes, {copies} layer copies per step (gate, up, down), one library call per projection", "cuda_graph": graph is not None},
            "frac_of_hbm_peak": bytes_step / (ms * 1e-3) / 1e9 / peak, "peak_source": f"of {src}",
            "rms_difference_to_this_library": agree, "clocks": clocks.summary()}
    # the prefill half through the package's mat-mat kernel (llama.cpp's mmq: int8 mma.sync, Q8_1 activations)
    try:
        M = 2048
        xp = torch.from_numpy(np.random.default_rng(2).standard_normal((M, HIDDEN), dtype=np.float32)).to(dev).to(torch.float16)
        with torch.cuda.stream(stream):
            for g, _, _ in layers[:3]:
                ops.ggml_mul_mat_a8(g, xp, Q4_K, INTER)
            ev0.record(stream)
            for _ in range(max(2, args.steps // 2)):
                for g, _, _ in layers:
                    ops.ggml_mul_mat_a8(g, xp, Q4_K, INTER)
            ev1.record(stream)
        stream.synchronize()
        us = ev0.elapsed_time(ev1) * 1e3 / (max(2, args.steps // 2) * copies)
        tf = 2.0 * M * INTER * HIDDEN / (us * 1e-6) / 1e12
        line["prefill"] = {"kernel": "vllm _custom_ops.ggml_mul_mat_a8 (llama.cpp mmq port), Q4_K 14336x4096 x M=2048, fp16 in and out",
                           "us_per_product": us, "value": tf, "unit": "TFLOP/s"}
    except Exception as exc:  # pragma: no cover
        line["prefill"] = {"unavailable": f"{type(exc).__name__}: {exc}"[:200]}
    if emit:
        print(json.dumps(line))
    return line


# ------------------------------------------------------------------------------------------------
# calibration rows: sustained mat-vec bytes per second and launch cost per block type
# ------------------------------------------------------------------------------------------------

def run_calibration(args, emit=True):
    """Per block type a synthetic 4096 x 4096 mat-vec (M = 1, bf16 in, fp32 out) over 24 distinct weight
    copies in one decode plan, and the cost of an (almost) empty launch: the quantities the reference's
    hardware calibration records per tensor type (icn-hardware/src/lib.rs:4043-4055;
    producer icn-server/src/main.rs:2989)."""
    import torch

    rank, local_rank, world = dist_env()
    if world > 1:
        return {"unavailable": "calibration rows are single-GPU"}
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    import magnitude_b200 as mb
    from magnitude_b200 import ggml_quant as gq

    be = mb.Backend(local_rank)
    stream = torch.cuda.Stream(device=dev)
    n = k = 4096
    copies, reps = 24, 12
    rows = []
    x = torch.randn(1, k, device=dev).to(torch.bfloat16)
    y = torch.empty((1, n), dtype=torch.float32, device=dev)
    tiny = be.upload(Q4_K, gq.synth_weights(Q4_K, 4, 256, 0), 4, 256)
    xt = torch.randn(1, 256, device=dev).to(torch.bfloat16)
    yt = torch.empty((1, 4), dtype=torch.float32, device=dev)

    def timed(fn, count):
        out = []
        for _ in range(count):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            with torch.cuda.stream(stream):
                e0.record(stream)
                fn()
                e1.record(stream)
            stream.synchronize()
            out.append(e0.elapsed_time(e1))
        return out

    for _ in range(3):
        be.project(tiny, xt, out=yt, stream=stream)
    launch_us = float(np.median(timed(lambda: be.project(tiny, xt, out=yt, stream=stream), 20))) * 1e3
    for qt, name, blk_e, blk_b in ((Q4_K, "Q4_K", 256, 144), (13, "Q5_K", 256, 176), (14, "Q6_K", 256, 210), (8, "Q8_0", 32, 34), (2, "Q4_0", 32, 18), (39, "MXFP4", 32, 17)):
        w0 = be.upload(qt, gq.synth_weights(qt, n, k, 0, encoder=mb.quantize), n, k)
        ws = [w0] + [w0.clone() for _ in range(copies - 1)]
        plan = be.plan([([w], x, [y]) for w in ws])
        for _ in range(3):
            plan.run(stream=stream)
        stream.synchronize()
        t = timed(lambda: plan.run(stream=stream), reps)
        st = sample_stats(t)
        nbytes = copies * (n * (k // blk_e) * blk_b + k * 2 + n * 4)
        rows.append(calibration_row(name, nbytes / (st["median_ms"] * 1e-3), launch_us, st["relative_spread"], reps))
        plan.close()
        del ws, w0
    be.sync(stream)
    tiny.close()
    be.close()
    line = {"metric": "hardware_calibration_rows", "rows": rows, "shape": "4096 x 4096, M = 1, 24 weight copies per run (one decode plan)",
            "launch_microseconds_definition": "device time of one call on a 4 x 256 weight"}
    if emit:
        print(json.dumps(line))
    return line


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
    ap.add_argument("--quick", action="store_true", help="headline figure only: no dependent / sustained / secondary measurements")
    ap.add_argument("--no-check", action="store_true", help="skip the host check of the step's results")
    ap.add_argument("--workload", choices=["decode", "prefill", "skinny", "calibration", "layer32b", "library"], default="decode",
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
    elif args.workload == "calibration":
        run_calibration(args)
    elif args.workload == "layer32b":
        run_layer32b(args)
    elif args.workload == "library":
        run_library_arm(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
