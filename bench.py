#!/usr/bin/env python
"""Benchmark of the hot path: the batch-split gated-MLP layer step on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (the single-GPU configuration of the fused-MLP metric): X [16384, 4096]
bf16 N(0,1), W_gate / W_up [14336, 4096], W_down [4096, 14336] bf16 N(0, 0.02),
out = (silu(X W_gate^T) * (X W_up^T)) W_down^T, executed as two micro-batches of
8192 rows. One "step" is one pass over the 16384 rows. With N > 1 the layer is
tensor-parallel (intermediate dimension sharded N ways, partial outputs reduced
across ranks, the reduction of micro-batch i overlapped with the GEMMs of i+1).

Prints ONE JSON line on rank 0. ``value`` is tokens/s with inputs resident in HBM,
``e2e`` the same metric with host buffers and the copies inside the timed region.
``--impl reference`` times the CPU restatement of the reference's operator chain
on the host cores instead (a bounded sample per step).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

H, I = 4096, 14336
ROWS = 16384
MICRO_BATCHES = 2
# dram__bytes_read.sum + dram__bytes_write.sum of one single-launch MLP (8192 rows, one GPU) from the 1-pass ncu
# capture summarised in profiles/gated_mlp_launch_list_rows16384.md; it only describes that shape
MLP_DRAM_BYTES_PER_LAUNCH = 1_633_166_336 + 296_816_640
METRIC = "prefill tokens/sec through the fused gated-MLP layer (2 micro-batches)"


def measured_peaks() -> tuple[dict, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler:
    """Samples SM clock, power and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int, period_ms: int = 50) -> None:
        self.samples: list[tuple[float, list[str]]] = []
        self._proc = None
        self._thread = None
        try:
            self._proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", str(period_ms),
                 "-i", str(gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self._thread = threading.Thread(target=self._pump, daemon=True)
            self._thread.start()
        except OSError:
            self._proc = None

    def _pump(self) -> None:
        assert self._proc is not None and self._proc.stdout is not None
        for line in self._proc.stdout:
            self.samples.append((time.time(), [c.strip() for c in line.split(",")]))

    def stop(self) -> None:
        if self._proc is not None:
            self._proc.terminate()
            try:
                self._proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self._proc.kill()

    def summary(self, t0: float, t1: float) -> dict:
        rows = [c for t, c in self.samples if t0 <= t <= t1 and len(c) >= 7]
        window = "timed region"
        if not rows:
            rows = [c for _, c in self.samples if len(c) >= 7]
            window = "whole run (timed region shorter than the sampling period)"
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0, "window": "nvidia-smi unavailable"}
        mhz = [float(c[0]) for c in rows if c[0].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(c[3 + i].lower().startswith("active") for c in rows)]
        power = [float(c[2]) for c in rows if c[2].replace(".", "").isdigit()]
        return {"sm_mhz": statistics.median(mhz) if mhz else None, "sm_max_mhz": float(rows[0][1]),
                "power_w_max": max(power) if power else None, "reasons": reasons, "samples": len(rows),
                "window": window}


# ------------------------------------------------------------------ CPU arm
def cpu_port_sample(target_seconds: float = 12.0, rows: int = 2048) -> tuple[float, float, int]:
    """Times the oracle's gated MLP (the reference's operator chain restated on PyTorch CPU ops,
    bf16, all host threads): passes over the same ``rows`` rows of the workload, after one untimed
    pass, until ``target_seconds`` of CPU work are done. Returns (tokens/s, seconds, passes)."""
    import torch

    from oracle import ops_oracle

    wg, wu, wd = cpu_weights()
    x = torch.randn(rows, H, generator=torch.Generator().manual_seed(1)).bfloat16()
    passes = 0
    with torch.inference_mode():
        ops_oracle.gated_mlp(x, wg, wu, wd)
        t0 = time.perf_counter()
        while True:
            ops_oracle.gated_mlp(x, wg, wu, wd)
            passes += 1
            elapsed = time.perf_counter() - t0
            if elapsed >= target_seconds or passes >= 10000:
                break
    return rows * passes / elapsed, elapsed, passes


def cpu_weights():
    import torch

    g = torch.Generator().manual_seed(0)
    wg = (torch.randn(I, H, generator=g) * 0.02).bfloat16()
    wu = (torch.randn(I, H, generator=g) * 0.02).bfloat16()
    wd = (torch.randn(H, I, generator=g) * 0.02).bfloat16()
    return wg, wu, wd


def run_reference_arm(args) -> None:
    """CPU implementation of the path on the host cores, all threads, bounded sample per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch

    from oracle import ops_oracle

    cores = torch.get_num_threads()
    wg, wu, wd = cpu_weights()
    g = torch.Generator().manual_seed(1)
    probe = torch.randn(16, H, generator=g).bfloat16()
    with torch.inference_mode():
        ops_oracle.gated_mlp(probe, wg, wu, wd)
        t0 = time.perf_counter()
        ops_oracle.gated_mlp(probe, wg, wu, wd)
        per_row = (time.perf_counter() - t0) / 16
    budget = min(2.0, 150.0 / max(1, args.steps + args.warmup))
    rows = int(max(16, min(ROWS, budget / per_row)) // 16 * 16)
    x = torch.randn(rows, H, generator=g).bfloat16()
    with torch.inference_mode():
        for _ in range(args.warmup):
            ops_oracle.gated_mlp(x, wg, wu, wd)
        t0 = time.perf_counter()
        for _ in range(args.steps):
            ops_oracle.gated_mlp(x, wg, wu, wd)
        dt = time.perf_counter() - t0
    value = rows * args.steps / dt
    sample = f"{rows} of {ROWS} rows per step, {args.steps} steps, bf16, torch CPU"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(args.gpus),
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def workload_config(n_gpus: int) -> dict:
    return {"workload": f"fused gated MLP, X[{ROWS},{H}] bf16, W_gate/W_up[{I},{H}], W_down[{H},{I}], "
                        f"{MICRO_BATCHES} micro-batches of {ROWS // MICRO_BATCHES} rows",
            "rows": ROWS, "hidden": H, "intermediate": I, "micro_batches": MICRO_BATCHES,
            "parallelism": f"tp{n_gpus}", "l2": "inputs larger than L2 (weights 352 MB + activations 604 MB per step)"}


def comm_plan(args, world: int, sms: int | None = None, multicast: bool | None = None) -> dict:
    """How the reduction and the GEMMs share the GPU at N > 1 (flags override the defaults): the
    reduction inside the NVLink switch on 16 CTAs, on 8 SMs that the GEMMs leave free.
    ``sms`` / ``multicast`` default to what the current device reports."""
    if world == 1:
        return {"comm": None, "comm_ctas": 0, "gemm_ctas": 0, "exclusive_sms": False}
    kind = args.comm
    if kind == "auto":
        if multicast is None:
            from dynaflow_b200.comm import multicast_supported

            multicast = multicast_supported()
        kind = "multicast" if multicast else "peer"
    comm_ctas = args.comm_ctas if args.comm_ctas > 0 else (16 if kind == "multicast" else 32)
    exclusive = not args.shared_sms
    if sms is None:
        import torch

        sms = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    gemm_ctas = args.gemm_ctas if args.gemm_ctas >= 0 else (sms - (comm_ctas + 1) // 2 if exclusive else 0)
    return {"comm": kind, "comm_ctas": comm_ctas, "gemm_ctas": gemm_ctas, "exclusive_sms": exclusive}


# ------------------------------------------------------------------ GPU arm
def run_ours(args) -> None:
    import torch
    import torch.distributed as dist

    from dynaflow_b200 import ops
    from dynaflow_b200.layer import TensorParallelGatedMLP

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    comm = None
    plan = comm_plan(args, world)
    if world > 1:
        from dynaflow_b200.comm import MulticastComm, PeerComm, set_exclusive_sms

        if plan["comm"] == "multicast":
            try:
                comm = MulticastComm(rank, world, ROWS // MICRO_BATCHES, H, slots=MICRO_BATCHES,
                                     n_ctas=plan["comm_ctas"], device=dev)
            except Exception as exc:  # noqa: BLE001 -- e.g. a driver without fabric support: same answer on every rank
                if args.comm == "multicast":
                    raise
                print(f"[bench] no multicast mapping ({exc}); using the peer-memory reduction", file=sys.stderr)
                args.comm = "peer"
                plan = comm_plan(args, world)
        if comm is None:
            comm = PeerComm(rank, world, ROWS // MICRO_BATCHES, H, slots=MICRO_BATCHES, n_ctas=plan["comm_ctas"], device=dev)
        set_exclusive_sms(plan["exclusive_sms"])
    layer = TensorParallelGatedMLP(H, I, rank=rank, world=world, max_rows=ROWS // MICRO_BATCHES,
                                   micro_batches=MICRO_BATCHES, seed=0, device=dev, comm=comm)
    layer.gemm_max_ctas = plan["gemm_ctas"]
    gen = torch.Generator().manual_seed(1)
    x_host = torch.randn(ROWS, H, generator=gen).bfloat16().pin_memory()
    out_host = torch.empty(ROWS, H, dtype=torch.bfloat16).pin_memory()
    x_dev = x_host.to(dev)
    out_dev = torch.empty(ROWS, H, dtype=torch.bfloat16, device=dev)
    cuts = [ROWS * i // MICRO_BATCHES for i in range(MICRO_BATCHES + 1)]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    sampler = ClockSampler(local_rank) if rank == 0 else None

    # ---- device-resident: value, and per-kernel times for the roofline
    # Consecutive steps pipeline like consecutive layers: the reduction of a step's last micro-batch
    # runs under the next step's first GEMMs; the stream joins the reductions before the end mark.
    for _ in range(args.warmup):
        layer.forward_device(x_dev, out_dev, cuts, join=False)
    layer.wait_reductions()
    barrier()
    marks = []
    t_wall0 = time.time()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(args.steps):
        marks.append(layer.forward_device(x_dev, out_dev, cuts, record_kernel_events=True, join=False))
    layer.wait_reductions()
    end.record()
    barrier()
    t_wall1 = time.time()
    ms_step = max_over_ranks(start.elapsed_time(end) / args.steps)
    mlp_ms = statistics.mean(m0.elapsed_time(m1) for step in marks for (m0, m1) in step)
    ops.check_status()
    # the same MLP as two launches, a few steps outside the timed region: how the time splits between the GEMMs
    for _ in range(2):
        layer.forward_device(x_dev, out_dev, cuts, record_kernel_events="split")
    split = [layer.forward_device(x_dev, out_dev, cuts, record_kernel_events="split") for _ in range(max(3, args.steps // 10))]
    barrier()
    gateup_ms = statistics.median(m0.elapsed_time(m1) for step in split for (m0, m1, _m2) in step)
    down_ms = statistics.median(m1.elapsed_time(m2) for step in split for (_m0, m1, m2) in step)
    ops.check_status()

    # ---- N > 1: how much of the reduction hides under the other micro-batch's GEMMs
    comm_stats = None
    if world > 1:
        chain_layers = 8
        norm_w = torch.ones(H, dtype=torch.bfloat16, device=dev)
        residual = torch.zeros(ROWS, H, dtype=torch.bfloat16, device=dev)

        def timed(**kw):
            for _ in range(2):
                residual.zero_()
                layer.forward_chain(x_dev, cuts, chain_layers, norm_w, residual, fused_norm=args.fused_norm, sharded_residual=not args.replicated_residual, **kw)
            barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            reps = max(4, args.steps // 16)
            a.record()
            for _ in range(reps):
                layer.forward_chain(x_dev, cuts, chain_layers, norm_w, residual, fused_norm=args.fused_norm, sharded_residual=not args.replicated_residual, **kw)
            b.record()
            barrier()
            return max_over_ranks(a.elapsed_time(b) / reps / chain_layers)

        t_overlap = timed()
        t_compute = timed(skip_comm=True)
        t_comm = timed(skip_compute=True)
        payload = ROWS * H * 2  # bytes reduced per block (all micro-batches)
        wire = 2.0 * (world - 1) / world * payload
        peak_tf = float(measured_peaks()[0]["bf16_tflops"])
        comm_stats = {"chain": f"{chain_layers} TP MLP blocks back to back; between them all-reduce + residual + RMSNorm: "
                               + ("reduce-scatter, add + norm on the owned rows (residual sharded by rows), all-gather, one launch"
                                  if not args.replicated_residual else
                                  ("replicated residual, one launch" if args.fused_norm
                                   else "replicated residual, reduction on few CTAs then normalisation over all SMs")),
                      "ms_per_block_overlapped": t_overlap, "ms_per_block_compute_only": t_compute,
                      "ms_per_block_comm_only": t_comm,
                      "hidden_frac": 1.0 - (t_overlap - t_compute) / t_comm,
                      "bus_gbs_comm_only": wire / (t_comm * 1e-3) / 1e9,
                      "nvlink_peak_gbs": 770.0, "nvlink_peak_source": "measured peer copy, per direction",
                      "roofline_ms_per_block": max(6.0 * ROWS * H * (I // world) / (peak_tf * 1e12),
                                                   (world - 1) / world * payload / 770e9) * 1e3,
                      "tokens_per_s_chain": ROWS / (t_overlap * 1e-3)}
        comm_stats["frac_of_roofline_chain"] = comm_stats["roofline_ms_per_block"] / t_overlap
        ops.check_status()

    # ---- end to end: pinned host buffers, copies inside the timed region
    for _ in range(args.warmup):
        layer.forward_host(x_host, out_host, cuts)
    barrier()
    s2, e2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s2.record()
    for _ in range(args.steps):
        layer.forward_host(x_host, out_host, cuts)
    e2.record()
    barrier()
    e2e_ms = max_over_ranks(s2.elapsed_time(e2) / args.steps)
    ops.check_status()
    if sampler is not None:
        sampler.stop()

    comm_summary = layer.comm_summary()
    if world > 1:
        # every rank leaves together: the regions are unmapped only once nobody can touch them any more
        barrier()
        comm.close()
        dist.barrier()
        dist.destroy_process_group()
    if rank != 0:
        return

    peaks, peak_kind = measured_peaks()
    rows_mb = ROWS // MICRO_BATCHES
    mlp_flops = 6.0 * rows_mb * H * (I // world)          # one launch: gate/up 4 M H I + down 2 M H I
    achieved = mlp_flops / (mlp_ms * 1e-3) / 1e12
    # denominator: the measured cuBLAS burst figure; the kernel is timed inside the long, power-capped step, so the
    # fraction of the measured SUSTAINED figure is printed beside it
    burst = float(peaks["bf16_tflops"])
    peak = burst
    sustained = float(peaks.get("bf16_tflops_sustained", burst))
    step_flops = 6.0 * ROWS * H * (I // world)
    traffic = MLP_DRAM_BYTES_PER_LAUNCH if (ROWS == 16384 and world == 1) else None

    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        rate, secs, passes = cpu_port_sample(12.0, 2048)
        import torch as _t

        cpu = {"value": rate, "unit": "tokens/s", "cores": _t.get_num_threads(), "kind": "port",
               "sample": f"2048 of {ROWS} rows, {passes} passes of the oracle's gated MLP in {secs:.1f} s (bf16, torch CPU)"}

    sweep = None
    if world == 1 and not args.no_sweep:
        sweep = m_sweep(layer, dev, peaks)

    line = {
        "metric": METRIC, "value": ROWS / (ms_step * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": dict(workload_config(world), **({"reduction": plan} if world > 1 else {})),
        "e2e": {"value": ROWS / (e2e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": ROWS * H * 2, "d2h_bytes_per_step": ROWS * H * 2},
        "gpu_launches": layer.launches_per_step * args.steps,
        "roofline": {"bound": "tensor",
                     "kernel": "gemm_tc_kernel<FUSED> (gate/up GEMM + SiLU*mul epilogue + down GEMM, one persistent launch)",
                     "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                     "peak_source": f"{peak_kind} cuBLAS bf16 burst", "frac_of_sustained": achieved / sustained,
                     "sustained_peak": sustained,
                     "frac_of_nominal_2250": achieved / 2250.0, "traffic": traffic,
                     "flops_per_launch": mlp_flops, "ms_per_launch": mlp_ms,
                     "as_two_launches": {"gateup_ms": gateup_ms, "down_ms": down_ms,
                                         "gateup_tflops": 4.0 * rows_mb * H * (I // world) / (gateup_ms * 1e-3) / 1e12,
                                         "down_tflops": 2.0 * rows_mb * H * (I // world) / (down_ms * 1e-3) / 1e12}},
        "mlp_pct_tensor_peak": 100.0 * step_flops / (ms_step * 1e-3) / 1e12 / burst,
        "clocks": sampler.summary(t_wall0, t_wall1) if sampler is not None else None,
        "cpu_baseline": cpu,
        "sweep": sweep,
    }
    if world > 1:
        line["comm"] = dict(comm_summary, **(comm_stats or {}))
    print(json.dumps(line))


def m_sweep(layer, dev, peaks) -> list[dict]:
    """The M sweep of the fused-MLP configuration: two micro-batches of M/2 rows, serial (one
    stream) and overlapped (one stream per micro-batch), against max(flops / tensor peak,
    bytes / HBM peak)."""
    import torch

    from dynaflow_b200 import ops

    out = []
    streams = layer.streams
    for rows in (16, 256, 2048, 8192, 16384):
        half = rows // 2
        x = torch.randn(rows, H, device=dev).bfloat16()
        y = torch.empty(rows, H, dtype=torch.bfloat16, device=dev)
        hs = [layer.h_views[i][:half] for i in range(2)]

        def serial():
            for i in range(2):
                ops.gated_mlp(x[i * half:(i + 1) * half], layer.w_gate, layer.w_up, layer.w_down,
                              out=y[i * half:(i + 1) * half], workspace=layer.workspaces[i])

        def overlapped():
            main = torch.cuda.current_stream()
            fork = torch.cuda.Event()
            fork.record(main)
            for i in range(2):
                streams[i].wait_event(fork)
                with torch.cuda.stream(streams[i]):
                    ops.gated_mlp(x[i * half:(i + 1) * half], layer.w_gate, layer.w_up, layer.w_down,
                                  out=y[i * half:(i + 1) * half], workspace=layer.workspaces[i])
                main.wait_stream(streams[i])

        def time_it(fn):
            for _ in range(5):
                fn()
            torch.cuda.synchronize()
            n = 200 if rows <= 2048 else 40
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(n):
                fn()
            b.record()
            torch.cuda.synchronize()
            return a.elapsed_time(b) / n

        t_serial, t_overlap = time_it(serial), time_it(overlapped)
        flops = 6.0 * rows * H * I
        bytes_min = 3.0 * H * I * 2 + 2.0 * rows * H * 2
        bound_ms = max(flops / (float(peaks["bf16_tflops"]) * 1e12), bytes_min / (float(peaks["hbm_gbs"]) * 1e9)) * 1e3
        out.append({"rows": rows, "ms_serial": t_serial, "ms_overlapped": t_overlap, "tflops_serial": flops / t_serial / 1e9,
                    "roofline_ms": bound_ms, "frac_of_roofline": bound_ms / min(t_serial, t_overlap),
                    "bound": "tensor" if flops / (float(peaks["bf16_tflops"]) * 1e12) > bytes_min / (float(peaks["hbm_gbs"]) * 1e9) else "hbm"})
        del hs
    ops.check_status()
    return out


def run_decoder(args) -> None:
    """Second workload (not the default line): Llama-3-8B-shaped decoder prefill, 8 x 2048 ids, two
    micro-batches, tensor parallel over the launched ranks. value = tokens/s of the whole stack."""
    import torch
    import torch.distributed as dist

    from dynaflow_b200 import ops
    from dynaflow_b200.decoder import DecoderShape, TensorParallelDecoder

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    shape = DecoderShape(layers=args.layers)
    batch, seq = 8, 2048
    plan = comm_plan(args, world)
    if world > 1:
        from dynaflow_b200.comm import set_exclusive_sms

        set_exclusive_sms(plan["exclusive_sms"])
    def build_decoder(p):
        return TensorParallelDecoder(shape, rank=rank, world=world, max_rows=batch * seq // MICRO_BATCHES,
                                     micro_batches=MICRO_BATCHES, seed=0, device=dev, n_ctas=p["comm_ctas"],
                                     multicast=p["comm"] == "multicast", gemm_max_ctas=p["gemm_ctas"])

    try:
        dec = build_decoder(plan)
    except Exception as exc:  # noqa: BLE001 -- no multicast mapping: the peer-memory reduction instead
        if plan["comm"] != "multicast" or args.comm == "multicast":
            raise
        print(f"[bench] no multicast mapping ({exc}); using the peer-memory reduction", file=sys.stderr)
        args.comm = "peer"
        plan = comm_plan(args, world)
        dec = build_decoder(plan)
    ids = torch.randint(0, shape.vocab, (batch, seq), generator=torch.Generator().manual_seed(1)).to(dev)

    def timed(**kw):
        for _ in range(max(2, args.warmup // 2)):
            dec.forward(ids, **kw)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = max(3, args.steps // 20)
        a.record()
        for _ in range(reps):
            dec.forward(ids, **kw)
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / reps
        if world > 1:
            t = torch.tensor([ms], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    t_all = timed()
    ops.check_status()
    line = {"workload": f"Llama-3-8B-shaped decoder prefill, {shape.layers} layers, ids {batch}x{seq}, "
                        f"{MICRO_BATCHES} micro-batches, tp{world}",
            "metric": "prefill tokens/sec", "unit": "tokens/s", "n_gpus": world, "ms_per_forward": t_all, "reduction": plan,
            "value": batch * seq / (t_all * 1e-3)}
    peaks, kind = measured_peaks()
    s = shape
    linear = 2.0 * (s.hidden * (s.heads + 2 * s.kv_heads) * s.head_dim + s.heads * s.head_dim * s.hidden
                    + 3 * s.hidden * s.intermediate)
    attn = 4.0 * ((seq + 1) / 2) * s.heads * s.head_dim
    flops = (linear + attn) * s.layers * batch * seq
    line["flops_per_forward"] = flops
    line["tflops_per_gpu"] = flops / world / (t_all * 1e-3) / 1e12
    line["frac_of_tensor_peak"] = line["tflops_per_gpu"] / float(peaks["bf16_tflops"])
    line["peak_source"] = f"{kind} cuBLAS bf16 burst"
    if world > 1:
        t_compute = timed(skip_comm=True)
        t_comm = timed(skip_compute=True)
        payload = 2 * s.layers * batch * seq * s.hidden * 2
        line["comm"] = {"ms_overlapped": t_all, "ms_compute_only": t_compute, "ms_comm_only": t_comm,
                        "hidden_frac": 1.0 - (t_all - t_compute) / t_comm,
                        "wire_ms_at_770": (world - 1) / world * payload / 770e9 * 1e3,
                        "roofline_ms": max(flops / world / (float(peaks["bf16_tflops"]) * 1e12),
                                           (world - 1) / world * payload / 770e9) * 1e3}
        line["frac_of_roofline"] = line["comm"]["roofline_ms"] / t_all
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
    dec.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_moe(args) -> None:
    """Third workload (not the default line): Mixtral-shaped top-2 MoE stack, 16384 tokens per step, 8 experts of
    intermediate 14336, expert parallel over the launched ranks (one rank: all experts local).
    value = tokens/s through `--moe-layers` layers (dispatch / expert / combine each)."""
    import torch
    import torch.distributed as dist

    from dynaflow_b200 import ops
    from dynaflow_b200.moe import ExpertParallelMoE

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    experts, tokens, layers = 8, ROWS, args.moe_layers
    per_rank = tokens // world
    gen = torch.Generator(device=dev).manual_seed(7)      # same weights on every rank; each keeps its experts

    def weight(*shape):
        return (torch.randn(*shape, device=dev, generator=gen) * 0.02).bfloat16()

    stack = []
    for _ in range(layers):
        w = (weight(experts, I, H), weight(experts, I, H), weight(experts, H, I))
        stack.append(ExpertParallelMoE(H, I, experts, per_rank, rank=rank, world=world, weights=w, slots=1,
                                       n_ctas=args.comm_ctas or 32, device=dev))
        del w
    x = torch.randn(per_rank, H, device=dev, generator=gen).bfloat16()
    logits = [torch.randn(per_rank, experts, device=dev, generator=gen).bfloat16() for _ in range(layers)]

    def step():
        for layer, lg in zip(stack, logits):      # every layer routes the same rows with its own router logits
            layer.forward(x, lg)

    for _ in range(max(3, args.warmup)):
        step()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = max(3, args.steps // 10)
    a.record()
    for _ in range(reps):
        step()
    b.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b) / reps
    if world > 1:
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ops.check_status()
    peaks, kind = measured_peaks()
    flops = 2.0 * tokens * 6.0 * H * I * layers               # two experts per token
    line = {"workload": f"Mixtral-shaped top-2 MoE, {layers} layers, {experts} experts x {I}, {tokens} tokens per step, ep{world}",
            "metric": "tokens/sec", "unit": "tokens/s", "n_gpus": world, "ms_per_step": ms, "value": tokens / (ms * 1e-3),
            "flops_per_step": flops, "tflops_per_gpu": flops / world / (ms * 1e-3) / 1e12,
            "frac_of_tensor_peak": flops / world / (ms * 1e-3) / 1e12 / float(peaks["bf16_tflops"]),
            "peak_source": f"{kind} cuBLAS bf16 burst", "steps": reps, "data": "synthetic"}
    # load balance of the first layer's routing (ids of all tokens, two experts each)
    counts = torch.bincount(stack[0].ids[0].flatten().to(torch.int64), minlength=experts).double()
    line["tokens_per_expert_max_over_mean"] = float((counts.max() / counts.mean()).item())
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
    for layer in stack:
        layer.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main() -> None:
    global ROWS
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--rows", type=int, default=ROWS, help="rows per step (default: the benchmark's 16384; "
                    "smaller values are for profiler captures only)")
    ap.add_argument("--comm", choices=["auto", "multicast", "peer"], default="auto",
                    help="N > 1: reduction inside the NVLink switch (multimem kernel) or over peer memory (two-shot "
                         "kernel); auto = multicast where the devices offer it")
    ap.add_argument("--comm-ctas", type=int, default=0, help="CTAs of the reduction kernel (N > 1; 0 = 16 for multicast, "
                    "32 for peer)")
    ap.add_argument("--gemm-ctas", type=int, default=-1, help="CTAs the GEMMs may use at N > 1 (0 = one per SM; default: "
                    "the SMs minus the ones the reduction's CTAs fill, two per SM)")
    ap.add_argument("--shared-sms", action="store_true", help="N > 1: let reduction CTAs share SMs with GEMM CTAs instead "
                    "of running on SMs of their own")
    ap.add_argument("--replicated-residual", action="store_true",
                    help="N > 1 chain: keep the residual stream replicated on every rank instead of sharded by rows")
    ap.add_argument("--moe-layers", type=int, default=4, help="moe workload: number of layers")
    ap.add_argument("--workload", choices=["mlp", "decoder", "moe"], default="mlp",
                    help="mlp: the fused gated-MLP layer step (the benchmark line); decoder: a Llama-3-8B-shaped "
                         "decoder prefill on the same kernels (reported separately)")
    ap.add_argument("--layers", type=int, default=32, help="decoder workload: number of layers")
    ap.add_argument("--fused-norm", action="store_true", help="N > 1 chain: one-launch all-reduce+RMSNorm kernel")
    ap.add_argument("--no-sweep", action="store_true", help="skip the M sweep (profiling runs)")
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU baseline leg (profiling runs)")
    args = ap.parse_args()
    if args.rows != ROWS:
        if args.rows <= 0 or args.rows % (MICRO_BATCHES * 8) != 0:
            raise SystemExit("--rows must be a positive multiple of 16")
        ROWS = args.rows
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference_arm(args)
    elif args.workload == "decoder":
        run_decoder(args)
    elif args.workload == "moe":
        run_moe(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
