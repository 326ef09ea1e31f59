#!/usr/bin/env python
"""Benchmark of the hot path: the batch-split gated-MLP layer step on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (the single-GPU configuration of the fused-MLP metric): X [16384, 4096]
bf16 N(0,1), W_gate / W_up [14336, 4096], W_down [4096, 14336] bf16 N(0, 0.02),
out = (silu(X W_gate^T) * (X W_up^T)) W_down^T, executed as two micro-batches of
8192 rows. One "step" is one pass over the 16384 rows. With N > 1 the layer is
tensor-parallel (intermediate dimension sharded N ways) and a step is one block of a
DEPENDENT chain, the way a decoder stacks them: x <- rmsnorm(allreduce(mlp(x)) + residual),
the reduction of micro-batch i under the GEMMs of micro-batch i+1.

Prints ONE JSON line on rank 0. ``value`` is tokens/s with inputs resident in HBM,
``e2e`` the same metric with host buffers and the copies inside the timed region,
``parity`` the result check made before the timed region (sampled rows against the
CPU oracle; at N > 1 also that every rank holds identical bits), ``decoder`` the
Llama-3-8B-shaped prefill (32 layers, ids 8 x 2048, two micro-batches) on the same
kernels with the fraction of communication hidden, ``torch_chain`` the operator chain
the reference's host model runs on the GPU (cuBLAS linear, silu * mul, cuBLAS linear)
timed beside the fused kernel. ``--impl reference`` times the reference package itself
on the host cores (a bounded sample per step).
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
import traceback

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

H, I = 4096, 14336
ROWS = 16384
MICRO_BATCHES = 2
# dram__bytes_read.sum + dram__bytes_write.sum of one single-launch MLP of 8192 rows on one GPU (one-pass ncu
# capture of this script); it only describes that shape
MLP_DRAM_BYTES_PER_LAUNCH = 1_633_166_336 + 296_816_640
METRIC = "prefill tokens/sec through the fused gated-MLP layer (2 micro-batches)"
TOL = 2e-2


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
def host_threads() -> int:
    """All host cores, whatever OMP_NUM_THREADS the launcher exported (torch.distributed.run sets 1)."""
    import torch

    n = os.cpu_count() or 1
    try:
        n = len(os.sched_getaffinity(0)) or n
    except (AttributeError, OSError):
        pass
    torch.set_num_threads(n)
    return torch.get_num_threads()


def cpu_weights():
    import torch

    g = torch.Generator().manual_seed(0)
    wg = (torch.randn(I, H, generator=g) * 0.02).bfloat16()
    wu = (torch.randn(I, H, generator=g) * 0.02).bfloat16()
    wd = (torch.randn(H, I, generator=g) * 0.02).bfloat16()
    return wg, wu, wd


def cpu_sample(target_seconds: float = 12.0, rows: int = 2048) -> dict:
    """The CPU baseline leg: the reference package itself (when installed under baseline/_ref; else
    the oracle's restatement of its operator chain) on all host threads, bf16: passes over the same
    ``rows`` rows of the workload, after one untimed pass, until ``target_seconds`` of CPU work
    are done."""
    import torch

    from oracle import ops_oracle

    cores = host_threads()
    step, how = reference_package_step()
    kind = "reference"
    if step is None:
        wg, wu, wd = cpu_weights()
        kind = "port"

        def step(x):
            with torch.inference_mode():
                return ops_oracle.gated_mlp(x, wg, wu, wd)

    x = torch.randn(rows, H, generator=torch.Generator().manual_seed(1)).bfloat16()
    passes = 0
    step(x)
    t0 = time.perf_counter()
    while True:
        step(x)
        passes += 1
        elapsed = time.perf_counter() - t0
        if elapsed >= target_seconds or passes >= 10000:
            break
    return {"value": rows * passes / elapsed, "unit": "tokens/s", "cores": cores, "kind": kind,
            "sample": f"{rows} of {ROWS} rows in two nano-batches, {passes} passes in {elapsed:.1f} s (bf16, torch CPU); {how}"}


def reference_package_step():
    """The reference package (installed unmodified under baseline/_ref) running the gated-MLP graph on
    the CPU in two nano-batches through its own manager, engine and executor; the policy is the
    round-robin schedule its examples use, written here against its public interface (its example
    policies are not part of the installed package). Returns ``(step(x) -> out, description)`` or
    ``(None, why)``."""
    import torch

    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "dynaflow")):
        return None, "baseline/_ref holds no installed reference package"
    sys.path.insert(0, ref_dir)
    try:
        import dynaflow.config as rcfg
        import dynaflow.interface as riface
        import dynaflow.manager as rmanager
        import dynaflow.matching as rmatching
    except Exception as exc:  # noqa: BLE001
        return None, f"the reference package does not import: {exc}"
    if not torch.cuda.is_available():
        # the reference's engine records CUDA events around every operator; without a driver they are inert
        import contextlib

        class _Inert:
            def __init__(self, *a, **k):
                pass

            def record(self, *a, **k):
                pass

            def wait(self, *a, **k):
                pass

            def synchronize(self):
                pass

        torch.cuda.Event = _Inert  # type: ignore[misc]
        torch.cuda.Stream = _Inert  # type: ignore[misc]
        torch.cuda.stream = lambda s: contextlib.nullcontext()  # type: ignore[assignment]

    class RoundRobin(riface.OpSchedulerBase):
        def __init__(self):
            super().__init__(policy_name="round-robin")

        def get_split_rules(self):
            return [rmatching.MatchingRule(condition=rmatching.Op(pattern=r"silu"))]

        def get_tag_rules(self):
            return {rmatching.MatchingRule(condition=rmatching.Op(pattern=r"silu")): {"act"}}

        def get_split_config(self, input_info, use_cudagraph):
            raise NotImplementedError("the bench overrides the split")

        async def schedule(self, context):
            live = list(range(context.split_config.num_nano_batches))
            while live:
                ops = []
                for b in list(live):
                    op = await context.pop(b)
                    if op is None:
                        live.remove(b)
                    else:
                        ops.append(op)
                for op in ops:
                    await context.execute((op,))

    class GatedMLP(torch.nn.Module):
        def __init__(self):
            super().__init__()
            wg, wu, wd = cpu_weights()
            self.gate_proj = torch.nn.Linear(H, I, bias=False, dtype=torch.bfloat16)
            self.up_proj = torch.nn.Linear(H, I, bias=False, dtype=torch.bfloat16)
            self.down_proj = torch.nn.Linear(I, H, bias=False, dtype=torch.bfloat16)
            with torch.no_grad():
                self.gate_proj.weight.copy_(wg)
                self.up_proj.weight.copy_(wu)
                self.down_proj.weight.copy_(wd)

        def forward(self, x):
            return self.down_proj(torch.nn.functional.silu(self.gate_proj(x)) * self.up_proj(x))

    cfg = rcfg.DynaFlowConfig("bench:RoundRobin", 2, rcfg.InductorConfig(False), rcfg.CUDAGraphConfig(False, [64]), {})
    manager = rmanager.DynaFlowManager()
    policy = RoundRobin()

    def backend(gm, example_inputs):
        manager.initialize(graph_module=gm, config=cfg, scheduler=policy, example_inputs=list(example_inputs))
        return manager.get_callable()

    model = GatedMLP().eval()
    torch._dynamo.reset()
    compiled = torch.compile(model, backend=backend, fullgraph=True)

    def step(x):
        import contextlib
        import io

        rows = x.shape[0]
        half = rows // 2
        torch._dynamo.mark_dynamic(x, 0)
        manager.override_split_config(riface.SplitConfig(
            num_nano_batches=2, batch_sizes=[half, rows - half], batch_indices=[0, half, rows],
            num_tokens=[half, rows - half], num_tokens_padded=[half, rows - half], split_indices=[0, half, rows],
            is_dryrun=False, use_cudagraph=False))
        with torch.inference_mode(), contextlib.redirect_stdout(io.StringIO()):
            return compiled(x)

    return step, "reference package (baseline/_ref, unmodified): DynaFlowManager + engine on the gated-MLP graph, 2 nano-batches"


def run_reference_arm(args) -> None:
    """The reference's CPU implementation of the path on the host cores, all threads, a bounded
    sample of the workload per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch

    from oracle import ops_oracle

    cores = host_threads()
    step, how = reference_package_step()
    kind = "reference"
    if step is None:
        # no installed reference package: the oracle's restatement of its operator chain
        wg, wu, wd = cpu_weights()
        kind, how = "port", f"oracle port ({how})"

        def step(x):
            with torch.inference_mode():
                return ops_oracle.gated_mlp(x, wg, wu, wd)

    g = torch.Generator().manual_seed(1)
    probe = torch.randn(64, H, generator=g).bfloat16()
    step(probe)                                   # traces / initialises
    t0 = time.perf_counter()
    step(probe)
    per_row = (time.perf_counter() - t0) / 64
    budget = min(2.0, 150.0 / max(1, args.steps + args.warmup))
    rows = int(max(64, min(ROWS, budget / per_row)) // 16 * 16)
    x = torch.randn(rows, H, generator=g).bfloat16()
    for _ in range(max(1, args.warmup)):
        out = step(x)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        out = step(x)
    dt = time.perf_counter() - t0
    # the arm's own result check: sampled rows against the oracle
    pick = torch.arange(0, rows, max(1, rows // 8))[:8]
    wg, wu, wd = cpu_weights()
    want = ops_oracle.gated_mlp_hf(x[pick], wg, wu, wd)
    rel = ((out[pick].float() - want.float()).abs().max() / want.float().abs().max()).item()
    value = rows * args.steps / dt
    sample = f"{rows} of {ROWS} rows per step (two nano-batches of {rows // 2}), {args.steps} steps, bf16, torch CPU, {cores} threads"
    config = dict(workload_config(args.gpus), sample=sample)
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": config, "how": how,
        "parity": {"checked": True, "max_rel_err": rel, "against": "oracle (operator-chain form), 8 sampled rows"},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": kind, "sample": sample},
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


# ---------------------------------------------------------- rank coordination
class PeerFailed(RuntimeError):
    """Another rank reported a failure at a synchronisation point."""


class RankSync:
    """Every host-side collective of the run after the communicators exist has ONE shape (an
    all-reduce MAX over five doubles: four values and a failure flag), so that a rank that fails
    can still pair with whatever synchronisation its peers reach next, tell them, and all ranks
    unmap their communicators together (a rank that exits while its memory is bound to an NVLink
    multicast object can fault its peers' GPUs)."""

    def __init__(self, world: int, device) -> None:
        self.world, self.device = world, device

    def reduce_max(self, values: list[float], fail: bool = False, quiet: bool = False) -> list[float]:
        if self.world == 1:
            return list(values)
        import torch
        import torch.distributed as dist

        padded = list(values) + [float("-inf")] * (4 - len(values)) + [1.0 if fail else 0.0]
        t = torch.tensor(padded, dtype=torch.float64, device=self.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        out = t.tolist()
        if out[4] > 0 and not fail and not quiet:
            raise PeerFailed("another rank failed")
        return out[:len(values)]

    def barrier(self) -> None:
        import torch

        if torch.cuda.is_available():
            torch.cuda.synchronize()
        self.reduce_max([0.0])

    def max_ms(self, ms: float) -> float:
        return self.reduce_max([ms])[0]

    def all_equal(self, digest: float) -> bool:
        hi, neg_lo = self.reduce_max([digest, -digest])
        return hi == -neg_lo


def leave_together(sync: RankSync, closers: list, error: str | None, learned: bool) -> str | None:
    """Every rank leaves together, whatever happened: tell the others (unless this rank learned of a
    failure at a synchronisation point, which consumed that exchange), stop launching, meet, unmap the
    communicators, meet again. Returns the error to exit with (its own, or that a peer failed)."""
    import torch

    if sync.world > 1:
        if not learned:
            try:
                sync.reduce_max([0.0], fail=error is not None)
            except PeerFailed as exc:
                error = error or str(exc)
        if torch.cuda.is_available():
            try:
                torch.cuda.synchronize()
            except Exception:  # noqa: BLE001
                traceback.print_exc()
        sync.reduce_max([0.0], quiet=True)
    for close in reversed(closers):
        try:
            close()
        except Exception:  # noqa: BLE001
            traceback.print_exc()
    if sync.world > 1:
        sync.reduce_max([0.0], quiet=True)
    return error


def last_block(sync: RankSync, fn) -> dict:
    """Runs the LAST measured block of a run so that its failure does not lose what was measured
    before: a rank whose block raises tells the others with one exchange (they are inside the block
    and learn of it at their next synchronisation point, which raises ``PeerFailed`` there), and
    every rank returns ``{"error": ...}`` in place of the block's figures. Nothing is launched on
    the communicators after that; the run then leaves as usual."""
    try:
        return fn()
    except PeerFailed as exc:  # learned at a synchronisation point: that exchange is consumed
        return {"error": str(exc)}
    except Exception as exc:  # noqa: BLE001
        traceback.print_exc()
        sync.reduce_max([0.0], fail=True)
        return {"error": f"{type(exc).__name__}: {exc}"}


def digest_of(t) -> float:
    """Order-independent exact checksum of a bf16 tensor's bits (fits a double exactly)."""
    import torch

    return float(t.contiguous().view(torch.int16).to(torch.int64).sum().item())


# ------------------------------------------------------------------ GPU arm
def parity_check(layer, comm, sync, rank: int, world: int, dev, x_dev, out_dev, cuts) -> dict:
    """One step before the timed region, checked: 24 sampled rows of every micro-batch against the
    CPU oracle (at N > 1 the fp32 rank-order sum of the per-shard oracle results), every rank
    holding identical bits, and at N > 1 the fused residual + RMSNorm form of the reduction against
    the oracle. Rank 0 evaluates the oracle; the others take part in the comparisons of bits."""
    import torch

    from dynaflow_b200 import ops
    from dynaflow_b200.layer import shard_bounds
    from oracle import ops_oracle

    rows_mb = ROWS // MICRO_BATCHES
    gen = torch.Generator().manual_seed(123)
    pick = torch.cat([torch.randint(0, rows_mb, (16,), generator=gen),
                      torch.tensor([0, 127, 128, rows_mb // 2, rows_mb - 128, rows_mb - 2, rows_mb - 1, 1])])
    rows = torch.cat([pick + cuts[mb] for mb in range(MICRO_BATCHES)])
    results: list = []
    layer.forward_device(x_dev, out_dev, cuts, results=results)
    torch.cuda.synchronize()
    ops.check_status()
    got_full = torch.cat(results) if world > 1 else out_dev
    identical = sync.all_equal(digest_of(got_full))
    got = got_full[rows.to(dev)].cpu()
    report = {"checked": True, "ranks_identical": bool(identical), "rows_sampled": int(rows.numel()),
              "against": "CPU oracle (oracle/ops_oracle.gated_mlp), fp32 rank-order sum of the per-shard results"}
    fused_got = fused_res = None
    if world > 1:
        # fused form of the reduction on the same partial sums: residual and weight from a seed
        g2 = torch.Generator().manual_seed(321)
        residual = torch.randn(ROWS, H, generator=g2).bfloat16()
        weight = (1 + 0.1 * torch.randn(H, generator=g2)).bfloat16()
        res_dev = residual.to(dev)
        outs = layer.forward_chain(x_dev, cuts, 1, weight.to(dev), res_dev, sharded_residual=True)
        torch.cuda.synchronize()
        ops.check_status()
        fused_full = torch.cat(list(outs))
        report["fused_ranks_identical"] = bool(sync.all_equal(digest_of(fused_full)))
        fused_got = fused_full[rows.to(dev)].cpu()
        fused_res = (residual, weight)
    worst = fused_worst = 0.0
    if rank == 0:
        host_threads()
        wg, wu, wd = cpu_weights()
        xs = x_dev[rows.to(dev)].cpu()
        parts = []
        for r in range(world):
            lo, hi = shard_bounds(I, r, world)
            parts.append(ops_oracle.gated_mlp(xs, wg[lo:hi], wu[lo:hi], wd[:, lo:hi]))
        acc = torch.zeros(xs.shape[0], H)
        for p in parts:
            acc += p.float()
        want = acc.bfloat16()
        worst = ((got.float() - want.float()).abs().max() / want.float().abs().max()).item()
        if fused_got is not None:
            residual, weight = fused_res
            want_out, _ = ops_oracle.allreduce_add_rmsnorm(parts, residual[rows], weight)
            fused_worst = ((fused_got.float() - want_out.float()).abs().max() / want_out.float().abs().max()).item()
    worst, fused_worst = sync.reduce_max([worst, fused_worst])
    report["max_rel_err"] = worst
    if world > 1:
        report["fused_add_rmsnorm_max_rel_err"] = fused_worst
    report["tolerance"] = TOL
    ok = identical and worst <= TOL and fused_worst <= TOL and report.get("fused_ranks_identical", True)
    report["ok"] = bool(ok)
    if not ok:
        raise AssertionError(f"parity check failed: {report}")
    return report


def torch_chain_ms(layer, x_dev, cuts, steps: int) -> dict:
    """The reference's own GPU operator chain for this layer, as its host model runs it inside a
    compute subgraph: cuBLAS linear, silu * mul, cuBLAS linear, bf16, the same tensors and
    micro-batches, timed in the same process outside the timed region of ``value``."""
    import torch
    import torch.nn.functional as F

    def step():
        for mb in range(len(cuts) - 1):
            x = x_dev[cuts[mb]:cuts[mb + 1]]
            F.linear(F.silu(F.linear(x, layer.w_gate)) * F.linear(x, layer.w_up), layer.w_down)

    with torch.inference_mode():
        for _ in range(3):
            step()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            step()
        b.record()
        torch.cuda.synchronize()
    ms = a.elapsed_time(b) / steps
    return {"ms_per_step": ms, "tokens_per_s": ROWS / (ms * 1e-3), "steps": steps,
            "what": "F.linear(gate), F.linear(up), silu * mul, F.linear(down) per micro-batch (cuBLAS + eager elementwise)"}


def decoder_block(args, sync, closers, rank: int, world: int, dev, plan: dict) -> dict:
    """Llama-3-8B-shaped decoder prefill (32 layers, hidden 4096, intermediate 14336, 32 query / 8
    key-value heads of 128, ids 8 x 2048, two micro-batches), tensor parallel over the ranks:
    tokens/s, fraction of the tensor peak and of the roofline, and at N > 1 how much of the
    communication the schedule hides."""
    import torch

    from dynaflow_b200 import ops
    from dynaflow_b200.decoder import DecoderShape, TensorParallelDecoder

    shape = DecoderShape(layers=args.layers)
    batch, seq = 8, 2048
    dec = TensorParallelDecoder(shape, rank=rank, world=world, max_rows=batch * seq // MICRO_BATCHES,
                                micro_batches=MICRO_BATCHES, seed=0, device=dev, n_ctas=max(plan["comm_ctas"], 1),
                                multicast=plan["comm"] == "multicast", gemm_max_ctas=plan["gemm_ctas"])
    closers.append(dec.close)
    ids = torch.randint(0, shape.vocab, (batch, seq), generator=torch.Generator().manual_seed(1)).to(dev)

    def timed(**kw):
        for _ in range(2):
            dec.forward(ids, **kw)
        sync.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 3
        a.record()
        for _ in range(reps):
            hidden = dec.forward(ids, **kw)
        b.record()
        sync.barrier()
        return sync.max_ms(a.elapsed_time(b) / reps), hidden

    t_all, hidden = timed()
    ops.check_status()
    identical = sync.all_equal(digest_of(hidden))
    peaks, kind = measured_peaks()
    s = shape
    linear = 2.0 * (s.hidden * (s.heads + 2 * s.kv_heads) * s.head_dim + s.heads * s.head_dim * s.hidden
                    + 3 * s.hidden * s.intermediate)
    attn = 4.0 * ((seq + 1) / 2) * s.heads * s.head_dim
    flops = (linear + attn) * s.layers * batch * seq
    peak = float(peaks["bf16_tflops"])
    out = {"workload": f"Llama-3-8B-shaped decoder prefill, {s.layers} layers, ids {batch}x{seq}, "
                       f"{MICRO_BATCHES} micro-batches, tp{world}; attention, GEMMs, RoPE, norms and reductions on "
                       "this library's kernels",
           "tokens_per_s": batch * seq / (t_all * 1e-3), "ms_per_forward": t_all, "flops_per_forward": flops,
           "tflops_per_gpu": flops / world / (t_all * 1e-3) / 1e12,
           "frac_of_tensor_peak": flops / world / (t_all * 1e-3) / 1e12 / peak,
           "peak_source": f"{kind} cuBLAS bf16 burst", "ranks_identical": bool(identical)}
    if world > 1:
        t_compute, _ = timed(skip_comm=True)
        t_comm, _ = timed(skip_compute=True)
        payload = 2 * s.layers * batch * seq * s.hidden * 2
        roofline_ms = max(flops / world / (peak * 1e12), (world - 1) / world * payload / 770e9) * 1e3
        out.update({"ms_compute_only": t_compute, "ms_comm_only": t_comm,
                    "hidden_frac": 1.0 - (t_all - t_compute) / t_comm,
                    "wire_ms_at_770_gbs": (world - 1) / world * payload / 770e9 * 1e3,
                    "roofline_ms": roofline_ms, "frac_of_roofline": roofline_ms / t_all})
    else:
        out["frac_of_roofline"] = out["frac_of_tensor_peak"]
    ops.check_status()
    return out


def small_gemm_block(args, rank: int, dev) -> dict:
    """The projections of a decode step for one tensor-parallel rank (of ``--shard-of``, default 8): 128 rows
    against the qkv, output, gate/up, down and vocabulary-shard weights, each shape as 24 launches on 24 copies of
    its weights (more than L2) inside one CUDA graph, CUDA events around five replays. Per shape: microseconds per
    launch (launch gap between dependent graph nodes included), weight bytes per second, and cuBLAS
    (``torch.matmul``) on the same tensors beside it."""
    import torch

    from dynaflow_b200 import ops
    from dynaflow_b200.decoder import DecoderShape

    n = args.shard_of if args.shard_of > 1 else 8
    s = DecoderShape()
    rows = args.decode_batch // MICRO_BATCHES
    q_cols, kv_cols = s.heads // n * s.head_dim, s.kv_heads // n * s.head_dim
    shapes = [("qkv", q_cols + 2 * kv_cols, s.hidden), ("output", s.hidden, q_cols), ("down", s.hidden, s.intermediate // n),
              ("vocabulary_shard", s.vocab // n, s.hidden)]
    copies, replays = 24, 5
    stream = torch.cuda.Stream(dev)

    def timed(fn) -> float:
        with torch.cuda.stream(stream):
            for i in range(3):
                fn(i)
            stream.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream, capture_error_mode="thread_local"):
                for i in range(copies):
                    fn(i)
            graph.replay()
            stream.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(replays):
                graph.replay()
            e1.record(stream)
            stream.synchronize()
        return e0.elapsed_time(e1) * 1000.0 / (replays * copies)

    gen = torch.Generator(device=dev).manual_seed(7)
    out: dict = {"workload": f"decode-step projections, {rows} rows, one rank's share of {n}", "shapes": {}}
    for name, N, K in shapes:
        a = torch.randn(rows, K, device=dev, generator=gen).bfloat16()
        w = [(torch.randn(N, K, device=dev, generator=gen) * 0.02).bfloat16() for _ in range(copies)]
        c = torch.empty(rows, N, device=dev, dtype=torch.bfloat16)
        us = timed(lambda i: ops.gemm_bf16(a, w[i], out=c))
        want = a.float() @ w[copies - 1].float().T
        err = ((c.float() - want).abs().max() / want.abs().max()).item()
        us_lib = timed(lambda i: torch.matmul(a, w[i].T, out=c))
        out["shapes"][name] = {"N": N, "K": K, "us": us, "weights_gbs": N * K * 2 / us / 1e3, "max_rel_err": err, "us_cublas": us_lib}
        del w
    H, I = s.hidden, s.intermediate // n
    x = torch.randn(rows, H, device=dev, generator=gen).bfloat16()
    wg = [(torch.randn(I, H, device=dev, generator=gen) * 0.02).bfloat16() for _ in range(copies)]
    wu = [(torch.randn(I, H, device=dev, generator=gen) * 0.02).bfloat16() for _ in range(copies)]
    h = torch.empty(rows, I, device=dev, dtype=torch.bfloat16)
    us = timed(lambda i: ops.gateup_silu(x, wg[i], wu[i], out=h))
    both = [torch.cat([wg[i], wu[i]]) for i in range(copies)]
    c2 = torch.empty(rows, 2 * I, device=dev, dtype=torch.bfloat16)
    us_lib = timed(lambda i: torch.matmul(x, both[i].T, out=c2))
    out["shapes"]["gate_up_silu"] = {"N": 2 * I, "K": H, "us": us, "weights_gbs": 2 * I * H * 2 / us / 1e3,
                                     "us_cublas": us_lib, "cublas_note": "one [2I, H] GEMM, no SiLU*mul"}
    ops.check_status()
    return out


def decode_block(args, sync, closers, rank: int, world: int, dev, plan: dict) -> dict:
    """Llama-3-8B-shaped decoder in DECODE: batch 256, one new token per sequence, key/value cache of
    4096 positions per sequence filled N(0,1), two micro-batches of 128, tensor parallel over the
    ranks, the whole step (every kernel and reduction of both streams) replayed as ONE CUDA graph.
    The step is bound by streaming weights and cache from HBM: tokens/s against that bound."""
    import torch

    from dynaflow_b200 import ops
    from dynaflow_b200.decoder import DecoderShape, TensorParallelDecoder

    shape = DecoderShape(layers=args.layers)
    if args.shard_of > 1:
        # one rank's share of an N-way tensor-parallel step on this GPU alone (no reductions): per-kernel profiling
        n = args.shard_of
        shape = DecoderShape(layers=args.layers, heads=shape.heads // n, kv_heads=shape.kv_heads // n,
                             intermediate=shape.intermediate // n, vocab=shape.vocab // n)
    batch, kv_len = args.decode_batch, args.kv_len
    dec = TensorParallelDecoder(shape, rank=rank, world=world, max_rows=batch // MICRO_BATCHES,
                                micro_batches=MICRO_BATCHES, seed=0, device=dev, n_ctas=max(plan["comm_ctas"], 1),
                                multicast=plan["comm"] == "multicast", gemm_max_ctas=plan["gemm_ctas"])
    closers.append(dec.close)
    dec.init_decode(batch, kv_len, context_len=kv_len, fill_seed=2)
    if args.decode_streams >= 0:
        dec.decode_streams_per_micro_batch = bool(args.decode_streams)
    ids = torch.randint(0, shape.vocab, (batch,), generator=torch.Generator().manual_seed(3)).to(dev)

    def timed(fn, reps):
        for _ in range(3):
            fn()
        sync.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            fn()
        b.record()
        sync.barrier()
        return sync.max_ms(a.elapsed_time(b) / reps)

    # One step first, with the device-side waits cut to a second: a reduction whose peers never arrive then
    # costs seconds, not minutes, and every rank learns of it here, before anything is timed.
    ops.set_timeout_ms(1000)
    trouble = None
    try:
        dec.decode_step(ids)
        torch.cuda.synchronize()
        ops.check_status()
    except Exception as exc:  # noqa: BLE001 -- told to the other ranks just below
        trouble = exc
    finally:
        ops.set_timeout_ms(2000)
    sync.reduce_max([0.0], fail=trouble is not None)
    if trouble is not None:   # the others know already (the exchange above): PeerFailed says "told"
        raise PeerFailed(f"the first decode step failed on rank {rank}: {type(trouble).__name__}: {trouble}") from trouble

    t_eager = timed(lambda: dec.decode_step(ids), 3)
    ops.check_status()
    replay, logits = dec.capture_decode(ids)
    t_graph = timed(replay, max(10, args.steps // 4))
    ops.check_status()
    identical = sync.all_equal(digest_of(torch.cat(dec.last_hidden)))
    finite = bool(torch.isfinite(torch.cat(logits).float()).all().item())
    peaks, kind = measured_peaks()
    weight_bytes = sum(t.numel() * 2 for layer in dec.layers for k, t in layer.items() if k.startswith("w"))
    weight_bytes += dec.lm_head_shard.numel() * 2
    kv_bytes = 2 * shape.layers * batch * kv_len * dec.kv_cols * 2
    total = weight_bytes + kv_bytes
    hbm = float(peaks["hbm_gbs"]) * 1e9
    out = {"workload": f"Llama-3-8B-shaped decode, {shape.layers} layers, batch {batch}, cache {kv_len} per sequence, "
                       f"{MICRO_BATCHES} micro-batches, tp{world}, one CUDA graph per step",
           "tokens_per_s": batch / (t_graph * 1e-3), "ms_per_step_graph": t_graph, "ms_per_step_eager_dispatch": t_eager,
           "hbm_bytes_per_step_per_gpu": total, "weights_bytes": weight_bytes, "kv_cache_bytes": kv_bytes,
           "achieved_gbs": total / (t_graph * 1e-3) / 1e9, "hbm_peak_gbs": float(peaks["hbm_gbs"]),
           "frac_of_hbm_roofline": total / hbm / (t_graph * 1e-3), "bound_tokens_per_s": batch / (total / hbm),
           "peak_source": f"{kind} copy bandwidth", "ranks_identical": bool(identical), "logits_finite": finite}
    if world > 1:
        replay_nc, _ = dec.capture_decode(ids, skip_comm=True)
        t_compute = timed(replay_nc, 10)
        replay_cc, _ = dec.capture_decode(ids, skip_compute=True)
        t_comm = timed(replay_cc, 10)
        out.update({"ms_compute_only": t_compute, "ms_comm_only": t_comm,
                    "hidden_frac": 1.0 - (t_graph - t_compute) / t_comm})
    ops.check_status()
    return out


def measure(args, sync, closers, rank: int, world: int, local_rank: int, dev) -> dict:
    import torch

    from dynaflow_b200 import ops
    from dynaflow_b200.layer import TensorParallelGatedMLP

    comm = comm_in = None
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
        closers.append(comm.close)
        comm_in = PeerComm(rank, world, ROWS // MICRO_BATCHES, H, slots=MICRO_BATCHES, n_ctas=plan["comm_ctas"], device=dev)
        closers.append(comm_in.close)
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
    norm_w = torch.ones(H, dtype=torch.bfloat16, device=dev)
    residual = torch.zeros(ROWS, H, dtype=torch.bfloat16, device=dev)
    chain_kw = dict(fused_norm=args.fused_norm, sharded_residual=not args.replicated_residual)

    sampler = ClockSampler(local_rank) if rank == 0 else None

    # ---- warm-up, then the result check, then the timed region
    if world == 1:
        for _ in range(args.warmup):
            layer.forward_device(x_dev, out_dev, cuts)
    else:
        layer.forward_chain(x_dev, cuts, args.warmup, norm_w, residual, **chain_kw)
    sync.barrier()
    ops.check_status()
    parity = parity_check(layer, comm, sync, rank, world, dev, x_dev, out_dev, cuts)
    sync.barrier()

    t_wall0 = time.time()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if world == 1:
        marks = []
        start.record()
        for _ in range(args.steps):
            marks.append(layer.forward_device(x_dev, out_dev, cuts, record_kernel_events=True))
        end.record()
        sync.barrier()
        mlp_ms = statistics.mean(m0.elapsed_time(m1) for step in marks for (m0, m1) in step)
        launches = layer.launches_per_step * args.steps
    else:
        # K dependent blocks: x <- rmsnorm(allreduce(mlp(x)) + residual), the reduction of a micro-batch under
        # the other micro-batch's GEMMs
        residual.zero_()
        timings: list = []
        start.record()
        layer.forward_chain(x_dev, cuts, args.steps, norm_w, residual, timings=timings, **chain_kw)
        end.record()
        sync.barrier()
        mlp_ms = statistics.mean(t0.elapsed_time(t1) for kind, t0, t1 in timings if kind == "mlp")
        launches = len(timings)
    t_wall1 = time.time()
    ms_step = sync.max_ms(start.elapsed_time(end) / args.steps)
    ops.check_status()

    # the same MLP as two launches, a few steps outside the timed region: how the time splits between the GEMMs
    for _ in range(2):
        layer.forward_device(x_dev, out_dev, cuts, record_kernel_events="split")
    split = [layer.forward_device(x_dev, out_dev, cuts, record_kernel_events="split") for _ in range(max(3, args.steps // 10))]
    sync.barrier()
    gateup_ms = statistics.median(m0.elapsed_time(m1) for step in split for (m0, m1, _m2) in step)
    down_ms = statistics.median(m1.elapsed_time(m2) for step in split for (_m0, m1, m2) in step)
    ops.check_status()

    # ---- N > 1: how much of the reduction hides under the other micro-batch's GEMMs
    comm_stats = None
    if world > 1:
        chain_layers = 8

        def timed(**kw):
            for _ in range(2):
                residual.zero_()
                layer.forward_chain(x_dev, cuts, chain_layers, norm_w, residual, **chain_kw, **kw)
            sync.barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            reps = max(4, args.steps // 16)
            a.record()
            for _ in range(reps):
                layer.forward_chain(x_dev, cuts, chain_layers, norm_w, residual, **chain_kw, **kw)
            b.record()
            sync.barrier()
            return sync.max_ms(a.elapsed_time(b) / reps / chain_layers)

        # all three measured the same way (short bursts at the same clocks); `value` keeps the long timed region
        t_overlap = timed()
        t_compute = timed(skip_comm=True)
        t_comm = timed(skip_compute=True)
        payload = ROWS * H * 2  # bytes reduced per block (all micro-batches)
        peak_tf = float(measured_peaks()[0]["bf16_tflops"])
        comm_stats = {"chain": "dependent TP MLP blocks; between them all-reduce + residual + RMSNorm: "
                               + ("reduce-scatter, add + norm on the owned rows (residual sharded by rows), all-gather, one launch"
                                  if not args.replicated_residual else
                                  ("replicated residual, one launch" if args.fused_norm
                                   else "replicated residual, reduction on few CTAs then normalisation over all SMs")),
                      "ms_per_block_overlapped": t_overlap, "ms_per_block_compute_only": t_compute,
                      "ms_per_block_comm_only": t_comm,
                      "hidden_frac": 1.0 - (t_overlap - t_compute) / t_comm,
                      # an in-switch reduction moves the payload once per direction and GPU; the peer form (W-1)/W of it, twice
                      "link_gbs_per_direction_comm_only": (payload if plan["comm"] == "multicast"
                                                           else 2.0 * (world - 1) / world * payload) / (t_comm * 1e-3) / 1e9,
                      "nvlink_peak_gbs": 770.0, "nvlink_peak_source": "measured peer copy, per direction",
                      "roofline_ms_per_block": max(6.0 * ROWS * H * (I // world) / (peak_tf * 1e12),
                                                   (world - 1) / world * payload / 770e9) * 1e3}
        comm_stats["frac_of_roofline_chain"] = comm_stats["roofline_ms_per_block"] / t_overlap
        ops.check_status()

    # ---- end to end: pinned host buffers, copies inside the timed region, the step driven through the drop-in API
    #      (DynaFlowManager.get_callable(): policy, nano-batch dispatch, native substitution of the MLP subgraph, the
    #      collectives as network-tagged subgraphs, whole-forward graph). Every rank owns 1/N of the rows of each
    #      micro-batch and copies only those in and out; copy-in, step and copy-out of consecutive steps ride on three
    #      streams with two buffers each.
    from dynaflow_b200.host_step import ManagedLayerStep

    if world == 1:
        sizes = [(0, cuts[i + 1] - cuts[i]) for i in range(MICRO_BATCHES)]
    else:
        sizes = [comm.slice_bounds(cuts[i + 1] - cuts[i]) for i in range(MICRO_BATCHES)]
    local = sum(hi - lo for lo, hi in sizes)
    cuts_local = [0]
    for lo, hi in sizes:
        cuts_local.append(cuts_local[-1] + hi - lo)
    xl = torch.cat([x_host[cuts[i] + lo: cuts[i] + hi] for i, (lo, hi) in enumerate(sizes)]).pin_memory()
    ol = torch.empty(local, H, dtype=torch.bfloat16).pin_memory()
    managed = ManagedLayerStep(layer, comm_in=comm_in, whole_forward_graph=True)
    main = torch.cuda.current_stream(dev)
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    x_bufs = [torch.empty(local, H, dtype=torch.bfloat16, device=dev) for _ in range(2)]
    o_bufs = [torch.empty(local, H, dtype=torch.bfloat16, device=dev) for _ in range(2)]
    consumed = [torch.cuda.Event() for _ in range(2)]
    arrived = [torch.cuda.Event() for _ in range(2)]
    ready = [torch.cuda.Event() for _ in range(2)]
    drained = [torch.cuda.Event() for _ in range(2)]
    for ev in consumed + drained:
        ev.record(main)
    step_no = [0]

    def e2e_step():
        k = step_no[0] & 1
        step_no[0] += 1
        with torch.cuda.stream(s_in):
            s_in.wait_event(consumed[k])
            x_bufs[k].copy_(xl, non_blocking=True)
            arrived[k].record(s_in)
        main.wait_event(arrived[k])
        main.wait_event(drained[k])
        y = managed(x_bufs[k], cuts_local)
        o_bufs[k].copy_(y)
        consumed[k].record(main)
        ready[k].record(main)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ready[k])
            ol.copy_(o_bufs[k], non_blocking=True)
            drained[k].record(s_out)

    def e2e_join():
        main.wait_stream(s_out)

    h2d = d2h = ROWS * H * 2          # whole job: each of the N ranks moves 1/N of it
    e2e_note = ("through DynaFlowManager.get_callable(): NanoFlow policy, 2 nano-batches, MLP subgraph substituted by the "
                "fused kernel" + ("" if world == 1 else ", all-gather / reduce-scatter as network-tagged subgraphs on the "
                                  "communication stream; each rank copies its 1/N of the rows in and out")
                + ", whole-forward graph replay; H2D, step and D2H of consecutive steps on three streams")
    for _ in range(args.warmup):
        e2e_step()
    e2e_join()
    sync.barrier()
    s2, e2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s2.record()
    for _ in range(args.steps):
        e2e_step()
    e2e_join()
    e2.record()
    sync.barrier()
    e2e_ms = sync.max_ms(s2.elapsed_time(e2) / args.steps)
    ops.check_status()
    # the end-to-end result, checked too: what came back to the host against the device-resident run
    results = []
    layer.forward_device(x_dev, out_dev, cuts, results=results)
    torch.cuda.synchronize()
    if world == 1:
        want_local = out_dev.cpu()
    else:
        want_local = torch.cat([results[i][lo:hi] for i, (lo, hi) in enumerate(sizes)]).cpu()
    rel = ((ol.float() - want_local.float()).abs().max() / want_local.float().abs().max()).item()
    e2e_equal = bool(sync.reduce_max([rel])[0] <= TOL)   # another summation order across ranks: within tolerance
    e2e_substituted = managed.substituted_per_step
    # the same step through the layer object (C ABI below TensorParallelGatedMLP), copies pipelined per micro-batch
    if world == 1:
        def abi_step():
            layer.forward_host(x_host, out_host, cuts)
    else:
        def abi_step():
            layer.forward_host_sliced(xl, ol, cuts, comm_in)
    for _ in range(args.warmup):
        abi_step()
    sync.barrier()
    s3, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s3.record()
    for _ in range(max(5, args.steps // 4)):
        abi_step()
    e3.record()
    sync.barrier()
    abi_ms = sync.max_ms(s3.elapsed_time(e3) / max(5, args.steps // 4))
    ops.check_status()
    if sampler is not None:
        sampler.stop()

    chain = torch_chain_ms(layer, x_dev, cuts, args.steps) if world == 1 else None
    decoder = decode = None
    if not args.no_decoder:
        decoder = decoder_block(args, sync, closers, rank, world, dev, plan)
        if world > 1:
            # (one GPU cannot hold the full key/value cache of this configuration beside the other workloads)
            # The last block of the run: if it fails, the line keeps everything measured before it and says so.
            decode = last_block(sync, lambda: decode_block(args, sync, closers, rank, world, dev, plan))

    peaks, peak_kind = measured_peaks()
    rows_mb = ROWS // MICRO_BATCHES
    mlp_flops = 6.0 * rows_mb * H * (I // world)          # one launch: gate/up 4 M H I + down 2 M H I
    achieved = mlp_flops / (mlp_ms * 1e-3) / 1e12
    burst = float(peaks["bf16_tflops"])
    sustained = float(peaks.get("bf16_tflops_sustained", burst))
    step_flops = 6.0 * ROWS * H * (I // world)
    traffic = MLP_DRAM_BYTES_PER_LAUNCH if (ROWS == 16384 and world == 1) else None

    cpu = None
    if world == 1 and not args.no_cpu_baseline and rank == 0:
        cpu = cpu_sample(12.0, 2048)

    sweep = None
    if world == 1 and not args.no_sweep:
        sweep = m_sweep(layer, dev, peaks)

    line = {
        "metric": METRIC, "value": ROWS / (ms_step * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": dict(workload_config(world), **({"reduction": plan, "step": "one block of a dependent chain: MLP, "
                                                   "all-reduce, residual add, RMSNorm"} if world > 1 else {})),
        "e2e": {"value": ROWS / (e2e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "how": e2e_note, "result_checked": e2e_equal,
                "through_manager": True, "subgraphs_substituted_per_step": e2e_substituted,
                "layer_object_c_abi": {"tokens_per_s": ROWS / (abi_ms * 1e-3), "ms_per_step": abi_ms}},
        "gpu_launches": launches,
        "parity": parity,
        "roofline": {"bound": "tensor",
                     "kernel": "gemm_tc_kernel<FUSED> (gate/up GEMM + SiLU*mul epilogue + down GEMM, one persistent launch)",
                     "achieved": achieved, "peak": burst, "unit": "TFLOP/s", "frac": achieved / burst,
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
        "torch_chain": chain,
        "decoder": decoder,
        "decode": decode,
        "sweep": sweep,
    }
    if chain is not None:
        line["torch_chain"]["fused_kernel_speedup"] = chain["ms_per_step"] / ms_step
    if world > 1:
        line["comm"] = dict(layer.comm_summary(), **(comm_stats or {}))
    return line


def run_ours(args) -> None:
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    sync = RankSync(world, dev)
    closers: list = []
    line, error, learned = None, None, False
    try:
        if args.workload == "moe":
            line = run_moe(args, sync, closers, rank, world, dev)
        elif args.workload == "decoder":
            line = decoder_block(args, sync, closers, rank, world, dev, comm_plan_applied(args, world))
        elif args.workload == "decode":
            line = decode_block(args, sync, closers, rank, world, dev, comm_plan_applied(args, world))
        elif args.workload == "small-gemm":
            if world != 1:
                raise SystemExit("--workload small-gemm runs on one GPU")
            line = small_gemm_block(args, rank, dev)
        else:
            line = measure(args, sync, closers, rank, world, local_rank, dev)
    except PeerFailed as exc:
        error, learned = str(exc), True
    except Exception as exc:  # noqa: BLE001 -- reported after every rank has left together
        traceback.print_exc()
        error = f"{type(exc).__name__}: {exc}"
    error = leave_together(sync, closers, error, learned)
    if world > 1:
        dist.destroy_process_group()
    if error is not None:
        print(f"[bench] rank {rank} failed: {error}", file=sys.stderr)
        sys.exit(1)
    if rank == 0:
        print(json.dumps(line))


def comm_plan_applied(args, world: int) -> dict:
    plan = comm_plan(args, world)
    if world > 1:
        from dynaflow_b200.comm import set_exclusive_sms

        set_exclusive_sms(plan["exclusive_sms"])
    return plan


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

        def unsplit():
            ops.gated_mlp(x, layer.w_gate, layer.w_up, layer.w_down, out=y, workspace=layer.workspaces[0])

        t_serial, t_overlap = time_it(serial), time_it(overlapped)
        # one nano-batch: what the split policy itself chooses below its minimum nano-batch size (the
        # reference's get_split_config returns a single nano-batch there), and the only form that
        # streams the weights once
        t_unsplit = time_it(unsplit) if rows <= layer.max_rows else None
        flops = 6.0 * rows * H * I
        bytes_min = 3.0 * H * I * 2 + 2.0 * rows * H * 2
        bound_ms = max(flops / (float(peaks["bf16_tflops"]) * 1e12), bytes_min / (float(peaks["hbm_gbs"]) * 1e9)) * 1e3
        best_split = min(t_serial, t_overlap)
        out.append({"rows": rows, "ms_serial": t_serial, "ms_overlapped": t_overlap, "ms_unsplit": t_unsplit,
                    "tflops_serial": flops / t_serial / 1e9,
                    "roofline_ms": bound_ms, "frac_of_roofline": bound_ms / best_split,
                    "frac_of_roofline_unsplit": (bound_ms / t_unsplit) if t_unsplit else None,
                    "bound": "tensor" if flops / (float(peaks["bf16_tflops"]) * 1e12) > bytes_min / (float(peaks["hbm_gbs"]) * 1e9) else "hbm"})
    ops.check_status()
    return out


def run_moe(args, sync, closers, rank: int, world: int, dev) -> dict:
    """Other workload (not the default line): Mixtral-shaped top-2 MoE stack, 16384 tokens per step, 8 experts of
    intermediate 14336, expert parallel over the launched ranks (one rank: all experts local), two nano-batches per
    rank in the dual-batch-overlap order (dispatch / combine of one nano-batch on the communication stream under the
    expert GEMMs of the other, ``examples/ae/scheduler/vllm/dbo.py:168-220``). ``--moe-exchange a2a`` moves only the
    routed rows (puts and pulls over peer memory), ``agrs`` is the all-gather / reduce-scatter form.
    value = tokens/s through `--moe-layers` layers."""
    import torch

    from dynaflow_b200 import ops
    from dynaflow_b200.moe import ExpertParallelMoE
    from oracle import ops_oracle

    experts, tokens, layers = 8, ROWS, args.moe_layers
    per_rank = tokens // world
    nb_tokens = per_rank // MICRO_BATCHES                  # one nano-batch of this rank
    gen = torch.Generator(device=dev).manual_seed(7)      # same weights on every rank; each keeps its experts

    def weight(*shape):
        return (torch.randn(*shape, device=dev, generator=gen) * 0.02).bfloat16()

    stack = []
    first_weights = None
    for li in range(layers):
        w = (weight(experts, I, H), weight(experts, I, H), weight(experts, H, I))
        if li == 0:
            first_weights = tuple(t[:, :, :].clone() for t in w)
        moe = ExpertParallelMoE(H, I, experts, nb_tokens, rank=rank, world=world, weights=w, slots=MICRO_BATCHES,
                                n_ctas=args.comm_ctas or 32, device=dev, exchange=args.moe_exchange)
        closers.append(moe.close)
        stack.append(moe)
        del w
    x = torch.randn(per_rank, H, device=dev, generator=torch.Generator(device=dev).manual_seed(100 + rank)).bfloat16()
    logits = [torch.randn(per_rank, experts, device=dev, generator=torch.Generator(device=dev).manual_seed(200 + 10 * li + rank)).bfloat16()
              for li in range(layers)]
    main = torch.cuda.current_stream(dev)
    comm_stream = torch.cuda.Stream(device=dev)
    outs = [[None] * MICRO_BATCHES for _ in range(layers)]

    def do_expert(layer, b, gathered, x_b, lg_b):
        if layer.exchange == "a2a":
            return layer.expert(None, None, slot=b)          # whatever rows the last dispatch delivered
        if gathered is None:                                  # compute only: the rows of the last full step
            gathered = ((layer.comm_x.result(b, layer.total_tokens), layer.comm_logits.result(b, layer.total_tokens))
                        if world > 1 else (x_b, lg_b))
        return layer.expert(*gathered, slot=b)

    def do_combine(layer, b, contrib):
        if layer.exchange == "a2a":
            return layer.combine(None, slot=b)
        if contrib is None:                                   # communication only: stale contributions
            contrib = layer.comm_out.partial(b, layer.total_tokens) if world > 1 else layer.local_contrib[b]
        return layer.combine(contrib, slot=b)

    def step(overlap: bool = True, skip_expert: bool = False, skip_comm: bool = False):
        """Per layer: disp0 | exp0 + disp1 | exp1 + comb0 | comb1, collectives on the communication stream."""
        cs = comm_stream if overlap else main
        for li, (layer, lg) in enumerate(zip(stack, logits)):
            xs = [x[b * nb_tokens:(b + 1) * nb_tokens] for b in range(MICRO_BATCHES)]
            lgs = [lg[b * nb_tokens:(b + 1) * nb_tokens] for b in range(MICRO_BATCHES)]
            disp, expd = [None] * MICRO_BATCHES, [None] * MICRO_BATCHES
            gathered = [None] * MICRO_BATCHES
            fork = torch.cuda.Event()
            fork.record(main)
            cs.wait_event(fork)
            for b in range(MICRO_BATCHES):
                with torch.cuda.stream(cs):
                    if not skip_comm:
                        gathered[b] = layer.dispatch(xs[b], lgs[b], slot=b)
                    disp[b] = torch.cuda.Event()
                    disp[b].record(cs)
            contrib = [None] * MICRO_BATCHES
            for b in range(MICRO_BATCHES):
                main.wait_event(disp[b])
                if not skip_expert:
                    contrib[b] = do_expert(layer, b, gathered[b], xs[b], lgs[b])
                expd[b] = torch.cuda.Event()
                expd[b].record(main)
                cs.wait_event(expd[b])
                with torch.cuda.stream(cs):
                    if not skip_comm:
                        outs[li][b] = do_combine(layer, b, contrib[b])
            main.wait_stream(cs)

    def timed(**kw):
        for _ in range(3):
            step(**kw)
        sync.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = max(3, args.steps // 10)
        a.record()
        for _ in range(reps):
            step(**kw)
        b.record()
        sync.barrier()
        return sync.max_ms(a.elapsed_time(b) / reps), reps

    # ---- result check before timing: this rank's rows of layer 0 against the CPU oracle (sampled tokens)
    step()
    torch.cuda.synchronize()
    ops.check_status()
    got = torch.cat([outs[0][b] for b in range(MICRO_BATCHES)])
    pick = torch.arange(0, per_rank, max(1, per_rank // 16))[:16]
    worst = 0.0
    host_threads()
    wg, wu, wd = (t.cpu() for t in first_weights)
    want = ops_oracle.moe_layer(x[pick].cpu(), logits[0][pick].cpu(), wg, wu, wd)
    worst = ((got[pick].float().cpu() - want.float()).abs().max() / want.float().abs().max()).item()
    worst = sync.reduce_max([worst])[0]
    if worst > TOL:
        raise AssertionError(f"MoE result check failed: max rel err {worst}")
    del first_weights, wg, wu, wd

    ms, reps = timed()
    ops.check_status()
    peaks, kind = measured_peaks()
    flops = 2.0 * tokens * 6.0 * H * I * layers               # two experts per token
    line = {"workload": f"Mixtral-shaped top-2 MoE, {layers} layers, {experts} experts x {I}, {tokens} tokens per step, ep{world}, "
                        f"{MICRO_BATCHES} nano-batches per rank in dual-batch-overlap order, exchange {args.moe_exchange}",
            "metric": "tokens/sec", "unit": "tokens/s", "n_gpus": world, "ms_per_step": ms, "value": tokens / (ms * 1e-3),
            "flops_per_step": flops, "tflops_per_gpu": flops / world / (ms * 1e-3) / 1e12,
            "frac_of_tensor_peak": flops / world / (ms * 1e-3) / 1e12 / float(peaks["bf16_tflops"]),
            "peak_source": f"{kind} cuBLAS bf16 burst", "steps": reps, "data": "synthetic",
            "parity": {"checked": True, "max_rel_err": worst, "against": "CPU oracle (ops_oracle.moe_layer), 16 sampled tokens per rank, layer 0"}}
    if world > 1:
        t_compute, _ = timed(skip_comm=True)
        t_comm, _ = timed(skip_expert=True)
        line.update({"ms_compute_only": t_compute, "ms_comm_only": t_comm,
                     "hidden_frac": 1.0 - (ms - t_compute) / t_comm})
        ops.check_status()
    # load balance of the first layer's routing (ids of this rank's view, two experts each)
    ids0 = stack[0].l_ids[0] if args.moe_exchange == "a2a" else stack[0].ids[0]
    counts = torch.bincount(ids0.flatten().to(torch.int64), minlength=experts).double()
    line["tokens_per_expert_max_over_mean"] = float((counts.max() / counts.mean()).item())
    return line


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
    ap.add_argument("--moe-exchange", choices=["a2a", "agrs"], default="a2a",
                    help="moe workload: all-to-all puts / pulls of the routed rows, or all-gather / reduce-scatter of all rows")
    ap.add_argument("--decode-batch", type=int, default=256, help="decode: sequences per step")
    ap.add_argument("--kv-len", type=int, default=4096, help="decode: cached positions per sequence")
    ap.add_argument("--decode-streams", type=int, default=-1, help="decode: 1 = one compute stream per micro-batch, 0 = one "
                    "for all (default: per micro-batch on one GPU, one for all with reductions)")
    ap.add_argument("--shard-of", type=int, default=1, help="decode on one GPU: run one rank's share of an N-way "
                    "tensor-parallel step (heads, key/value heads, intermediate and vocabulary divided by N, no reductions)")
    ap.add_argument("--workload", choices=["mlp", "decoder", "decode", "moe", "small-gemm"], default="mlp",
                    help="mlp: the fused gated-MLP layer step (the benchmark line, which also carries the decoder "
                         "block); decoder / decode / moe: that workload alone; small-gemm: the decode step's "
                         "projections per launch, one GPU")
    ap.add_argument("--layers", type=int, default=32, help="decoder: number of layers")
    ap.add_argument("--fused-norm", action="store_true", help="N > 1 chain: one-launch all-reduce+RMSNorm kernel")
    ap.add_argument("--no-sweep", action="store_true", help="skip the M sweep (profiling runs)")
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU baseline leg (profiling runs)")
    ap.add_argument("--no-decoder", action="store_true", help="skip the decoder block (profiling runs)")
    args = ap.parse_args()
    if args.rows != ROWS:
        if args.rows <= 0 or args.rows % (MICRO_BATCHES * 8) != 0:
            raise SystemExit("--rows must be a positive multiple of 16")
        ROWS = args.rows
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
