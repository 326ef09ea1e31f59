"""The batch-split gated-MLP layer step as a user-facing object.

``TensorParallelGatedMLP`` owns one rank's weight shards, the per-micro-batch
scratch for the bf16 intermediate, and the streams of the overlapped schedule:

* ``forward_device`` runs the micro-batches back to back on the caller's stream
  (inputs and outputs resident in HBM);
* ``forward_host`` takes pinned host buffers: micro-batch ``i`` is copied in, run
  and copied out on its own stream, so the copies of one micro-batch hide under
  the GEMMs of the other -- the same interleaving the NanoFlow policy produces
  for ``network``-tagged subgraphs (``examples/ae/scheduler/hf/nanoflow.py:123-146``).

With ``world > 1`` the intermediate dimension is sharded (gate/up by output rows,
down by input columns, i.e. Megatron column/row parallel) and the partial outputs
of a micro-batch are summed across ranks by the peer-memory all-reduce on the
communication stream while the next micro-batch's GEMMs run.
"""
from __future__ import annotations

from typing import Any

import torch

from . import ops


class TensorParallelGatedMLP:
    def __init__(self, hidden: int, intermediate: int, *, rank: int = 0, world: int = 1, max_rows: int,
                 micro_batches: int = 2, seed: int = 0, device: torch.device | None = None,
                 weights: tuple[torch.Tensor, torch.Tensor, torch.Tensor] | None = None,
                 comm: Any | None = None) -> None:
        if intermediate % world != 0:
            raise ValueError("the intermediate size must divide evenly across ranks")
        self.hidden, self.intermediate = hidden, intermediate
        self.rank, self.world = rank, world
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.micro_batches = micro_batches
        self.max_rows = max_rows
        lo, hi = shard_bounds(intermediate, rank, world)
        shard = hi - lo
        if weights is None:
            # full weights N(0, 0.02) from the seed (identical on every rank), then this rank's shard
            g = torch.Generator().manual_seed(seed)
            w_gate = (torch.randn(intermediate, hidden, generator=g) * 0.02).bfloat16()
            w_up = (torch.randn(intermediate, hidden, generator=g) * 0.02).bfloat16()
            w_down = (torch.randn(hidden, intermediate, generator=g) * 0.02).bfloat16()
        else:
            w_gate, w_up, w_down = weights
        self.w_gate = w_gate[lo:hi].contiguous().to(self.device)
        self.w_up = w_up[lo:hi].contiguous().to(self.device)
        self.w_down = w_down[:, lo:hi].contiguous().to(self.device)
        self.shard = shard
        ws_bytes = ops.mlp_workspace_bytes(max_rows, hidden, shard)
        self.workspaces = [torch.empty(ws_bytes, dtype=torch.uint8, device=self.device) for _ in range(micro_batches)]
        self.h_views = [ws[: max_rows * shard * 2].view(torch.bfloat16).view(max_rows, shard) for ws in self.workspaces]
        self.streams = [torch.cuda.Stream(device=self.device) for _ in range(micro_batches)]
        self.staging_in = [torch.empty(max_rows, hidden, dtype=torch.bfloat16, device=self.device)
                           for _ in range(micro_batches)]
        self.staging_out = [torch.empty(max_rows, hidden, dtype=torch.bfloat16, device=self.device)
                            for _ in range(micro_batches)]
        self.comm = comm
        if world > 1 and comm is None:
            raise ValueError("world > 1 needs a communicator (dynaflow_b200.comm.PeerComm)")
        # kernels of this library per step at the benchmark's shapes: one persistent MLP launch per
        # micro-batch (two below a wave of tiles) plus one reduction per micro-batch
        self.launches_per_step = micro_batches + (micro_batches if world > 1 else 0)
        # CTAs the GEMMs may use (0 = one per SM). Fewer leaves whole SMs to the reduction that
        # runs beside the next micro-batch's GEMMs.
        self.gemm_max_ctas = 0
        # per slot: the event after which the slot's partial-output buffer may be overwritten
        self._slot_free: list[torch.cuda.Event | None] = [None] * micro_batches

    # ------------------------------------------------------------------
    def _mlp(self, x: torch.Tensor, out: torch.Tensor, mb: int, record: bool):
        rows = x.shape[0]
        h = self.h_views[mb][:rows]
        marks = None
        if record == "split":
            # the two GEMMs as separate launches, an event between them (measurement of the split only)
            m0, m1, m2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
            m0.record()
            ops.gateup_silu(x, self.w_gate, self.w_up, out=h, max_ctas=self.gemm_max_ctas)
            m1.record()
            ops.gemm_bf16(h, self.w_down, out=out, max_ctas=self.gemm_max_ctas)
            m2.record()
            marks = (m0, m1, m2)
        elif record:
            m0, m1 = (torch.cuda.Event(enable_timing=True) for _ in range(2))
            m0.record()
            ops.gated_mlp(x, self.w_gate, self.w_up, self.w_down, out=out, workspace=self.workspaces[mb],
                          max_ctas=self.gemm_max_ctas)
            m1.record()
            marks = (m0, m1)
        else:
            ops.gated_mlp(x, self.w_gate, self.w_up, self.w_down, out=out, workspace=self.workspaces[mb],
                          max_ctas=self.gemm_max_ctas)
        return marks

    def forward_device(self, x: torch.Tensor, out: torch.Tensor, cuts: list[int], record_kernel_events: bool | str = False,
                       results: list | None = None, skip_comm: bool = False, skip_compute: bool = False,
                       join: bool = True):
        """Runs ``mlp(x[cuts[i]:cuts[i+1]])`` for every micro-batch ``i`` on the current stream.

        ``record_kernel_events``: ``True`` returns a (start, end) event pair around every micro-batch's
        MLP launch, ``"split"`` runs gate/up and down as two launches with an event between them.
        Single rank: the rows land in ``out``. Tensor parallel: each micro-batch's partial
        output is written straight into the communicator's region and reduced on the
        communication stream while the next micro-batch's GEMMs run; the reduced rows
        are then ``comm.result(slot, rows)`` (appended to ``results`` if given), and the
        current stream waits for the last reduction before the call returns -- unless
        ``join=False``: then consecutive calls pipeline the way consecutive layers do, the last
        micro-batch's reduction running under the next call's first GEMMs (each GEMM waits only
        for the previous reduction out of its own slot, whose buffer it overwrites), and the
        caller joins with ``wait_reductions()`` before reading a result.
        ``skip_comm`` / ``skip_compute`` run the same schedule with the reductions, resp. the
        GEMMs, left out (measurement of how much communication the overlap hides)."""
        marks = []
        main = torch.cuda.current_stream(self.device)
        for mb in range(len(cuts) - 1):
            lo, hi = cuts[mb], cuts[mb + 1]
            if hi == lo:
                continue
            slot = mb % self.micro_batches
            target = out[lo:hi] if self.world == 1 else self.comm.partial(slot, hi - lo)
            if self.world > 1 and self._slot_free[slot] is not None:
                main.wait_event(self._slot_free[slot])
                self._slot_free[slot] = None
            if not skip_compute:
                m = self._mlp(x[lo:hi], target, slot, record_kernel_events)
                if m is not None:
                    marks.append(m)
            if self.world > 1 and not skip_comm:
                ready = torch.cuda.Event()
                ready.record(main)
                self.comm.stream.wait_event(ready)
                with torch.cuda.stream(self.comm.stream):
                    reduced = self.comm.all_reduce(slot, hi - lo)
                    freed = torch.cuda.Event()
                    freed.record(self.comm.stream)
                self._slot_free[slot] = freed
                if results is not None:
                    results.append(reduced)
            elif results is not None:
                results.append(target)
        if self.world > 1 and join:
            self.wait_reductions()
        return marks

    def wait_reductions(self) -> None:
        """Makes the current stream wait for every reduction issued so far."""
        if self.world > 1:
            torch.cuda.current_stream(self.device).wait_stream(self.comm.stream)
            self._slot_free = [None] * self.micro_batches

    def forward_chain(self, x: torch.Tensor, cuts: list[int], layers: int, norm_weight: torch.Tensor,
                      residual: torch.Tensor, skip_comm: bool = False, skip_compute: bool = False,
                      fused_norm: bool = True, sharded_residual: bool = False,
                      timings: list | None = None) -> list[torch.Tensor]:
        """``layers`` tensor-parallel MLP blocks back to back, the way a decoder runs them: for
        every micro-batch ``x <- rmsnorm(allreduce(mlp(x)) + residual) * w`` with the fused
        reduction kernel on the communication stream, so that the reduction of micro-batch
        ``i`` runs under the GEMMs of micro-batch ``i+1`` -- of the same block or, for the last
        micro-batch, of the next block. (All blocks share this object's weights; it exists to
        measure the steady-state overlap.) With ``sharded_residual`` the residual stream is
        sharded by rows and the add + RMSNorm happen inside the reduction, between its two
        shots; the block's output is then the communicator's result buffer, which the next
        block's reduction of the same micro-batch overwrites -- after that block's GEMMs have
        consumed it. Returns the per-micro-batch outputs. ``timings``, if given, receives one
        ``(kind, start_event, end_event)`` per GEMM pair ("mlp") and per reduction ("reduce")."""
        assert self.world > 1 and self.comm is not None
        main = torch.cuda.current_stream(self.device)
        comm_stream = self.comm.stream
        n_mb = len(cuts) - 1
        xs = [x[cuts[i]:cuts[i + 1]] for i in range(n_mb)]
        res = [residual[cuts[i]:cuts[i + 1]] for i in range(n_mb)]
        outs = [self.staging_out[i % self.micro_batches][: cuts[i + 1] - cuts[i]] for i in range(n_mb)]
        start = torch.cuda.Event()
        start.record(main)
        comm_stream.wait_event(start)
        reduced: list[torch.cuda.Event | None] = [None] * n_mb
        for _layer in range(layers):
            for mb in range(n_mb):
                rows = cuts[mb + 1] - cuts[mb]
                slot = mb % self.micro_batches
                if reduced[mb] is not None:
                    main.wait_event(reduced[mb])          # this micro-batch's input is the previous block's output
                if not skip_compute:
                    if timings is not None:
                        t0 = torch.cuda.Event(enable_timing=True)
                        t0.record(main)
                    self._mlp(xs[mb], self.comm.partial(slot, rows), slot, False)
                    if timings is not None:
                        t1 = torch.cuda.Event(enable_timing=True)
                        t1.record(main)
                        timings.append(("mlp", t0, t1))
                ready = torch.cuda.Event()
                ready.record(main)
                if not skip_comm:
                    comm_stream.wait_event(ready)
                    with torch.cuda.stream(comm_stream):
                        if timings is not None:
                            c0 = torch.cuda.Event(enable_timing=True)
                            c0.record(comm_stream)
                        if sharded_residual:
                            nxt = self.comm.all_reduce_add_rmsnorm_sharded(slot, rows, res[mb], norm_weight)
                        else:
                            self.comm.all_reduce_add_rmsnorm(slot, rows, res[mb], norm_weight, outs[mb], res[mb],
                                                             fused=fused_norm)
                            nxt = outs[mb]
                        done = torch.cuda.Event(enable_timing=timings is not None)
                        done.record(comm_stream)
                        if timings is not None:
                            timings.append(("reduce", c0, done))
                    reduced[mb] = done
                    xs[mb] = nxt
                    if sharded_residual:
                        outs[mb] = nxt
        main.wait_stream(comm_stream)
        return outs

    def forward_host(self, x_host: torch.Tensor, out_host: torch.Tensor, cuts: list[int]) -> None:
        """Same step from pinned host memory: copy-in, GEMMs, reduction and copy-out of a
        micro-batch ride on that micro-batch's own stream. ``x_host`` must be complete on the
        host when this is called (the copies do not wait for the caller's stream); the caller's
        stream waits for both micro-batches' copy-out before anything it enqueues afterwards.
        Consecutive calls pipeline: the copies of one micro-batch slot run under the GEMMs of
        the other slot, across calls too."""
        main = torch.cuda.current_stream(self.device)
        joins = []
        for mb in range(len(cuts) - 1):
            lo, hi = cuts[mb], cuts[mb + 1]
            if hi == lo:
                continue
            slot = mb % self.micro_batches
            stream = self.streams[slot]
            with torch.cuda.stream(stream):
                xin = self.staging_in[slot][: hi - lo]
                xin.copy_(x_host[lo:hi], non_blocking=True)
                if self.world == 1:
                    yout = self.staging_out[slot][: hi - lo]
                    self._mlp(xin, yout, slot, False)
                else:
                    self._mlp(xin, self.comm.partial(slot, hi - lo), slot, False)
                    # reductions of all micro-batches go through the ONE communication stream, so
                    # every rank issues them in the same order and two of them never wait on each
                    # other across GPUs in opposite orders
                    ready = torch.cuda.Event()
                    ready.record(stream)
                    self.comm.stream.wait_event(ready)
                    with torch.cuda.stream(self.comm.stream):
                        yout = self.comm.all_reduce(slot, hi - lo)
                        reduced = torch.cuda.Event()
                        reduced.record(self.comm.stream)
                    stream.wait_event(reduced)
                out_host[lo:hi].copy_(yout, non_blocking=True)
                done = torch.cuda.Event()
                done.record(stream)
                joins.append(done)
        for done in joins:
            main.wait_event(done)

    def forward_host_sliced(self, x_host_local: torch.Tensor, out_host_local: torch.Tensor, cuts: list[int],
                            comm_in: Any) -> None:
        """The host-staged step at ``world > 1`` without replicated copies: of every micro-batch
        ``[cuts[i], cuts[i+1])`` this rank owns the row slice ``comm.slice_bounds(rows)``;
        ``x_host_local`` / ``out_host_local`` (pinned) hold this rank's slices of all micro-batches
        back to back. Per micro-batch, on its own stream: copy the slice in, all-gather the
        micro-batch over NVLink (``comm_in``, a second communicator for the input rows), run the
        GEMMs on all rows, reduce-scatter the partial outputs, copy the owned rows out. Host
        traffic per rank and step is ``2 * rows * hidden * 2 / world`` bytes. The collectives of all
        micro-batches go through the one communication stream, in the same order on every rank."""
        assert self.world > 1 and self.comm is not None
        main = torch.cuda.current_stream(self.device)
        cs = self.comm.stream
        plan = []
        base = 0
        for mb in range(len(cuts) - 1):
            rows = cuts[mb + 1] - cuts[mb]
            if rows == 0:
                continue
            lo, hi = self.comm.slice_bounds(rows)
            plan.append((mb % self.micro_batches, rows, lo, hi, base))
            base += hi - lo
        # first the copies in and the all-gathers of every micro-batch, then the GEMMs: the second
        # micro-batch's rows arrive under the first one's GEMMs
        gathered = []
        for slot, rows, lo, hi, at in plan:
            stream = self.streams[slot]
            with torch.cuda.stream(stream):
                comm_in.partial(slot, rows)[lo:hi].copy_(x_host_local[at:at + hi - lo], non_blocking=True)
                ready = torch.cuda.Event()
                ready.record(stream)
            cs.wait_event(ready)
            with torch.cuda.stream(cs):
                x_all = comm_in.all_gather(slot, rows)
                ev = torch.cuda.Event()
                ev.record(cs)
            gathered.append((x_all, ev))
        joins = []
        for (slot, rows, lo, hi, at), (x_all, ev) in zip(plan, gathered):
            stream = self.streams[slot]
            with torch.cuda.stream(stream):
                stream.wait_event(ev)
                self._mlp(x_all, self.comm.partial(slot, rows), slot, False)
                done = torch.cuda.Event()
                done.record(stream)
                cs.wait_event(done)
                with torch.cuda.stream(cs):
                    y_mine = self.comm.reduce_scatter(slot, rows)
                    reduced = torch.cuda.Event()
                    reduced.record(cs)
                stream.wait_event(reduced)
                out_host_local[at:at + hi - lo].copy_(y_mine, non_blocking=True)
                out_done = torch.cuda.Event()
                out_done.record(stream)
                joins.append(out_done)
        for ev in joins:
            main.wait_event(ev)

    def comm_summary(self) -> dict:
        return self.comm.summary() if self.comm is not None else {}


def shard_bounds(intermediate: int, rank: int, world: int) -> tuple[int, int]:
    """Rows of W_gate / W_up (columns of W_down) that rank ``rank`` of ``world`` owns."""
    if intermediate % world != 0:
        raise ValueError("the intermediate size must divide evenly across ranks")
    shard = intermediate // world
    return rank * shard, (rank + 1) * shard
