"""Whole-forward schedule graphs: the policy's interleaving of all nano-batches on all
streams, recorded once per split shape and replayed as ONE CUDA graph.

The reference re-runs its policy coroutine and engine loop for every forward: for a
Llama-3-8B prefill with the NanoFlow cuts that is about 390 operator dispatches, each
with two event-loop round trips, two CUDA events and an NVTX range
(``dynaflow/runtime/engine.py:272-424``); its own study measures that class of launch
bubble at up to 45 % GPU idle (``examples/ae/MOE.md:59-66``). A policy's decisions depend
only on the split shape (number of nano-batches, their row counts) and on the operator
tags, so here the first forward of a shape runs the policy live under stream capture
-- the policy's ``torch.cuda.stream(...)`` switches become forks, the engine's
per-nano-batch events become the edges between them -- and every later forward of that
shape is one ``cudaGraphLaunch`` after copying the dynamic inputs into the graph's
static input tensors.

Enabled with ``additional_config["whole_forward_graph"] = True``. What it requires of
the host: every operator must be capturable (no host synchronisation, no allocation
outside the graph's pool -- true of this library's kernels, whose peer flags carry a
device-side sequence number for exactly this reason), and the policy must not make
decisions that vary between forwards of the same shape (set
``additional_config["whole_forward_graph_keys"]`` to a callable returning extra key
material if it does). Outputs live in the graph's memory pool and are overwritten by
the next replay of the same shape, as with the reference's per-subgraph CUDA graphs
(``dynaflow/executor/cudagraph.py:108-123``).
"""
from __future__ import annotations

from collections.abc import Callable
from typing import Any

import torch

from ..interface import SplitConfig


class _Captured:
    __slots__ = ("graph", "static_args", "output", "replays", "trace")

    def __init__(self, graph: Any, static_args: list, output: Any, trace: list) -> None:
        self.graph = graph
        self.static_args = static_args
        self.output = output
        self.replays = 0
        self.trace = trace


def _key_of(cfg: SplitConfig, args: tuple, extra: Any) -> tuple:
    shapes = tuple((tuple(a.shape), a.dtype, a.device.index) if isinstance(a, torch.Tensor) else ("v", a)
                   for a in args)
    return (cfg.num_nano_batches, tuple(cfg.num_tokens), tuple(cfg.num_tokens_padded), tuple(cfg.split_indices),
            cfg.use_cudagraph, shapes, extra)


class WholeForwardGraphs:
    """Cache of captured forwards, one per split shape."""

    def __init__(self, run_split: Callable[[SplitConfig, tuple, dict], Any], is_dynamic_arg: Callable[[int], bool],
                 extra_key: Callable[[], Any] | None = None, warmup_runs: int = 1) -> None:
        self._run_split = run_split
        self._is_dynamic = is_dynamic_arg
        self._extra_key = extra_key
        self._warmup_runs = warmup_runs
        self._entries: dict[tuple, _Captured] = {}
        self._pool = None
        self.captures = 0

    def __len__(self) -> int:
        return len(self._entries)

    def run(self, cfg: SplitConfig, args: tuple, kwargs: dict, last_trace: Callable[[], list]) -> Any:
        key = _key_of(cfg, args, self._extra_key() if self._extra_key is not None else None)
        entry = self._entries.get(key)
        if entry is None:
            entry = self._capture(cfg, args, kwargs, last_trace)
            self._entries[key] = entry
        else:
            for static, live in zip(entry.static_args, args):
                if isinstance(static, torch.Tensor) and static is not live:
                    static.copy_(live, non_blocking=True)
        entry.graph.replay()
        entry.replays += 1
        return entry.output

    def _capture(self, cfg: SplitConfig, args: tuple, kwargs: dict, last_trace: Callable[[], list]) -> _Captured:
        # dynamic inputs get graph-owned copies; weights and other static-shape inputs are
        # captured by address (they must stay where they are, as for any CUDA graph)
        static_args = [a.clone() if isinstance(a, torch.Tensor) and self._is_dynamic(i) else a
                       for i, a in enumerate(args)]
        current = torch.cuda.current_stream()
        side = torch.cuda.Stream()
        side.wait_stream(current)
        with torch.cuda.stream(side):
            for _ in range(self._warmup_runs):   # lazy initialisation (handles, workspaces) happens here, uncaptured
                self._run_split(cfg, tuple(static_args), kwargs)
        current.wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        if self._pool is None:
            self._pool = torch.cuda.graph_pool_handle()
        with torch.cuda.graph(graph, pool=self._pool):
            output = self._run_split(cfg, tuple(static_args), kwargs)
        self.captures += 1
        return _Captured(graph, static_args, output, list(last_trace()))
