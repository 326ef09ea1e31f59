"""Entry point a host framework talks to.

Public surface and semantics follow the reference's ``dynaflow/manager.py``:

* ``initialize(graph_module, config, scheduler, example_inputs)`` partitions and
  tags the traced forward, wraps each subgraph in its back-end and builds the
  engine (``manager.py:37-112``);
* ``prepare(batch_size, num_tokens, is_dryrun, use_cudagraph)`` asks the policy
  for the next step's ``SplitConfig`` (a trivial one-nano-batch config before
  initialisation or for a dry run) and caches it; ``override_split_config``
  replaces it (``manager.py:114-159``);
* ``get_callable()`` returns the synchronous forward; every call consumes the
  cached config (``manager.py:161-190``) and merges per-nano-batch results by
  concatenation along dim 0, field by field for tuples (``manager.py:236-261``).

Addition: with ``additional_config["whole_forward_graph"]`` the split forward of each
split shape is captured once as a single multi-stream CUDA graph and replayed
(``runtime/graph_schedule.py``).

Differences: nothing is printed per forward (set ``DYNAFLOW_LOG=1`` to log the
split config), the readable graph dump is only written when ``DYNAFLOW_DUMP_GRAPH``
is set, and no asyncio event loop is created per forward.
"""
from __future__ import annotations

import os
import tempfile
from collections.abc import Callable
from typing import Any

import torch
import torch.fx

from .config import DynaFlowConfig
from .executor.compiler import SubgraphCompiler
from .interface import InputInfo, OpSchedulerBase, SplitConfig
from .matching import split_graph, tag_graph
from .runtime.engine import DynaFlowEngine
from .runtime.graph_schedule import WholeForwardGraphs


def _targets_without(gm: torch.fx.GraphModule, forbidden_tag: str) -> list[str]:
    """Names of tagged subgraphs whose tag set lacks ``forbidden_tag``."""
    return [name for name, module in gm.named_modules()
            if isinstance(getattr(module, "tag", None), set) and forbidden_tag not in module.tag]


def merge_nano_batch_results(results: dict[int, Any], num_nano_batches: int) -> Any:
    """Joins per-nano-batch outputs into the unsplit forward's output: tensors are
    concatenated on dim 0, tuples field by field, anything else is taken from
    nano-batch 0."""
    first = results[0]
    if any(not isinstance(results[i], type(first)) for i in range(num_nano_batches)):
        raise AssertionError(f"Results have different types: {results}")
    if isinstance(first, torch.Tensor):
        return torch.cat([results[i] for i in range(num_nano_batches)], dim=0)
    if isinstance(first, tuple):
        width = len(first)
        if any(len(results[i]) != width for i in range(num_nano_batches)):
            raise AssertionError(f"Results have different number of elements: {results}")
        merged = []
        for field in range(width):
            parts = [results[i][field] for i in range(num_nano_batches)]
            if any(not isinstance(part, torch.Tensor) for part in parts):
                raise AssertionError(f"Elements are not tensors: {parts}")
            merged.append(torch.cat(parts, dim=0))
        return tuple(merged)
    return first


class DynaFlowManager:
    def __init__(self) -> None:
        self.initialized = False
        self.config: DynaFlowConfig | None = None
        self.graph_module: torch.fx.GraphModule | None = None
        self.cached_config: SplitConfig | None = None
        self.scheduler: OpSchedulerBase | None = None
        self.engine: DynaFlowEngine | None = None
        self.forward_graphs: WholeForwardGraphs | None = None

    def initialize(self, graph_module: torch.fx.GraphModule, config: DynaFlowConfig, scheduler: OpSchedulerBase,
                   example_inputs: list[Any]) -> None:
        """Must be called from inside a ``torch.compile`` backend with dim 0 of the
        dynamic inputs marked dynamic, so that every subgraph receives the row
        count as a ``torch.SymInt``."""
        self.initialized = True
        self.config = config
        self.graph_module = split_graph(graph_module, scheduler.get_split_rules())
        tag_graph(self.graph_module, scheduler.get_tag_rules())
        inductor_targets = _targets_without(self.graph_module, "no-inductor") if config.inductor_config.enabled else []
        cudagraph_targets = _targets_without(self.graph_module, "no-cudagraph") if config.cudagraph_config.enabled else []

        if os.environ.get("DYNAFLOW_DUMP_GRAPH"):
            path = os.path.join(tempfile.mkdtemp(), "gm_with_subgraphs.py")
            with open(path, "w") as f:
                f.write(f"# Inductor targets (ignored by this backend): {inductor_targets}\n")
                f.write(f"# CUDAGraph targets: {cudagraph_targets}\n")
                f.write(self.graph_module.print_readable(print_output=False))
            print(f"Graph saved to {path}")

        SubgraphCompiler(self.graph_module, config, inductor_compile_targets=inductor_targets,
                         cudagraph_targets=cudagraph_targets).run(*example_inputs)
        self.engine = DynaFlowEngine(self.graph_module, config)
        self.scheduler = scheduler
        self.forward_graphs = None
        if config.additional_config.get("whole_forward_graph", False):
            engine = self.engine

            def is_dynamic(idx: int) -> bool:
                example = engine.placeholder_nodes[idx].meta.get("example_value", None)
                return (isinstance(example, torch.Tensor) and example.dim() > 0
                        and isinstance(example.shape[0], torch.SymInt))

            self.forward_graphs = WholeForwardGraphs(self._forward_split, is_dynamic,
                                                     config.additional_config.get("whole_forward_graph_keys"))

    def prepare(self, batch_size: int, num_tokens: list[int], is_dryrun: bool = False,
                use_cudagraph: bool = False) -> SplitConfig:
        total = sum(num_tokens)
        if not self.initialized or is_dryrun:
            self.cached_config = SplitConfig(num_nano_batches=1, batch_sizes=[batch_size],
                                             batch_indices=[0, batch_size], num_tokens=[total],
                                             num_tokens_padded=[total], split_indices=[0, total],
                                             is_dryrun=is_dryrun, use_cudagraph=use_cudagraph)
        else:
            assert self.scheduler is not None
            self.cached_config = self.scheduler.get_split_config(InputInfo(batch_size, num_tokens, total),
                                                                 use_cudagraph=use_cudagraph)
        return self.cached_config

    def override_split_config(self, split_config: SplitConfig) -> None:
        self.cached_config = split_config

    def get_callable(self) -> Callable[..., Any]:
        assert self.initialized

        def _forward(*args: Any, **kwargs: Any) -> Any:
            cfg = self.cached_config
            assert cfg is not None and self.engine is not None and self.scheduler is not None, \
                "prepare() or override_split_config() must be called before every forward"
            if os.environ.get("DYNAFLOW_LOG"):
                print(f"Executing with SplitConfig: {cfg}")
            try:
                if not cfg.is_dryrun and cfg.num_nano_batches == 1 and cfg.allow_fallback:
                    return self.engine.execute_single_batch(cfg, args, kwargs)
                if self.forward_graphs is not None and not cfg.is_dryrun and not cfg.use_cudagraph and not kwargs:
                    engine = self.engine
                    return self.forward_graphs.run(cfg, args, kwargs, lambda: engine.last_trace)
                return self._forward_split(cfg, args, kwargs)
            finally:
                self.cached_config = None

        return _forward

    def _forward_split(self, cfg: SplitConfig, args: tuple, kwargs: dict) -> Any:
        assert self.engine is not None and self.scheduler is not None
        if cfg.is_dryrun:
            results, events = self.engine.dryrun(args, kwargs, cfg)
            count = 1
        else:
            results, events = self.engine.execute(args, kwargs, cfg, self.scheduler)
            count = cfg.num_nano_batches
        for event in events:
            event.wait()  # the caller's stream now depends on every nano-batch's last operator
        return merge_nano_batch_results(results, count)
