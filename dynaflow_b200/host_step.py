"""The gated-MLP layer step driven through the drop-in API, the way a host drives the reference
(``dynaflow/manager.py:161-190``): a PyTorch module is traced once under ``torch.compile`` with a
backend that hands the FX graph to ``DynaFlowManager.initialize``; every later call goes through
``manager.get_callable()``, i.e. split configuration, policy, per-nano-batch dispatch and merge.

The traced module is the tensor-parallel block as a host model would write it::

    x_all = tp_all_gather(x_local)            # world > 1 only
    y     = down(silu(gate(x_all)) * up(x_all))
    y_loc = tp_reduce_scatter(y)              # world > 1 only

The policy (``NanoFlowScheduler``) cuts the MLP and the two collectives into subgraphs of their own,
tags the collectives ``network`` (they run on the communication stream, the reference's
``examples/ae/scheduler/hf/nanoflow.py:123-146``) and substitutes the MLP subgraph by the native
fused kernel with ``func=``. The two collectives are registered PyTorch custom operators whose
implementation launches this library's peer-memory kernels on the current stream; which
micro-batch slot they work on is read from the engine's current operator handle
(``dynaflow/runtime/env.py:48-70``). With ``whole_forward_graph`` the policy runs once per split
shape under stream capture and later steps are one graph launch.
"""
from __future__ import annotations

import contextlib
import io
from typing import Any

import torch

from . import ops
from .config import CUDAGraphConfig, DynaFlowConfig, InductorConfig
from .interface import SplitConfig
from .manager import DynaFlowManager
from .matching import MatchingRule, Op
from .policies import NanoFlowScheduler, gated_mlp_rule
from .runtime.env import get_op_handle

_ACTIVE: "ManagedLayerStep | None" = None


def _slot() -> int:
    handle = get_op_handle()
    if isinstance(handle, tuple):
        handle = handle[0]
    return handle.batch_idx


@torch.library.custom_op("dynaflow_b200::tp_all_gather", mutates_args=())
def tp_all_gather(x: torch.Tensor) -> torch.Tensor:
    """This rank's rows of a micro-batch -> all ranks' rows (rank order), over NVLink."""
    step = _ACTIVE
    assert step is not None and step.comm_in is not None, "no tensor-parallel step is active"
    slot = _slot() % step.layer.micro_batches
    rows = x.shape[0] * step.world
    lo, hi = step.comm_in.slice_bounds(rows)
    step.comm_in.partial(slot, rows)[lo:hi].copy_(x)
    return step.comm_in.all_gather(slot, rows)


@tp_all_gather.register_fake
def _(x: torch.Tensor) -> torch.Tensor:
    world = _ACTIVE.world if _ACTIVE is not None else 1
    return x.new_empty((x.shape[0] * world, x.shape[1]))


@torch.library.custom_op("dynaflow_b200::tp_reduce_scatter", mutates_args=())
def tp_reduce_scatter(y: torch.Tensor) -> torch.Tensor:
    """Every rank's partial sums of a micro-batch -> this rank's rows of their sum."""
    step = _ACTIVE
    assert step is not None and step.layer.comm is not None, "no tensor-parallel step is active"
    slot = _slot() % step.layer.micro_batches
    rows = y.shape[0]
    partial = step.layer.comm.partial(slot, rows)
    if y.data_ptr() != partial.data_ptr():        # the MLP substitute writes there directly; anything else is copied
        partial.copy_(y)
    return step.layer.comm.reduce_scatter(slot, rows).clone()


@tp_reduce_scatter.register_fake
def _(y: torch.Tensor) -> torch.Tensor:
    world = _ACTIVE.world if _ACTIVE is not None else 1
    return y.new_empty((y.shape[0] // world, y.shape[1]))


class _Block(torch.nn.Module):
    """The block as host model code. The weights are this rank's shards (no copy)."""

    def __init__(self, layer: Any, world: int) -> None:
        super().__init__()
        self.world = world
        self.gate_proj = torch.nn.Linear(layer.hidden, layer.shard, bias=False, dtype=torch.bfloat16, device=layer.device)
        self.up_proj = torch.nn.Linear(layer.hidden, layer.shard, bias=False, dtype=torch.bfloat16, device=layer.device)
        self.down_proj = torch.nn.Linear(layer.shard, layer.hidden, bias=False, dtype=torch.bfloat16, device=layer.device)
        self.gate_proj.weight = torch.nn.Parameter(layer.w_gate, requires_grad=False)
        self.up_proj.weight = torch.nn.Parameter(layer.w_up, requires_grad=False)
        self.down_proj.weight = torch.nn.Parameter(layer.w_down, requires_grad=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.world > 1:
            x = torch.ops.dynaflow_b200.tp_all_gather(x)
        y = self.down_proj(torch.nn.functional.silu(self.gate_proj(x)) * self.up_proj(x))
        if self.world > 1:
            y = torch.ops.dynaflow_b200.tp_reduce_scatter(y)
        return y


class ManagedLayerStep:
    """``step(x_local) -> y_local`` through ``DynaFlowManager.get_callable()``.

    ``x_local``: this rank's rows ``[rows / world, hidden]`` on the device (all rows with one rank);
    ``cuts_local``: nano-batch boundaries in those rows. The result is a fresh tensor per call (with
    ``whole_forward_graph`` the graph's output buffer, valid until the next call)."""

    def __init__(self, layer: Any, comm_in: Any = None, whole_forward_graph: bool = True) -> None:
        self.layer, self.comm_in = layer, comm_in
        self.world = layer.world
        config = DynaFlowConfig("dynaflow_b200.policies:NanoFlowScheduler", layer.micro_batches, InductorConfig(False),
                                CUDAGraphConfig(False, [1]),
                                {"min_nano_split_tokens": 1, "whole_forward_graph": whole_forward_graph})
        mlp = gated_mlp_rule()
        gather = MatchingRule(condition=Op(pattern=r"tp_all_gather.*"))
        scatter = MatchingRule(condition=Op(pattern=r"tp_reduce_scatter.*"))
        rules = [mlp] + ([gather, scatter] if self.world > 1 else [])
        tags = {mlp: {"mlp"}}
        if self.world > 1:
            tags[gather] = {"network", "gather"}
            tags[scatter] = {"network", "scatter"}
        self.policy = NanoFlowScheduler(config, split_rules=rules, tag_rules=tags)
        if self.world > 1 and layer.comm is not None:
            self.policy.comm_stream = layer.comm.stream      # the one stream every rank issues its collectives on
        self.policy.substitutions["mlp"] = self._native_mlp
        self.manager = DynaFlowManager()
        self.config = config
        self.block = _Block(layer, self.world)

        def backend(gm, example_inputs):
            self.manager.initialize(graph_module=gm, config=config, scheduler=self.policy,
                                    example_inputs=list(example_inputs))
            return self.manager.get_callable()

        torch._dynamo.reset()
        self.compiled = torch.compile(self.block, backend=backend, fullgraph=True, dynamic=True)

    def _native_mlp(self, x: torch.Tensor, *rest: Any) -> torch.Tensor:
        """``func=`` substitute of the MLP subgraph: its arguments arrive in graph order (activation,
        row count, gate / up / down weights); one persistent launch of the fused kernel into the
        slot's partial-sum buffer (tensor parallel) or a fresh tensor."""
        weights = [a for a in rest if isinstance(a, torch.Tensor)]
        w_gate, w_up, w_down = weights[:3]
        slot = _slot() % self.layer.micro_batches
        rows = x.shape[0]
        out = self.layer.comm.partial(slot, rows) if self.world > 1 else torch.empty_like(x)
        return ops.gated_mlp(x, w_gate, w_up, w_down, out=out, workspace=self.layer.workspaces[slot],
                             max_ctas=self.layer.gemm_max_ctas)

    def __call__(self, x_local: torch.Tensor, cuts_local: list[int]) -> torch.Tensor:
        global _ACTIVE
        _ACTIVE = self
        n = len(cuts_local) - 1
        sizes = [cuts_local[i + 1] - cuts_local[i] for i in range(n)]
        torch._dynamo.mark_dynamic(x_local, 0)
        self.manager.override_split_config(SplitConfig(n, sizes, list(cuts_local), list(sizes), list(sizes), list(cuts_local),
                                                       is_dryrun=False, use_cudagraph=False, allow_fallback=False))
        with torch.inference_mode(), contextlib.redirect_stdout(io.StringIO()):
            return self.compiled(x_local)

    @property
    def substituted_per_step(self) -> int:
        trace = self.manager.engine.last_trace if self.manager.engine is not None else []
        return sum(1 for *_rest, substituted in trace if substituted)
