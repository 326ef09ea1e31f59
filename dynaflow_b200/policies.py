"""Scheduling policies shipped with the backend.

They restate the reference's example policies (``examples/ae/scheduler/``) without
any dependency on a serving framework, so that they run on any traced model:

* ``NanoFlowScheduler``: balanced two-way split at a request boundary and a
  round-robin schedule that sends ``network``-tagged subgraphs to a communication
  stream (``hf/nanoflow.py:66-146``, ``vllm/nanoflow.py:98-151``);
* ``EqualSplitScheduler``: n-way equal split with a one-operator skew of
  nano-batch 0 (``megatron/nanoflow.py:43-102``).

Subclasses supply the split / tag rules for their model, and may substitute
subgraphs by native kernels through ``substitutions`` (tag -> callable).
"""
from __future__ import annotations

import contextlib
import itertools
from collections.abc import Callable
from typing import Any

import torch

from .config import DynaFlowConfig
from .interface import ExecutionContext, InputInfo, OperatorHandle, OpSchedulerBase, SplitConfig
from .matching import MatchingRule
from .utils import pack_tokens


def gated_mlp_rule() -> MatchingRule:
    """Matches a Hugging Face style gated MLP as ONE subgraph: gate linear, SiLU, up
    linear, product, down linear, in the order Dynamo traces
    ``down_proj(act_fn(gate_proj(x)) * up_proj(x))``."""
    from .matching import Op

    return MatchingRule(condition=(Op("linear"), Op("silu"), Op("linear"), Op("mul"), Op("linear")))


def native_gated_mlp(x: torch.Tensor, rows: Any, w_gate: torch.Tensor, w_up: torch.Tensor,
                     w_down: torch.Tensor) -> torch.Tensor:
    """Substitute for the subgraph cut by ``gated_mlp_rule``: its arguments arrive in
    graph order (activation, row count, gate / up / down weights in ``nn.Linear``
    layout). Runs the fused sm_100a kernels on the current stream."""
    from . import ops

    flat = x.reshape(-1, x.shape[-1])
    if not flat.is_contiguous():
        flat = flat.contiguous()
    return ops.gated_mlp(flat, w_gate, w_up, w_down).view(*x.shape[:-1], w_down.shape[0])


def _make_stream() -> Any:
    return torch.cuda.Stream() if torch.cuda.is_available() else None


def _on(stream: Any):
    return torch.cuda.stream(stream) if stream is not None else contextlib.nullcontext()


class _StreamedPolicy(OpSchedulerBase):
    """Common part: two streams, rule tables, tag-driven substitution."""

    def __init__(self, config: DynaFlowConfig, policy_name: str,
                 split_rules: list[MatchingRule] | None = None,
                 tag_rules: dict[MatchingRule, set[str]] | None = None) -> None:
        super().__init__(policy_name=policy_name)
        self.config = config
        self.comm_stream = _make_stream()
        self.comp_stream = _make_stream()
        self._split_rules = list(split_rules or [])
        self._tag_rules = dict(tag_rules or {})
        # tag -> func(*subgraph_args); the first tag of an operator found here wins
        self.substitutions: dict[str, Callable[..., Any]] = {}

    def get_split_rules(self) -> list[MatchingRule]:
        return self._split_rules

    def get_tag_rules(self) -> dict[MatchingRule, set[str]]:
        return self._tag_rules

    def _stream_for(self, op: OperatorHandle) -> Any:
        return self.comm_stream if "network" in op.tag else self.comp_stream

    def _func_for(self, op: OperatorHandle) -> Callable[..., Any] | None:
        for tag, func in self.substitutions.items():
            if tag in op.tag:
                return func
        return None

    async def _run(self, context: ExecutionContext, op: OperatorHandle) -> None:
        with _on(self._stream_for(op)):
            await context.execute((op,), self._func_for(op))


class NanoFlowScheduler(_StreamedPolicy):
    def __init__(self, config: DynaFlowConfig, split_rules: list[MatchingRule] | None = None,
                 tag_rules: dict[MatchingRule, set[str]] | None = None) -> None:
        super().__init__(config, "nanoflow", split_rules, tag_rules)
        self.min_nano_split_tokens = config.additional_config["min_nano_split_tokens"]
        self.max_num_nano_batches = config.max_num_splits
        self.cudagraph_capture_sizes = config.cudagraph_config.capture_sizes

    def get_split_config(self, input_info: InputInfo, use_cudagraph: bool) -> SplitConfig:
        sizes = self.cudagraph_capture_sizes
        prefix = list(itertools.accumulate(input_info.num_tokens, initial=0))
        total = prefix[-1]
        mid = min(range(len(prefix)), key=lambda i: abs(2 * prefix[i] - total))
        left, right = prefix[mid], total - prefix[mid]
        if min(left, right) < self.min_nano_split_tokens:
            padded = total
            if use_cudagraph:
                padded, use_cudagraph = pack_tokens(total, sizes)
            return SplitConfig(1, [input_info.batch_size], [0, input_info.batch_size], [total], [padded],
                               [0, total], is_dryrun=False, use_cudagraph=use_cudagraph)
        padded_pair = [left, right]
        if use_cudagraph:
            packed = [pack_tokens(n, sizes) for n in padded_pair]
            if all(fits for _, fits in packed):
                padded_pair = [p for p, _ in packed]
            else:
                use_cudagraph = False
        return SplitConfig(2, [mid, input_info.batch_size - mid], [0, mid, input_info.batch_size], [left, right],
                           padded_pair, [0, left, total], is_dryrun=False, use_cudagraph=use_cudagraph)

    async def schedule(self, context: ExecutionContext) -> None:
        live = list(range(context.split_config.num_nano_batches))
        while live:
            round_ops: list[OperatorHandle] = []
            for b in live:  # removal while iterating skips the next entry for this round, as in the reference
                op = await context.pop(b)
                if op is None:
                    live.remove(b)
                else:
                    round_ops.append(op)
            for op in round_ops:
                await self._run(context, op)


class EqualSplitScheduler(_StreamedPolicy):
    def __init__(self, config: DynaFlowConfig, split_rules: list[MatchingRule] | None = None,
                 tag_rules: dict[MatchingRule, set[str]] | None = None) -> None:
        super().__init__(config, "nanoflow-equal", split_rules, tag_rules)
        self.num_nano_batches = config.additional_config.get("num_nano_batches", 2)
        self.min_nano_split_tokens = config.additional_config.get("min_nano_split_tokens", 1)

    def get_split_config(self, input_info: InputInfo, use_cudagraph: bool = False) -> SplitConfig:
        rows = input_info.batch_size
        n = self.num_nano_batches
        chunk = rows // n
        if chunk < self.min_nano_split_tokens:
            n = max(1, rows // self.min_nano_split_tokens)
            chunk = rows // n if n > 1 else rows
        if n <= 1:
            return SplitConfig(1, [rows], [0, rows], [rows], [rows], [0, rows], is_dryrun=False,
                               use_cudagraph=use_cudagraph)
        sizes = [chunk] * (n - 1) + [rows - chunk * (n - 1)]
        cuts = [chunk * i for i in range(n)] + [rows]
        return SplitConfig(n, sizes, cuts, list(sizes), list(sizes), list(cuts), is_dryrun=False,
                           use_cudagraph=use_cudagraph)

    async def schedule(self, context: ExecutionContext) -> None:
        live = list(range(context.split_config.num_nano_batches))
        if len(live) >= 2:
            # skew: nano-batch 0 runs one operator ahead so that its communication
            # falls under nano-batch 1's computation from then on
            op = await context.pop(0)
            if op is None:
                live.remove(0)
            else:
                await self._run(context, op)
        while live:
            for b in list(live):
                op = await context.pop(b)
                if op is None:
                    live.remove(b)
                else:
                    await self._run(context, op)


def agree_on_split(split_config: SplitConfig, batch_size: int, group: Any = None) -> tuple[SplitConfig, list[list[int]]]:
    """Cross-rank agreement on the nano-batch split for data-parallel ranks that meet in a
    collective inside the forward (expert parallelism): if any rank decided not to split, no
    rank splits, since all ranks must issue the same number of collectives
    (``examples/ae/patch/vllm.patch:598-632``). Host-side, CPU objects only.

    Returns the possibly downgraded config and, per nano-batch, the padded row count of
    every rank (what the reference packs into ``DPMetadata``, ``vllm.patch:634-664``)."""
    import torch.distributed as dist

    if not dist.is_available() or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return split_config, [[n] for n in split_config.num_tokens_padded]
    world = dist.get_world_size(group)
    configs: list[Any] = [None] * world
    dist.all_gather_object(configs, split_config, group=group)
    if any(c.num_nano_batches == 1 for c in configs) and split_config.num_nano_batches != 1:
        total, padded = sum(split_config.num_tokens), sum(split_config.num_tokens_padded)
        split_config = SplitConfig(1, [batch_size], [0, batch_size], [total], [padded], [0, total],
                                   is_dryrun=split_config.is_dryrun, use_cudagraph=False)
    if any(c.num_nano_batches == 1 for c in configs):
        dist.all_gather_object(configs, split_config, group=group)
    rows = [[c.num_tokens_padded[i] for c in configs] for i in range(split_config.num_nano_batches)]
    return split_config, rows


class DBOScheduler(_StreamedPolicy):
    """Dual-batch overlap for MoE layers: a hand-written interleaving that puts the dispatch and
    combine all-to-alls of one nano-batch under the attention and expert GEMMs of the other
    (``examples/ae/scheduler/vllm/dbo.py``). Framework-free restatement: subgraphs are recognised
    by the tags ``attention`` / ``dispatch`` / ``expert`` / ``combine`` that the subclass's tag
    rules assign; ``network``-tagged operators go to the communication stream.
    ``before_execute(batch_idx, op)`` is called ahead of every operator, for hosts that keep
    per-nano-batch state (attention / data-parallel metadata) in a global context
    (``dbo.py:213-217``)."""

    WARM_UP = (("attention", 0),)
    SEQUENCE = (("attention", 1), ("dispatch", 0), ("expert", 0), ("dispatch", 1), ("expert", 1),
                ("combine", 0), ("attention", 0), ("combine", 1))

    def __init__(self, config: DynaFlowConfig, split_rules: list[MatchingRule] | None = None,
                 tag_rules: dict[MatchingRule, set[str]] | None = None) -> None:
        super().__init__(config, "dbo", split_rules, tag_rules)
        self.min_nano_split_tokens = config.additional_config["min_nano_split_tokens"]
        self.max_num_nano_batches = config.max_num_splits
        self.cudagraph_capture_sizes = config.cudagraph_config.capture_sizes
        self._splitter = NanoFlowScheduler.get_split_config  # same balanced two-way split (dbo.py:94-148)

    def get_split_config(self, input_info: InputInfo, use_cudagraph: bool) -> SplitConfig:
        return self._splitter(self, input_info, use_cudagraph)  # type: ignore[arg-type]

    def before_execute(self, batch_idx: int, op: OperatorHandle) -> None:
        """Hook for hosts; does nothing by default."""

    async def schedule(self, context: ExecutionContext) -> None:
        n = context.split_config.num_nano_batches
        if n == 1:
            self.before_execute(0, None)  # type: ignore[arg-type]
            while (op := await context.pop(0)) is not None:
                await context.execute((op,), self._func_for(op))
            return
        ordered = {kind for kind, _ in self.SEQUENCE}
        live = list(range(n))
        turn_of = list(self.WARM_UP)          # whose turn it is, and for which kind of operator
        position = -len(self.WARM_UP)
        current = live[0]
        held: list[OperatorHandle | None] = [None] * n
        while live:
            if held[current] is not None:
                op, held[current] = held[current], None
            else:
                op = await context.pop(current)
                if op is None:                 # this nano-batch is done: the other one takes the next turn
                    live.remove(current)
                    current ^= 1
                    position += 1
                    continue
                if not ordered.intersection(op.tag):
                    with _on(self.comp_stream):
                        await context.execute((op,), self._func_for(op))
                    continue
                if turn_of[position][1] != current:
                    held[current] = op          # too early: hold it, let the other nano-batch catch up
                    current ^= 1
                    continue
            assert turn_of[position][0] in op.tag, f"expected a {turn_of[position][0]} operator, got {op.tag}"
            position += 1
            if position > 0:
                position %= len(self.SEQUENCE)
            elif position == 0:
                turn_of = list(self.SEQUENCE)
            self.before_execute(current, op)
            await self._run(context, op)
