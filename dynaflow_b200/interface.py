"""Policy-facing API: split descriptors, operator handles, the execution context
and the scheduler base class.

Names and argument meaning follow the reference's ``dynaflow/interface.py`` so
that policy files run unmodified. The machinery underneath differs: ``pop`` and
``execute`` do not go through asyncio queues to a second coroutine; they call
straight into the engine's micro-batch dispatcher and complete without
suspending, so a policy coroutine is driven by a single ``send`` and costs no
event-loop round trip per operator.
"""
from __future__ import annotations

import abc
import dataclasses
from collections.abc import Callable
from typing import TYPE_CHECKING, Any

from .matching import MatchingRule

if TYPE_CHECKING:  # pragma: no cover
    from .runtime.engine import NanoBatchDispatcher


@dataclasses.dataclass
class InputInfo:
    """What a policy sees of the next batch (``dynaflow/interface.py:9-21``):
    number of requests, rows (tokens) per request, and their sum."""

    batch_size: int
    num_tokens: list[int]
    total_num_tokens: int


@dataclasses.dataclass
class SplitConfig:
    """How the next forward is cut into nano-batches (``dynaflow/interface.py:24-52``).

    ``batch_indices`` cuts the request axis and ``split_indices`` the row axis
    (dim 0 of every dynamic input); both have ``num_nano_batches + 1`` entries.
    ``num_tokens_padded[i]`` is the row count nano-batch ``i`` executes with
    (>= ``num_tokens[i]`` when padded up to a capture size). With
    ``allow_fallback`` a single nano-batch bypasses the policy entirely.
    """

    num_nano_batches: int
    batch_sizes: list[int]
    batch_indices: list[int]
    num_tokens: list[int]
    num_tokens_padded: list[int]
    split_indices: list[int]
    is_dryrun: bool
    use_cudagraph: bool
    allow_fallback: bool = True


@dataclasses.dataclass(eq=False, frozen=True)
class OperatorHandle:
    """One subgraph of one nano-batch, as handed to a policy
    (``dynaflow/interface.py:55-73``). Compared by identity."""

    module_name: str
    batch_idx: int
    batch_size: int
    tag: set[str]
    _is_dryrun: bool
    _use_cudagraph: bool


class ExecutionContext:
    """The object a policy's ``schedule`` coroutine drives
    (``dynaflow/interface.py:76-127``)."""

    def __init__(self, split_config: SplitConfig, dispatcher: "NanoBatchDispatcher") -> None:
        self._split_config = split_config
        self._dispatcher = dispatcher

    @property
    def split_config(self) -> SplitConfig:
        return self._split_config

    async def pop(self, batch_idx: int) -> OperatorHandle | None:
        """Next ready operator of nano-batch ``batch_idx`` in program order, or
        ``None`` once that nano-batch has produced its output."""
        return self._dispatcher.pop(batch_idx)

    async def execute(self, operator: OperatorHandle | tuple[OperatorHandle, ...],
                      func: Callable[..., Any] | None = None) -> None:
        """Runs the operator on the CUDA stream that is current in the caller.
        With ``func`` the subgraph is replaced: ``func`` receives the subgraph's
        tensor arguments in graph order and must return the same structure."""
        ops = operator if isinstance(operator, tuple) else (operator,)
        self._dispatcher.execute(ops, func)


class OpSchedulerBase(abc.ABC):
    """Base class of scheduling policies (``dynaflow/interface.py:130-156``)."""

    def __init__(self, policy_name: str | None = None) -> None:
        self.policy_name = policy_name

    @abc.abstractmethod
    def get_split_rules(self) -> list[MatchingRule]:
        """Rules whose matches become subgraphs of their own (cut-around)."""

    @abc.abstractmethod
    def get_tag_rules(self) -> dict[MatchingRule, set[str]]:
        """Rule -> tags added to every subgraph the rule matches inside."""

    @abc.abstractmethod
    def get_split_config(self, input_info: InputInfo, use_cudagraph: bool) -> SplitConfig:
        """Decides the nano-batch split of the next forward."""

    @abc.abstractmethod
    async def schedule(self, context: ExecutionContext) -> None:
        """Pops ready operators and executes them in the order and on the
        streams the policy chooses."""
