"""Per-nano-batch value store with reference counting, and the "current operator" slot.

Mirrors the contract of the reference's ``dynaflow/runtime/env.py``: a value is
stored together with the number of graph users of its node and dropped when the
last user has fetched it (``env.py:10-46``); ``get_op_handle`` / ``set_op_handle``
expose which operator is executing to the subgraph back-ends (``env.py:48-70``).
"""
from __future__ import annotations

import contextlib
from collections.abc import Iterator
from typing import Any

import torch.fx

from ..interface import OperatorHandle


class ActivationBuffer:
    """A produced value and how many consumers have yet to read it."""

    __slots__ = ("data", "ref_count")

    def __init__(self, data: Any, ref_count: int) -> None:
        self.data = data
        self.ref_count = ref_count

    def get_ref(self) -> Any:
        value = self.data
        self.ref_count -= 1
        if self.ref_count == 0:
            self.data = None  # last consumer: let the activation be freed
        return value


class ExecutionEnvironment:
    """``env[batch_idx][node]`` -> ``ActivationBuffer``."""

    def __init__(self, num_nano_batches: int) -> None:
        self.env: list[dict[torch.fx.Node, ActivationBuffer]] = [dict() for _ in range(num_nano_batches)]

    def put(self, batch_idx: int, node: torch.fx.Node, data: Any) -> None:
        self.env[batch_idx][node] = ActivationBuffer(data, len(node.users))

    def get(self, batch_idx: int, node: torch.fx.Node) -> Any:
        value = self.env[batch_idx][node].get_ref()
        assert value is not None, f"value of {node.name} was already released"
        return value


_current_op_handle: OperatorHandle | tuple[OperatorHandle, ...] | None = None


def get_op_handle() -> OperatorHandle | tuple[OperatorHandle, ...]:
    """The operator being executed; only valid inside ``set_op_handle``."""
    assert _current_op_handle is not None, "no operator is executing"
    return _current_op_handle


@contextlib.contextmanager
def set_op_handle(handle: OperatorHandle | tuple[OperatorHandle, ...]) -> Iterator[None]:
    global _current_op_handle
    saved = _current_op_handle
    _current_op_handle = handle
    try:
        yield
    finally:
        _current_op_handle = saved
