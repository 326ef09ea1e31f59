"""CUDA-graph capture and replay of one subgraph, keyed by nano-batch and padded size.

Contract of the reference's ``dynaflow/executor/cudagraph.py:68-123``: outside
CUDA-graph mode the wrapper is transparent; the first time a (size, nano-batch)
pair is seen must be a dry run, which captures into the memory pool of that
nano-batch index; later calls check that inputs still live at the captured
addresses (``RuntimeError`` otherwise), replay, and return the captured outputs.

Differences: with ``CUDAGraphConfig.copy_mismatched_inputs`` a moved input is copied
into its captured location instead of raising; captured outputs are held by the entry itself instead of through
vLLM's ``weak_ref_tensor`` custom op (``cudagraph.py:37-65``), so no third-party
extension is needed; pools are keyed per nano-batch index exactly as in
``cudagraph.py:11-31`` and an optional hook lets a host share them with its
communication library.
"""
from __future__ import annotations

from collections.abc import Callable
from typing import Any

import torch

from ..config import CUDAGraphConfig
from ..interface import OperatorHandle
from ..runtime.env import get_op_handle


class CUDAGraphPool:
    """One graph memory pool per nano-batch index, created on first use."""

    def __init__(self) -> None:
        self.pools: dict[int, Any] = {}
        self.on_pool_selected: Callable[[Any], None] | None = None

    def get_pool(self, key: int) -> Any:
        pool = self.pools.get(key)
        if pool is None:
            pool = torch.cuda.graph_pool_handle()
            self.pools[key] = pool
        if self.on_pool_selected is not None:
            self.on_pool_selected(pool)
        return pool


_global_pool = CUDAGraphPool()


def _tensor_addresses(args: tuple) -> list[int]:
    return [a.data_ptr() for a in args if isinstance(a, torch.Tensor)]


class CUDAGraphWrapper:
    def __init__(self, runnable: Callable[..., Any], config: CUDAGraphConfig) -> None:
        self.runnable = runnable
        self.config = config
        self._entries: dict[tuple[int, int, int], dict[str, Any]] = {}

    def __call__(self, *args: Any, **kwargs: Any) -> Any:
        handle = get_op_handle()
        if not isinstance(handle, OperatorHandle) or not handle._use_cudagraph:
            return self.runnable(*args, **kwargs)

        key = (handle.batch_size, handle.batch_idx, handle.batch_size)
        entry = self._entries.get(key)
        if entry is None:
            if not handle._is_dryrun:
                raise AssertionError(
                    f"no CUDA graph captured for {handle.module_name} at size {handle.batch_size} "
                    f"(nano-batch {handle.batch_idx}); capture needs a dry run first")
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, pool=_global_pool.get_pool(handle.batch_idx)):
                out = self.runnable(*args, **kwargs)
            self._entries[key] = {"graph": graph, "out": out, "inputs": _tensor_addresses(args),
                                  "static_inputs": [a for a in args if isinstance(a, torch.Tensor)]}
            return out

        if getattr(self.config, "copy_mismatched_inputs", False):
            live = [a for a in args if isinstance(a, torch.Tensor)]
            for captured, new in zip(entry["static_inputs"], live):
                if captured.data_ptr() != new.data_ptr():
                    captured.copy_(new)  # on the current stream, ahead of the replay
        elif self.config.check_ptr_consistency and _tensor_addresses(args) != entry["inputs"]:
            raise RuntimeError("CUDAGraph input addresses changed between capture and replay")
        entry["graph"].replay()
        return entry["out"]
