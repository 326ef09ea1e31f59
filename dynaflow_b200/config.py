"""Configuration objects of the scheduling layer.

Field names, defaults and meaning are those of the reference's
``dynaflow/config.py:6-29`` so that host glue and policy files which build these
objects keep working unchanged.
"""
from __future__ import annotations

import dataclasses
from typing import Any


@dataclasses.dataclass
class CUDAGraphConfig:
    """Per-subgraph CUDA-graph capture (``dynaflow/config.py:6-11``).

    ``capture_sizes`` are the padded row counts a nano-batch may be captured at;
    ``check_ptr_consistency`` makes a replay verify that the input tensors still
    live at the captured addresses. ``weak_ref_output`` is accepted for
    compatibility; captured outputs are always owned by the capture entry here.

    ``copy_mismatched_inputs`` (not in the reference) turns the pointer check into a
    repair: an input that arrives at another address than the captured one -- the
    output of an eagerly executed or substituted subgraph -- is copied into the
    captured input before the replay instead of raising.
    """

    enabled: bool
    capture_sizes: list[int]
    weak_ref_output: bool = True
    check_ptr_consistency: bool = True
    copy_mismatched_inputs: bool = False


@dataclasses.dataclass
class InductorConfig:
    """TorchInductor settings (``dynaflow/config.py:14-20``).

    This backend has no Triton/Inductor code path. The object is kept so that
    hosts can construct it; ``enabled=True`` is accepted and ignored with a
    one-time warning (subgraphs run as traced, hot operators are substituted by
    the native kernels instead).
    """

    enabled: bool
    compile_sizes: set[int] | None = None
    options: dict | None = None
    disable_remote_cache: bool = True
    disable_autograd_cache: bool = True


@dataclasses.dataclass
class DynaFlowConfig:
    """Top-level configuration (``dynaflow/config.py:23-29``).

    ``scheduler_path`` is ``"file.py:ClassName"`` of the policy, ``max_num_splits``
    bounds the number of nano-batches, ``additional_config`` carries
    policy-private keys (``min_nano_split_tokens`` and the like).
    """

    scheduler_path: str
    max_num_splits: int
    inductor_config: InductorConfig
    cudagraph_config: CUDAGraphConfig
    additional_config: dict[str, Any] = dataclasses.field(default_factory=dict)
