"""Wraps every subgraph of a split model in a ``SubgraphBackend``.

Same contract as the reference's ``dynaflow/executor/compiler.py``: the split
graph is interpreted once on fake tensors to find, for each subgraph call, the
first argument that is a ``torch.SymInt`` (the dynamic row count,
``compiler.py:126-150``); the subgraph module is then replaced in the parent's
``__dict__`` by a backend object that dispatches on that size at call time
(``compiler.py:69-85``).

There is no TorchInductor path here (``compiler.py:58-66`` would call it): the
``use_inductor`` flag is accepted and the subgraph runs as traced. Hot operators
reach the native kernels through policy substitution (``func=``) instead.
"""
from __future__ import annotations

import warnings
from collections.abc import Callable
from typing import Any

import torch
import torch.fx as fx

from ..config import CUDAGraphConfig, DynaFlowConfig, InductorConfig
from ..interface import OperatorHandle
from ..runtime.env import get_op_handle
from .cudagraph import CUDAGraphWrapper

_warned_inductor = False


def _warn_inductor_once() -> None:
    global _warned_inductor
    if not _warned_inductor:
        _warned_inductor = True
        warnings.warn("InductorConfig.enabled is ignored: dynaflow_b200 has no Triton/Inductor path; "
                      "subgraphs run as traced and hot operators use the native sm_100a kernels",
                      stacklevel=3)


class SubgraphBackend:
    """Callable stand-in for one subgraph module."""

    def __init__(self, subgraph_gm: fx.GraphModule, shape_arg_index: int, inductor_config: InductorConfig,
                 cudagraph_config: CUDAGraphConfig, *, use_inductor: bool, use_cudagraph: bool) -> None:
        assert not use_inductor or inductor_config.enabled
        assert not use_cudagraph or cudagraph_config.enabled
        self.gm = subgraph_gm
        tag = getattr(subgraph_gm, "tag", set())
        assert isinstance(tag, set)
        self.tag: set[str] = tag
        self.shape_arg_index = shape_arg_index
        self.inductor_config = inductor_config
        self.cudagraph_config = cudagraph_config
        self.use_inductor = use_inductor
        self.use_cudagraph = use_cudagraph
        self.callable_dynamic: Callable[..., Any] | None = None
        self.callables_per_size: dict[int, Callable[..., Any]] = {}
        if use_inductor:
            _warn_inductor_once()

    def compile(self, example_inputs: list[Any], runtime_shape: int | None = None) -> Callable[..., Any]:
        """Returns the callable for a dynamic (``runtime_shape is None``) or fixed row count."""
        shape = example_inputs[self.shape_arg_index]
        if runtime_shape is None:
            assert isinstance(shape, (torch.SymInt, int))
        else:
            assert int(shape) == runtime_shape
        fn: Callable[..., Any] = self.gm
        return CUDAGraphWrapper(fn, self.cudagraph_config) if self.use_cudagraph else fn

    def __call__(self, *args: Any, **kwargs: Any) -> Any:
        assert self.shape_arg_index < len(args)
        size = int(args[self.shape_arg_index])
        fixed = self.inductor_config.compile_sizes
        if fixed is not None and size in fixed:
            fn = self.callables_per_size.get(size)
            if fn is None:
                handle = get_op_handle()
                assert isinstance(handle, OperatorHandle) and handle._is_dryrun, \
                    "a size-specific callable can only be created during a dry run"
                fn = self.callables_per_size[size] = self.compile(list(args), size)
            return fn(*args, **kwargs)
        assert self.callable_dynamic is not None
        return self.callable_dynamic(*args, **kwargs)


class SubgraphCompiler(fx.Interpreter):
    """Fake-tensor interpretation of the split graph that installs the back-ends."""

    def __init__(self, module: fx.GraphModule, config: DynaFlowConfig, *, inductor_compile_targets: list[str],
                 cudagraph_targets: list[str]) -> None:
        super().__init__(module)
        from torch._guards import detect_fake_mode

        self.config = config
        self.inductor_compile_targets = set(inductor_compile_targets)
        self.cudagraph_targets = set(cudagraph_targets)
        self.fake_mode = detect_fake_mode()

    def run(self, *args: Any, initial_env: dict[fx.Node, Any] | None = None,
            enable_io_processing: bool = True) -> Any:
        if self.fake_mode is None:
            raise AssertionError("SubgraphCompiler must run inside a torch.compile backend "
                                 "(no fake-tensor mode is active)")
        from torch._dispatch.python import enable_python_dispatcher

        fake_args = [self.fake_mode.from_tensor(a) if isinstance(a, torch.Tensor) else a for a in args]
        with self.fake_mode, enable_python_dispatcher():
            return super().run(*fake_args)

    def call_module(self, target: Any, args: tuple, kwargs: dict) -> Any:
        assert isinstance(target, str)
        result = super().call_module(target, args, kwargs)
        submodule = self.fetch_attr(target)
        assert isinstance(submodule, fx.GraphModule)
        shape_index = next((i for i, a in enumerate(args) if isinstance(a, torch.SymInt)), None)
        # every subgraph must receive the dynamic row count, i.e. dim 0 of the
        # model inputs has to be marked dynamic before tracing
        assert shape_index is not None, f"subgraph {target} receives no torch.SymInt argument"
        backend = SubgraphBackend(submodule, shape_index, self.config.inductor_config, self.config.cudagraph_config,
                                  use_inductor=target in self.inductor_compile_targets,
                                  use_cudagraph=target in self.cudagraph_targets)
        backend.callable_dynamic = backend.compile(list(args))
        self.module.__dict__[target] = backend
        return result
