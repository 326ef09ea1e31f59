"""Micro-batch dispatch engine.

Executes a split FX graph once per nano-batch, interleaved in the order a policy
chooses. Observable behaviour follows the reference's
``dynaflow/runtime/engine.py``:

* dynamic inputs (dim 0 symbolic) are sliced ``[split_indices[b]:split_indices[b+1]]``
  per nano-batch, static-shape inputs are passed whole, and a ``SymInt`` input
  equal to the padded total becomes the nano-batch's padded row count
  (``engine.py:436-479``);
* operators of one nano-batch run strictly in program order, ordered across
  streams by one CUDA event per nano-batch (``engine.py:302-303, 383-389``);
* a substitute ``func`` receives the subgraph's node arguments in graph order
  (``engine.py:304-325``); grouping several operators in one ``execute`` is not
  implemented (``engine.py:321-329``);
* a single nano-batch with ``allow_fallback`` bypasses the policy
  (``engine.py:179-220``); a dry run replays the graph once per nano-batch slot
  to capture CUDA graphs on static input buffers (``engine.py:81-177``).

What is different underneath. The reference runs engine and policy as two
asyncio coroutines that hand every operator across two queues. Here the top-level
graph is lowered once into a flat step list, and ``ExecutionContext.pop`` /
``execute`` call straight into a ``NanoBatchDispatcher``: ready operators are
computed on demand and executed inline on the caller's current stream, so the
policy coroutine never suspends and is driven by one ``send`` (a policy that
awaits other things runs on an event loop when
``additional_config['policy_uses_event_loop']`` is set). A policy that
would stall the reference's loop forever (popping past a non-operator node with
work outstanding, executing out of order, returning early) raises instead.
Each nano-batch slot owns its static input buffers (the reference aliases one
dict across slots, ``engine.py:40``, so two live nano-batches overwrite each
other's inputs under CUDA graphs).
"""
from __future__ import annotations

from collections.abc import Callable
from typing import Any

import torch
import torch.fx

from ..config import DynaFlowConfig
from ..interface import ExecutionContext, OperatorHandle, OpSchedulerBase, SplitConfig
from .env import ExecutionEnvironment, set_op_handle

# step kinds of the lowered top-level program
_PLACEHOLDER, _GET_ATTR, _CALL_FUNCTION, _CALL_METHOD, _CALL_MODULE, _OUTPUT = range(6)
# placeholder kinds: not one / static-shape value (weights) / tensor split by rows / symbolic row count
_PH_NONE, _PH_STATIC, _PH_ROWS, _PH_SYMINT = range(4)
_KIND = {"placeholder": _PLACEHOLDER, "get_attr": _GET_ATTR, "call_function": _CALL_FUNCTION,
         "call_method": _CALL_METHOD, "call_module": _CALL_MODULE, "output": _OUTPUT}


class _NullEvent:
    """Stands in for ``torch.cuda.Event`` when the graph runs on CPU tensors
    (host-logic tests); ordering is then the program order of the one thread."""

    def record(self, stream: Any = None) -> None:
        pass

    def wait(self, stream: Any = None) -> None:
        pass

    def synchronize(self) -> None:
        pass


def _new_event() -> Any:
    if torch.cuda.is_available():
        return torch.cuda.Event()
    return _NullEvent()


def _current_stream_id() -> int:
    if torch.cuda.is_available():
        return torch.cuda.current_stream().cuda_stream
    return 0


class _Step:
    __slots__ = ("kind", "node", "target", "placeholder_idx", "placeholder_kind")

    def __init__(self, node: torch.fx.Node, placeholder_idx: int) -> None:
        if node.op not in _KIND:
            raise ValueError(f"Invalid node operation: {node.op}")
        self.kind = _KIND[node.op]
        self.node = node
        self.target = node.target
        self.placeholder_idx = placeholder_idx
        # what a placeholder is, decided once from its traced example value (a decoder's weights are
        # placeholders too: hundreds of them per forward and nano-batch)
        self.placeholder_kind = _PH_NONE
        if node.op == "placeholder":
            example = node.meta.get("example_value", None)
            if isinstance(example, torch.Tensor):
                dynamic = example.dim() > 0 and isinstance(example.shape[0], torch.SymInt)
                self.placeholder_kind = _PH_ROWS if dynamic else _PH_STATIC
            elif isinstance(example, torch.SymInt):
                self.placeholder_kind = _PH_SYMINT


class DynaFlowEngine:
    """Holds the lowered program of one split graph and runs forwards over it."""

    def __init__(self, graph_module: torch.fx.GraphModule, config: DynaFlowConfig) -> None:
        self.graph_module = graph_module
        self.config = config
        self.max_static_rows: int = int(config.additional_config.get("max_static_rows", 16384))
        # static input buffers for CUDA-graph mode: one dict per nano-batch slot
        self.input_buffers: list[dict[int, torch.Tensor]] = [dict() for _ in range(config.max_num_splits)]

        self.placeholder_nodes: list[torch.fx.Node] = []
        self.placeholder_node_to_idx: dict[torch.fx.Node, int] = {}
        self.module_name_to_node: dict[str, torch.fx.Node] = {}
        self.get_attr_cache: dict[str, Any] = {}
        self.steps: list[_Step] = []
        for node in graph_module.graph.nodes:
            idx = -1
            if node.op == "placeholder":
                idx = len(self.placeholder_nodes)
                self.placeholder_nodes.append(node)
                self.placeholder_node_to_idx[node] = idx
            elif node.op == "call_module":
                assert isinstance(node.target, str)
                self.module_name_to_node[node.target] = node
            elif node.op == "get_attr":
                assert isinstance(node.target, str)
                self.get_attr_cache[node.target] = getattr(graph_module, node.target)
            self.steps.append(_Step(node, idx))
        # (module_name, batch_idx, stream id, substituted) of the most recent split forward
        self.last_trace: list[tuple[str, int, int, bool]] = []

    # ------------------------------------------------------------------ inputs
    def allocate_input_buffer(self, batch_idx: int, placeholder_idx: int, num_tokens: int,
                              example_value: torch.Tensor) -> None:
        if self.input_buffers[batch_idx].get(placeholder_idx) is None:
            self.input_buffers[batch_idx][placeholder_idx] = torch.zeros(
                (num_tokens,) + tuple(example_value.shape[1:]), dtype=example_value.dtype,
                device=example_value.device)

    def _bind_placeholder(self, step: _Step, batch_idx: int, args: tuple, env: ExecutionEnvironment,
                          cfg: SplitConfig) -> None:
        node, idx = step.node, step.placeholder_idx
        kind = step.placeholder_kind
        if kind == _PH_STATIC:
            env.put(batch_idx, node, args[idx])  # weights and other static-shape inputs
        elif kind == _PH_ROWS:
            start, stop = cfg.split_indices[batch_idx], cfg.split_indices[batch_idx + 1]
            if cfg.use_cudagraph:
                buf = self.input_buffers[batch_idx].get(idx)
                assert buf is not None, "CUDA-graph mode needs a dry run to allocate the static input buffers"
                buf[:cfg.num_tokens[batch_idx]].copy_(args[idx][start:stop])
                env.put(batch_idx, node, buf[:cfg.num_tokens_padded[batch_idx]])
            else:
                env.put(batch_idx, node, args[idx][start:stop])
        elif kind == _PH_SYMINT:
            if args[idx] == sum(cfg.num_tokens_padded):
                env.put(batch_idx, node, cfg.num_tokens_padded[batch_idx])
            else:
                env.put(batch_idx, node, args[idx])
        else:
            raise ValueError(f"Invalid example value type: {type(node.meta.get('example_value', None))}")

    def _run_simple_step(self, step: _Step, batch_idx: int, args: tuple, env: ExecutionEnvironment,
                         cfg: SplitConfig) -> None:
        """Everything that is not a subgraph call or the output."""
        node = step.node
        if step.kind == _PLACEHOLDER:
            self._bind_placeholder(step, batch_idx, args, env, cfg)
        elif step.kind == _GET_ATTR:
            env.put(batch_idx, node, self.get_attr_cache[step.target])
        elif step.kind == _CALL_FUNCTION:
            assert callable(step.target)
            a = [env.get(batch_idx, x) if isinstance(x, torch.fx.Node) else x for x in node.args]
            kw = {k: env.get(batch_idx, v) if isinstance(v, torch.fx.Node) else v for k, v in node.kwargs.items()}
            env.put(batch_idx, node, step.target(*a, **kw))
        elif step.kind == _CALL_METHOD:
            assert isinstance(step.target, str)
            obj = env.get(batch_idx, node.args[0])
            a = [env.get(batch_idx, x) if isinstance(x, torch.fx.Node) else x for x in node.args[1:]]
            kw = {k: env.get(batch_idx, v) if isinstance(v, torch.fx.Node) else v for k, v in node.kwargs.items()}
            env.put(batch_idx, node, getattr(obj, step.target)(*a, **kw))
        else:
            raise ValueError(f"Invalid node operation: {node.op}")

    @staticmethod
    def _collect_output(node: torch.fx.Node, batch_idx: int, env: ExecutionEnvironment) -> Any:
        out = node.args[0]
        if isinstance(out, torch.fx.Node):
            return env.get(batch_idx, out)
        if isinstance(out, (tuple, list)):
            return tuple(env.get(batch_idx, x) if isinstance(x, torch.fx.Node) else x for x in out)
        return out

    # ----------------------------------------------------------------- dry run
    def dryrun(self, args: tuple, kwargs: dict, split_config: SplitConfig) -> tuple[dict[int, Any], list[Any]]:
        """Warm-up / capture pass: one nano-batch, no policy. In CUDA-graph mode the
        graph runs once per nano-batch slot so that every slot captures its own graphs
        against its own static input buffers."""
        assert split_config.num_nano_batches == 1 and split_config.is_dryrun
        slots = self.config.max_num_splits if split_config.use_cudagraph else 1
        rows = split_config.num_tokens_padded[0]
        env = ExecutionEnvironment(slots)
        events = [_new_event() for _ in range(slots)]
        results: dict[int, Any] = {}
        for b in range(slots):
            for step in self.steps:
                node = step.node
                if step.kind == _PLACEHOLDER:
                    idx = step.placeholder_idx
                    example = node.meta.get("example_value", None)
                    if isinstance(example, torch.SymInt):
                        assert args[idx] == rows
                        env.put(b, node, rows)
                        continue
                    assert isinstance(example, torch.Tensor)
                    dynamic = example.dim() > 0 and isinstance(example.shape[0], torch.SymInt)
                    if not dynamic or not split_config.use_cudagraph:
                        env.put(b, node, args[idx])
                        continue
                    self.allocate_input_buffer(b, idx, self.max_static_rows, example)
                    buf = self.input_buffers[b][idx]
                    buf[:rows].copy_(args[idx][:rows])
                    env.put(b, node, buf[:rows])
                elif step.kind == _CALL_MODULE:
                    module = getattr(self.graph_module, step.target)
                    tag = getattr(module, "tag", set())
                    assert isinstance(tag, set)
                    a = [env.get(b, x) if isinstance(x, torch.fx.Node) else x for x in node.args]
                    kw = {k: env.get(b, v) if isinstance(v, torch.fx.Node) else v for k, v in node.kwargs.items()}
                    handle = OperatorHandle(module_name=step.target, batch_idx=b, batch_size=rows, tag=tag,
                                            _is_dryrun=True, _use_cudagraph=split_config.use_cudagraph)
                    with set_op_handle(handle):
                        env.put(b, node, module(*a, **kw))
                elif step.kind == _OUTPUT:
                    results[b] = self._collect_output(node, b, env)
                else:
                    self._run_simple_step(step, b, args, env, split_config)
            events[b].record()
        return {0: results[0]}, events

    # ----------------------------------------------------- single nano-batch
    def execute_single_batch(self, split_config: SplitConfig, args: tuple, kwargs: dict) -> Any:
        """One nano-batch without a policy: the (patched) graph module is called
        directly; in CUDA-graph mode dynamic inputs are first copied into slot 0's
        static buffers, the tensors the graphs were captured on."""
        rows = split_config.num_tokens_padded[0]
        new_args = list(args)
        for node in self.placeholder_nodes:
            idx = self.placeholder_node_to_idx[node]
            example = node.meta.get("example_value", None)
            if isinstance(example, torch.SymInt):
                if args[idx] == rows:
                    new_args[idx] = rows
            elif (isinstance(example, torch.Tensor) and example.dim() > 0
                  and isinstance(example.shape[0], torch.SymInt) and split_config.use_cudagraph):
                buf = self.input_buffers[0][idx]
                buf[:rows].copy_(args[idx])
                new_args[idx] = buf[:rows]
        handle = OperatorHandle(module_name=type(self.graph_module).__name__, batch_idx=0, batch_size=rows,
                                tag=set(), _is_dryrun=False, _use_cudagraph=split_config.use_cudagraph)
        with set_op_handle(handle):
            return self.graph_module(*new_args, **kwargs)

    # -------------------------------------------------------- split execution
    def execute(self, args: tuple, kwargs: dict, split_config: SplitConfig,
                scheduler: OpSchedulerBase) -> tuple[dict[int, Any], list[Any]]:
        """Runs every nano-batch under the policy. Returns per-nano-batch results and
        the event that marks the end of each nano-batch's last operator."""
        dispatcher = NanoBatchDispatcher(self, args, split_config)
        context = ExecutionContext(split_config, dispatcher)
        if self.config.additional_config.get("policy_uses_event_loop", False):
            import asyncio

            asyncio.run(scheduler.schedule(context))
        else:
            coroutine = scheduler.schedule(context)
            try:
                coroutine.send(None)
            except StopIteration:
                pass
            else:
                coroutine.close()
                raise RuntimeError(
                    "the policy's schedule() suspended on something other than context.pop/execute; set "
                    "additional_config['policy_uses_event_loop'] = True to run it on an asyncio event loop")
        dispatcher.finish()
        self.last_trace = dispatcher.trace
        return dispatcher.results, dispatcher.events


class NanoBatchDispatcher:
    """State of one split forward: program counter, outstanding operators, last
    event and results of every nano-batch."""

    def __init__(self, engine: DynaFlowEngine, args: tuple, split_config: SplitConfig) -> None:
        n = split_config.num_nano_batches
        self.engine = engine
        self.args = args
        self.cfg = split_config
        self.env = ExecutionEnvironment(n)
        self.pc = [0] * n
        self.outstanding: list[list[OperatorHandle]] = [[] for _ in range(n)]
        self.done = [False] * n
        self.results: dict[int, Any] = {}
        self.events = [_new_event() for _ in range(n)]
        self.last_stream: list[int | None] = [None] * n
        self.trace: list[tuple[str, int, int, bool]] = []
        for b in range(n):
            self._advance(b)
            self.events[b].record()
            self.last_stream[b] = _current_stream_id()

    def _advance(self, b: int) -> None:
        """Runs nano-batch ``b`` forward over non-operator steps up to the next
        subgraph call or through the output."""
        steps = self.engine.steps
        while self.pc[b] < len(steps):
            step = steps[self.pc[b]]
            if step.kind == _CALL_MODULE:
                return
            if step.kind == _OUTPUT:
                self.results[b] = DynaFlowEngine._collect_output(step.node, b, self.env)
                self.pc[b] += 1
                self.done[b] = True
                return
            self.engine._run_simple_step(step, b, self.args, self.env, self.cfg)
            self.pc[b] += 1
        self.done[b] = True

    def pop(self, b: int) -> OperatorHandle | None:
        if self.done[b]:
            return None
        steps = self.engine.steps
        step = steps[self.pc[b]] if self.pc[b] < len(steps) else None
        if step is None or step.kind != _CALL_MODULE:
            raise RuntimeError(
                f"nano-batch {b}: pop() with {len(self.outstanding[b])} operator(s) still to execute and no "
                "further operator ready; the policy has to execute what it popped first")
        module = getattr(self.engine.graph_module, step.target)
        tag = getattr(module, "tag", set())
        assert isinstance(tag, set)
        handle = OperatorHandle(module_name=step.target, batch_idx=b, batch_size=self.cfg.num_tokens_padded[b],
                                tag=tag, _is_dryrun=self.cfg.is_dryrun, _use_cudagraph=self.cfg.use_cudagraph)
        self.outstanding[b].append(handle)
        self.pc[b] += 1
        return handle

    def execute(self, operators: tuple[OperatorHandle, ...], func: Callable[..., Any] | None) -> None:
        if len(operators) != 1:
            raise NotImplementedError("Operator batching is not implemented")
        op = operators[0]
        b = op.batch_idx
        if not self.outstanding[b] or self.outstanding[b][0] is not op:
            raise RuntimeError(f"nano-batch {b}: operators must execute in the order they were popped "
                               f"(got {op.module_name})")
        node = self.engine.module_name_to_node[op.module_name]
        stream_id = _current_stream_id()
        if self.last_stream[b] != stream_id:
            self.events[b].wait()  # cross-stream dependency on this nano-batch's previous operator
        a = [self.env.get(b, x) for x in node.args if isinstance(x, torch.fx.Node)]
        kw = {k: self.env.get(b, v) if isinstance(v, torch.fx.Node) else v for k, v in node.kwargs.items()}
        with torch.cuda.nvtx.range(f"op_{op.module_name}_{b}"), set_op_handle(op):
            if func is not None:
                result = func(*a, **kw)
            else:
                result = getattr(self.engine.graph_module, op.module_name)(*a, **kw)
        self.events[b].record()
        self.last_stream[b] = stream_id
        self.env.put(b, node, result)
        self.outstanding[b].pop(0)
        self.trace.append((op.module_name, b, stream_id, func is not None))
        if not self.outstanding[b]:
            self._advance(b)

    def finish(self) -> None:
        unfinished = [b for b, d in enumerate(self.done) if not d]
        if unfinished:
            raise RuntimeError(f"the policy returned while nano-batch(es) {unfinished} still had operators to run")
