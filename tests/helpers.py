"""Shared test helpers: run a model through dynaflow_b200's manager the way the
reference's minimal host does (``examples/ae/scripts/bench_hf_transformers.py:17-105``)."""
import contextlib
import io

import torch

from dynaflow_b200.config import CUDAGraphConfig, DynaFlowConfig, InductorConfig
from dynaflow_b200.interface import SplitConfig
from dynaflow_b200.manager import DynaFlowManager
from dynaflow_b200.matching import MatchingRule, Op
from dynaflow_b200.policies import NanoFlowScheduler


def make_config(max_splits=2, capture_sizes=(64, 128, 256), cudagraph=False, copy_inputs=False, **additional):
    additional.setdefault("min_nano_split_tokens", 1)
    return DynaFlowConfig("unused:unused", max_splits, InductorConfig(False),
                          CUDAGraphConfig(cudagraph, list(capture_sizes), copy_mismatched_inputs=copy_inputs),
                          dict(additional))


def cut_policy(pattern, tag, config=None, cls=NanoFlowScheduler):
    config = config or make_config()
    rule = MatchingRule(condition=Op(pattern=pattern))
    return cls(config, split_rules=[rule], tag_rules={rule: {tag}})


def two_way(cuts, padded=None, **kw):
    sizes = [cuts[1] - cuts[0], cuts[2] - cuts[1]]
    return SplitConfig(2, sizes, list(cuts), list(sizes), list(padded or sizes), list(cuts), is_dryrun=False,
                       use_cudagraph=kw.pop("use_cudagraph", False), **kw)


class Host:
    """torch.compile host: traces ``model`` once and runs it through a DynaFlowManager."""

    def __init__(self, model, policy, config=None):
        self.manager = DynaFlowManager()
        self.policy = policy
        self.config = config or policy.config
        self.model = model

        def backend(gm, example_inputs):
            if not any(isinstance(i, torch.SymInt) for i in example_inputs):
                return gm
            self.manager.initialize(graph_module=gm, config=self.config, scheduler=policy,
                                    example_inputs=list(example_inputs))
            return self.manager.get_callable()

        torch._dynamo.reset()
        self.compiled = torch.compile(model, backend=backend, fullgraph=True)

    def run(self, inputs, split):
        for t in inputs:
            if isinstance(t, torch.Tensor):
                torch._dynamo.mark_dynamic(t, 0)
        self.manager.override_split_config(split)
        with torch.inference_mode(), contextlib.redirect_stdout(io.StringIO()):
            return self.compiled(*inputs)

    @property
    def trace(self):
        return [(name, b) for name, b, _stream, _sub in self.manager.engine.last_trace]

    @property
    def tags(self):
        gm = self.manager.graph_module
        return {name: sorted(gm.__dict__[name].tag) for name in self.manager.engine.module_name_to_node}
