"""Host-side mirror of the reference interface: split configs, matching, engine, manager.
Everything here is pinned against fixtures the reference package produced."""
import json
import os

import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

from conftest import GOLDEN
from helpers import Host, cut_policy, make_config, two_way
from dynaflow_b200.interface import InputInfo, SplitConfig
from dynaflow_b200.matching import MatchingRule, Mod, Op, assign_subgraph_ids
from dynaflow_b200.policies import EqualSplitScheduler, NanoFlowScheduler
from dynaflow_b200.utils import pack_tokens
from oracle import llama_oracle, split_oracle


def _load(name):
    with open(os.path.join(GOLDEN, name)) as f:
        return json.load(f)


def _as_dict(cfg: SplitConfig) -> dict:
    import dataclasses
    return dataclasses.asdict(cfg)


def test_nanoflow_get_split_config_matches_reference_golden():
    for entry in _load("split_configs.json")["nanoflow"]:
        c = entry["case"]
        policy = NanoFlowScheduler(make_config(capture_sizes=c["sizes"], cudagraph=True,
                                               min_nano_split_tokens=c["min_tokens"]))
        got = policy.get_split_config(InputInfo(len(c["num_tokens"]), c["num_tokens"], sum(c["num_tokens"])), c["cg"])
        assert _as_dict(got) == entry["split"], c


def test_equal_split_matches_reference_golden():
    for entry in _load("split_configs.json")["equal"]:
        c = entry["case"]
        policy = EqualSplitScheduler(make_config(max_splits=c["n"], min_nano_split_tokens=c["min_tokens"],
                                                 num_nano_batches=c["n"]))
        got = policy.get_split_config(InputInfo(c["rows"], [c["rows"]], c["rows"]), False)
        assert _as_dict(got) == entry["split"], c


def test_baseline_configs_split_as_surveyed():
    policy = NanoFlowScheduler(make_config(min_nano_split_tokens=64))
    got = policy.get_split_config(InputInfo(8, [2048] * 8, 16384), False)   # Llama-3-8B prefill, 8 x 2048
    assert got.split_indices == [0, 8192, 16384] and got.batch_indices == [0, 4, 8]
    got = policy.get_split_config(InputInfo(256, [1] * 256, 256), True)     # decode, batch 256
    assert got.split_indices == [0, 128, 256] and got.num_tokens_padded == [128, 128] and got.use_cudagraph


def test_pack_tokens():
    assert pack_tokens(100, [256, 64, 128]) == split_oracle.pack_tokens(100, [256, 64, 128]) == (128, True)
    assert pack_tokens(256, [64, 256]) == (256, True)
    assert pack_tokens(257, [64, 256]) == split_oracle.pack_tokens(257, [64, 256]) == (257, False)
    assert pack_tokens(0, [8]) == (8, True)


# ------------------------------------------------------------------ matching
class _Norm(nn.Module):
    def forward(self, x):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-5)


class _Tiny(nn.Module):
    def __init__(self):
        super().__init__()
        self.a = nn.Linear(8, 8, bias=False)
        self.n1 = _Norm()
        self.n2 = _Norm()

    def forward(self, x):
        y = F.silu(self.a(x))
        y = self.n1(y)
        y = torch.relu(y)
        return self.n2(y) + 1


def _trace(model, x):
    graphs = []

    def backend(gm, _):
        graphs.append(gm)
        return gm

    torch._dynamo.reset()
    torch._dynamo.mark_dynamic(x, 0)
    torch.compile(model, backend=backend, fullgraph=True)(x)
    return graphs[0]


def test_op_mod_and_rule_matching():
    gm = _trace(_Tiny(), torch.randn(6, 8))
    nodes = list(gm.graph.nodes)
    silu = next(i for i, n in enumerate(nodes) if Op("silu").matches(n))
    assert not Op("sil").matches(nodes[silu])            # full match, not prefix
    assert Op(r"si.*").matches(nodes[silu])
    assert not Op("silu").matches(nodes[0])              # placeholder
    run = Mod(_Norm).matches(nodes[silu + 1:])
    assert run >= 4                                        # pow, mean, add, rsqrt, mul of ONE instance
    assert Mod(_Norm).matches(nodes[silu + 1 + run:]) == 0  # relu follows
    rule = MatchingRule((Op("silu"), Mod(_Norm)))
    assert rule.matches(nodes, silu) == 1 + run
    assert rule.matches(nodes, silu + 1) == 0
    vetoed = MatchingRule((Op("silu"), Mod(_Norm)), hook=lambda nl, i: False)
    assert vetoed.matches(nodes, silu) == 0
    assert hash(rule) != hash(vetoed) and {rule: 1}[rule] == 1  # usable as dict keys
    ids = assign_subgraph_ids(nodes, [rule])
    assert ids[nodes[silu]] == ids[nodes[silu + run]] == 1
    assert ids[nodes[silu - 1]] == 0 and ids[nodes[silu + 1 + run]] == 2


# ---------------------------------------------------------- engine / manager
SMALL = llama_oracle.LlamaShape(hidden=64, intermediate=96, heads=4, kv_heads=4, head_dim=16, layers=2, vocab=128)


@pytest.fixture(scope="module")
def small_model():
    return llama_oracle.build(SMALL, seed=0)


def test_split_equals_unsplit_small(small_model):
    ids = llama_oracle.make_ids(6, 12, SMALL.vocab)
    host = Host(small_model, cut_policy(r"scaled_dot_product_attention", "attention"))
    with torch.inference_mode():
        want = small_model(ids)
    for cuts in ([0, 3, 6], [0, 1, 6], [0, 5, 6]):
        got = host.run((ids,), two_way(cuts))
        rel = (got - want).abs().max() / want.abs().max()
        assert got.shape == want.shape and rel <= 1e-5, (cuts, rel)
    assert host.tags == {"submod_0": [], "submod_1": ["attention"], "submod_2": [], "submod_3": ["attention"],
                         "submod_4": []}
    names = sorted(host.tags, key=lambda s: int(s.split("_")[1]))
    assert host.trace == split_oracle.round_robin_trace([names, names])


def test_single_nano_batch_fallback_and_forced_policy(small_model):
    ids = llama_oracle.make_ids(4, 8, SMALL.vocab)
    host = Host(small_model, cut_policy(r"scaled_dot_product_attention", "attention"))
    with torch.inference_mode():
        want = small_model(ids)
    one = SplitConfig(1, [4], [0, 4], [4], [4], [0, 4], is_dryrun=False, use_cudagraph=False)
    got = host.run((ids,), one)
    assert torch.equal(got, want)
    host.manager.engine.last_trace = []
    forced = SplitConfig(1, [4], [0, 4], [4], [4], [0, 4], is_dryrun=False, use_cudagraph=False, allow_fallback=False)
    got = host.run((ids,), forced)
    assert torch.equal(got, want) and len(host.trace) == 5
    dry = SplitConfig(1, [4], [0, 4], [4], [4], [0, 4], is_dryrun=True, use_cudagraph=False)
    assert torch.equal(host.run((ids,), dry), want)
    # the cached config is consumed by every forward
    with pytest.raises(AssertionError):
        host.compiled(ids)


def test_substitution_receives_graph_order_args(small_model):
    ids = llama_oracle.make_ids(4, 8, SMALL.vocab)
    policy = cut_policy(r"scaled_dot_product_attention", "attention")
    seen = []

    def my_attention(*args):
        tensors = [a for a in args if isinstance(a, torch.Tensor)]
        seen.append(len(tensors))
        q, k, v = tensors[-3:]
        return F.scaled_dot_product_attention(q, k, v, is_causal=True)

    policy.substitutions["attention"] = my_attention
    host = Host(small_model, policy)
    with torch.inference_mode():
        want = small_model(ids)
    got = host.run((ids,), two_way([0, 2, 4]))
    assert len(seen) == 4 and (got - want).abs().max() / want.abs().max() <= 1e-5
    assert [s for *_, s in host.manager.engine.last_trace].count(True) == 4


def test_equal_split_three_way_skewed_trace(small_model):
    ids = llama_oracle.make_ids(7, 8, SMALL.vocab)
    cfg = make_config(max_splits=3, num_nano_batches=3)
    policy = cut_policy(r"scaled_dot_product_attention", "attention", cfg, cls=EqualSplitScheduler)
    host = Host(small_model, policy)
    split = policy.get_split_config(InputInfo(7, [7], 7))
    assert split.split_indices == [0, 2, 4, 7]
    with torch.inference_mode():
        want = small_model(ids)
    got = host.run((ids,), split)
    assert (got - want).abs().max() / want.abs().max() <= 1e-5
    names = sorted(host.tags, key=lambda s: int(s.split("_")[1]))
    assert host.trace == split_oracle.skewed_trace([names] * 3)


def test_policy_errors_raise_instead_of_hanging(small_model):
    from dynaflow_b200.interface import OpSchedulerBase

    ids = llama_oracle.make_ids(4, 8, SMALL.vocab)

    class _Base(NanoFlowScheduler):
        pass

    class PopsTwice(_Base):
        async def schedule(self, context):
            await context.pop(0)
            await context.pop(0)

    class OutOfOrder(_Base):
        async def schedule(self, context):
            a = await context.pop(0)
            await context.execute((a,))
            b = await context.pop(0)
            await context.execute((a,))

    class ReturnsEarly(_Base):
        async def schedule(self, context):
            a = await context.pop(0)
            await context.execute((a,))

    class Groups(_Base):
        async def schedule(self, context):
            a, b = await context.pop(0), await context.pop(1)
            await context.execute((a, b))

    for cls, exc in ((PopsTwice, RuntimeError), (OutOfOrder, RuntimeError), (ReturnsEarly, RuntimeError),
                     (Groups, NotImplementedError)):
        policy = cut_policy(r"scaled_dot_product_attention", "attention", cls=cls)
        host = Host(small_model, policy)
        with pytest.raises(exc):
            host.run((ids,), two_way([0, 2, 4]))
    assert issubclass(NanoFlowScheduler, OpSchedulerBase)


def test_tuple_outputs_are_merged_field_by_field():
    class Two(nn.Module):
        def forward(self, x):
            y = F.silu(x)
            return y + 1, y * 2

    x = torch.randn(10, 4)
    host = Host(Two(), cut_policy(r"silu", "act"))
    a, b = host.run((x,), two_way([0, 3, 10]))
    assert a.shape == b.shape == x.shape
    # (vectorised CPU exp may differ in the last bit between a 12- and a 40-element call)
    assert torch.allclose(a, F.silu(x) + 1, rtol=1e-6, atol=1e-6) and torch.allclose(b, F.silu(x) * 2, rtol=1e-6, atol=1e-6)


# --------------------------------------------------- the CPU parity configuration
def test_c1_llama_against_reference_golden():
    golden = _load("c1_llama.json")
    shape = llama_oracle.LlamaShape(**golden["shape"])
    model = llama_oracle.build(shape, seed=golden["weights_seed"])
    ids = llama_oracle.make_ids(4, 256, shape.vocab, seed=golden["ids_seed"])
    host = Host(model, cut_policy(r"scaled_dot_product_attention", "attention"))
    sample_ref = torch.tensor(golden["logits_sample"])
    with torch.inference_mode():
        unsplit = model(ids)
    for run in golden["runs"]:
        got = host.run((ids,), SplitConfig(**run["split"]))
        assert host.tags == run["tags"]
        assert [list(t) for t in host.trace] == run["trace"]          # routing: bit-exact
        rel = (got - unsplit).abs().max() / unsplit.abs().max()
        assert rel <= 1e-5
        if run["split"]["split_indices"] == [0, 2, 4]:
            assert run["equal_to_unsplit"] and torch.equal(got, unsplit)  # as observed for the reference
        sample = got[:, ::32, ::1000]
        assert (sample - sample_ref).abs().max() / golden["logits_abs_max"] <= 1e-5


def test_dbo_policy_matches_reference_golden(monkeypatch):
    """The MoE dual-batch-overlap policy against the order and streams the reference's own
    policy produced for the same tagged operator programs."""
    import asyncio
    import contextlib

    import dynaflow_b200.policies as policies
    from dynaflow_b200.interface import OperatorHandle

    current = {"stream": "default"}

    @contextlib.contextmanager
    def fake_on(stream):
        prev, current["stream"] = current["stream"], stream
        try:
            yield
        finally:
            current["stream"] = prev

    monkeypatch.setattr(policies, "_on", fake_on)
    for case in _load("dbo_trace.json")["cases"]:
        program, n = case["program"], case["batches"]
        policy = policies.DBOScheduler(make_config())
        policy.comm_stream, policy.comp_stream = "comm", "comp"
        swaps = []
        policy.before_execute = lambda b, op: swaps.append(b)
        trace = []

        class Ctx:
            split_config = SplitConfig(n, [1] * n, list(range(n + 1)), [1] * n, [1] * n, list(range(n + 1)), False, False)
            cursor = [0] * n

            async def pop(self, b):
                if self.cursor[b] >= len(program):
                    return None
                name, tags = program[self.cursor[b]]
                self.cursor[b] += 1
                return OperatorHandle(name, b, 1, set(tags), False, False)

            async def execute(self, ops, func=None):
                trace.append([ops[0].module_name, ops[0].batch_idx, current["stream"]])

        asyncio.run(policy.schedule(Ctx()))
        assert trace == case["trace"], (case["layers"], n)
        assert swaps, "the per-operator host hook was never called"
