"""Build-container-only checks that need the reference tree: its policy files must
load and run UNMODIFIED against dynaflow_b200 (aliased as ``dynaflow``), and
get_split_config must agree with the reference on generated request lists."""
import importlib.util
import os
import subprocess
import sys
import textwrap

import pytest

from conftest import REFERENCE, ROOT

pytestmark = pytest.mark.reference

SCRIPT = textwrap.dedent("""
    import contextlib, importlib.util, io, json, sys
    import torch
    sys.path.insert(0, {root!r}); sys.path.insert(0, {root!r} + "/tests")
    import dynaflow_b200
    dynaflow_b200.install_as_dynaflow()
    import dynaflow.interface, dynaflow.matching            # resolved to dynaflow_b200
    assert dynaflow.interface.__name__ == "dynaflow_b200.interface"
    # CPU stand-ins for what the policy constructor asks of torch.cuda
    class _S:
        def __init__(self, *a, **k): pass
    torch.cuda.Stream = _S
    torch.cuda.stream = lambda s: contextlib.nullcontext()
    spec = importlib.util.spec_from_file_location("_ref_policy", {ref!r} + "/examples/ae/scheduler/hf/nanoflow.py")
    mod = importlib.util.module_from_spec(spec); spec.loader.exec_module(mod)
    from helpers import Host, make_config, two_way
    from dynaflow_b200.matching import MatchingRule, Op
    from oracle import llama_oracle, split_oracle

    class Policy(mod.NanoFlowScheduler):      # the reference's schedule() and get_split_config(), our cut
        def get_split_rules(self):
            return [MatchingRule(condition=Op(pattern=r"scaled_dot_product_attention"))]
        def get_tag_rules(self):
            return {{MatchingRule(condition=Op(pattern=r"scaled_dot_product_attention")): {{"network"}}}}

    cfg = make_config(min_nano_split_tokens=1)
    shape = llama_oracle.LlamaShape(hidden=64, intermediate=96, heads=4, kv_heads=4, head_dim=16, layers=2, vocab=128)
    model = llama_oracle.build(shape)
    ids = llama_oracle.make_ids(6, 10, shape.vocab)
    host = Host(model, Policy(cfg), cfg)
    with torch.inference_mode():
        want = model(ids)
    got = host.run((ids,), two_way([0, 2, 6]))
    names = sorted(host.tags, key=lambda s: int(s.split("_")[1]))
    ok = bool((got - want).abs().max() / want.abs().max() <= 1e-5) and host.trace == split_oracle.round_robin_trace([names, names])
    print(json.dumps({{"ok": ok, "n_ops": len(host.trace)}}))
""")


def test_reference_hf_policy_runs_unmodified():
    code = SCRIPT.format(root=ROOT, ref=REFERENCE)
    proc = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-3000:]
    assert '"ok": true' in proc.stdout.splitlines()[-1]


def test_get_split_config_agrees_with_live_reference():
    hypothesis = pytest.importorskip("hypothesis")
    from hypothesis import given, settings, strategies as st

    from oracle import split_oracle

    # load the reference's arithmetic without importing its package into this process:
    # run it in a child and compare a generated batch of cases
    cases = []

    @settings(max_examples=150, deadline=None)
    @given(st.lists(st.integers(1, 4096), min_size=1, max_size=16), st.sampled_from([1, 16, 64, 256]),
           st.lists(st.sampled_from([8, 32, 64, 128, 512, 2048, 8192]), min_size=1, max_size=4, unique=True),
           st.booleans())
    def collect(tokens, min_tokens, sizes, cg):
        cases.append(dict(num_tokens=tokens, min_tokens=min_tokens, sizes=sizes, cg=cg))

    collect()
    child = textwrap.dedent("""
        import contextlib, dataclasses, importlib.util, json, sys
        import torch
        sys.path.insert(0, {ref!r})
        class _S:
            def __init__(self, *a, **k): pass
        torch.cuda.Stream = _S
        import dynaflow.config as C, dynaflow.interface as I
        spec = importlib.util.spec_from_file_location("_p", {ref!r} + "/examples/ae/scheduler/hf/nanoflow.py")
        m = importlib.util.module_from_spec(spec); spec.loader.exec_module(m)
        out = []
        for c in json.load(sys.stdin):
            cfg = C.DynaFlowConfig("a:b", 2, C.InductorConfig(False), C.CUDAGraphConfig(True, c["sizes"]),
                                   {{"min_nano_split_tokens": c["min_tokens"]}})
            s = m.NanoFlowScheduler(cfg).get_split_config(I.InputInfo(len(c["num_tokens"]), c["num_tokens"], sum(c["num_tokens"])), c["cg"])
            out.append(dataclasses.asdict(s))
        print(json.dumps(out))
    """).format(ref=REFERENCE)
    import json
    proc = subprocess.run([sys.executable, "-c", child], input=json.dumps(cases), capture_output=True, text=True,
                          timeout=600)
    assert proc.returncode == 0, proc.stderr[-3000:]
    ref_out = json.loads(proc.stdout.splitlines()[-1])
    import dataclasses

    from helpers import make_config
    from dynaflow_b200.interface import InputInfo
    from dynaflow_b200.policies import NanoFlowScheduler
    for c, want in zip(cases, ref_out):
        assert split_oracle.nanoflow_split(c["num_tokens"], c["min_tokens"], c["sizes"], c["cg"]) == want, c
        pol = NanoFlowScheduler(make_config(capture_sizes=c["sizes"], cudagraph=True, min_nano_split_tokens=c["min_tokens"]))
        got = pol.get_split_config(InputInfo(len(c["num_tokens"]), c["num_tokens"], sum(c["num_tokens"])), c["cg"])
        assert dataclasses.asdict(got) == want, c
