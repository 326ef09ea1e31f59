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


_OVERHEAD_CHILD = textwrap.dedent("""
    import contextlib, importlib.util, io, json, sys, time
    import torch
    which = sys.argv[1]
    sys.path.insert(0, {root!r}); sys.path.insert(0, {root!r} + "/tests")
    from oracle import llama_oracle
    torch.set_num_threads(1)
    shape = llama_oracle.LlamaShape(hidden=32, intermediate=64, heads=2, kv_heads=2, head_dim=16, layers=16, vocab=64)
    model = llama_oracle.build(shape)
    ids = llama_oracle.make_ids(4, 8, shape.vocab)
    cuts = [0, 2, 4]
    if which == "reference":
        # the reference package itself, with inert stand-ins for the CUDA events / streams it creates
        class _E:
            def __init__(self, *a, **k): pass
            def record(self, *a, **k): pass
            def wait(self, *a, **k): pass
            def synchronize(self): pass
        class _S:
            def __init__(self, *a, **k): pass
        torch.cuda.Event, torch.cuda.Stream = _E, _S
        torch.cuda.stream = lambda s: contextlib.nullcontext()
        sys.path.insert(0, {ref!r})
        import dynaflow.config as C, dynaflow.interface as I, dynaflow.matching as M, dynaflow.manager as G
        spec = importlib.util.spec_from_file_location("_p", {ref!r} + "/examples/ae/scheduler/hf/nanoflow.py")
        hf = importlib.util.module_from_spec(spec); spec.loader.exec_module(hf)
        class Policy(hf.NanoFlowScheduler):
            def get_split_rules(self):
                return [M.MatchingRule(condition=M.Op(pattern=r"scaled_dot_product_attention"))]
            def get_tag_rules(self):
                return {{M.MatchingRule(condition=M.Op(pattern=r"scaled_dot_product_attention")): {{"network"}}}}
        cfg = C.DynaFlowConfig("x:y", 2, C.InductorConfig(False), C.CUDAGraphConfig(False, [64]), {{"min_nano_split_tokens": 1}})
        manager, policy = G.DynaFlowManager(), Policy(cfg)
        def backend(gm, example_inputs):
            manager.initialize(graph_module=gm, config=cfg, scheduler=policy, example_inputs=list(example_inputs))
            return manager.get_callable()
        split = lambda: I.SplitConfig(2, [2, 2], cuts, [2, 2], [2, 2], cuts, False, False)
        n_ops = lambda: 2 * len(manager.engine.module_name_to_node)
    else:
        from helpers import cut_policy, make_config, two_way
        from dynaflow_b200.manager import DynaFlowManager
        cfg = make_config()
        manager, policy = DynaFlowManager(), cut_policy(r"scaled_dot_product_attention", "network", cfg)
        def backend(gm, example_inputs):
            manager.initialize(graph_module=gm, config=cfg, scheduler=policy, example_inputs=list(example_inputs))
            return manager.get_callable()
        split = lambda: two_way(cuts)
        n_ops = lambda: 2 * len(manager.engine.module_name_to_node)
    torch._dynamo.reset()
    torch._dynamo.mark_dynamic(ids, 0)
    compiled = torch.compile(model, backend=backend, fullgraph=True)
    def forward():
        manager.override_split_config(split())
        with torch.inference_mode(), contextlib.redirect_stdout(io.StringIO()):
            return compiled(ids)
    for _ in range(5):
        out = forward()
    best = float("inf")
    for _ in range(5):
        t0 = time.perf_counter()
        for _ in range(20):
            forward()
        best = min(best, (time.perf_counter() - t0) / 20)
    with torch.inference_mode():
        t0 = time.perf_counter()
        for _ in range(20):
            want = model(ids)
        eager = (time.perf_counter() - t0) / 20
    ok = bool((out - want).abs().max() / want.abs().max() <= 1e-5)
    print(json.dumps({{"which": which, "ms_per_forward": best * 1e3, "ms_eager_unsplit": eager * 1e3, "dispatches": n_ops(), "ok": ok}}))
""")


def test_host_dispatch_overhead_vs_reference(capsys):
    """Host cost of one split forward (2 nano-batches, 16-layer toy decoder cut at attention: 66 operator
    dispatches, CPU tensors small enough that dispatch dominates): this package's synchronous dispatcher
    against the reference's engine/policy coroutine pair on a per-forward event loop
    (``dynaflow/manager.py:161-261``, ``runtime/engine.py:222-424``), same policy logic, same machine."""
    import json

    results = {}
    for which in ("reference", "ours"):
        code = _OVERHEAD_CHILD.format(root=ROOT, ref=REFERENCE)
        proc = subprocess.run([sys.executable, "-c", code, which], capture_output=True, text=True, timeout=900)
        assert proc.returncode == 0, proc.stderr[-3000:]
        results[which] = json.loads(proc.stdout.splitlines()[-1])
        assert results[which]["ok"]
    ref, ours = results["reference"], results["ours"]
    assert ref["dispatches"] == ours["dispatches"]
    with capsys.disabled():
        print(f"\nhost dispatch, {ours['dispatches']} dispatches per forward: reference {ref['ms_per_forward']:.3f} ms, "
              f"dynaflow_b200 {ours['ms_per_forward']:.3f} ms (unsplit eager model {ours['ms_eager_unsplit']:.3f} ms)")
    # measured: 10.0 ms against 12.1 ms; the bound leaves room for a loaded machine
    assert ours["ms_per_forward"] < 1.3 * ref["ms_per_forward"]
