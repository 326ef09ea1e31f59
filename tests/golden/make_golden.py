"""Generates the golden fixtures in this directory by running the REFERENCE package.

Run in the build container only (the reference tree is not available elsewhere):

    python tests/golden/make_golden.py [/path/to/reference]

The reference's engine records CUDA events unconditionally
(``dynaflow/runtime/engine.py:254-266``) and its example policies create CUDA
streams in their constructors; on a machine without a GPU this script replaces
``torch.cuda.Event`` / ``Stream`` / ``stream`` by inert stand-ins. Nothing else of
the reference is modified. Outputs:

    split_configs.json   get_split_config of the reference NanoFlow policies
    c1_llama.json        partition, tags, dispatch order and sampled logits of the
                         2-layer decoder split into two nano-batches
    dbo_trace.json       execution order and streams of the reference's DBO (MoE) policy
    mlp_split.npz/.json  bf16 gated-MLP graph executed by the reference in two
                         ragged nano-batches (inputs, weights, output)
    norm_split.npz/.json residual add + RMSNorm (Hugging Face's LlamaRMSNorm, bf16, eps 1e-5)
                         executed by the reference in two ragged nano-batches
    moe_split.npz/.json  Mixtral-style top-2 mixture of gated-MLP experts (router arithmetic of
                         Hugging Face's MixtralTopKRouter) executed the same way
"""
from __future__ import annotations

import contextlib
import dataclasses
import importlib.util
import io
import json
import os
import random
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(os.path.dirname(HERE))
REFERENCE = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("DYNAFLOW_REFERENCE", "/root/reference")


class _InertEvent:
    def __init__(self, *a, **k):
        pass

    def record(self, *a, **k):
        pass

    def wait(self, *a, **k):
        pass

    def synchronize(self):
        pass


class _InertStream:
    def __init__(self, *a, **k):
        pass


def install_cpu_shims() -> None:
    torch.cuda.Event = _InertEvent  # type: ignore[misc]
    torch.cuda.Stream = _InertStream  # type: ignore[misc]
    torch.cuda.stream = lambda s: contextlib.nullcontext()  # type: ignore[assignment]


def load_policy_module(path: str, name: str):
    spec = importlib.util.spec_from_file_location(name, path)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def split_cases() -> list[dict]:
    rng = random.Random(1234)
    cases = [
        dict(num_tokens=[2048] * 8, min_tokens=64, sizes=[64, 128, 256], cg=False),
        dict(num_tokens=[1] * 256, min_tokens=64, sizes=[64, 128, 256], cg=True),
        dict(num_tokens=[1] * 256, min_tokens=64, sizes=[64, 100], cg=True),
        dict(num_tokens=[5], min_tokens=1, sizes=[8], cg=False),
        dict(num_tokens=[5], min_tokens=1, sizes=[8], cg=True),
        dict(num_tokens=[100, 1], min_tokens=2, sizes=[64, 128], cg=True),
        dict(num_tokens=[3, 3], min_tokens=3, sizes=[2, 4], cg=True),
        dict(num_tokens=[7, 1, 1, 7], min_tokens=1, sizes=[16], cg=False),
        dict(num_tokens=[10, 10, 10], min_tokens=1, sizes=[16], cg=True),
        dict(num_tokens=[300, 20, 20], min_tokens=30, sizes=[512], cg=True),
    ]
    for _ in range(40):
        n = rng.randint(1, 12)
        toks = [rng.randint(1, 600) for _ in range(n)]
        sizes = sorted(rng.sample([8, 16, 32, 64, 128, 256, 512, 1024, 2048, 4096], rng.randint(1, 5)))
        rng.shuffle(sizes)
        cases.append(dict(num_tokens=toks, min_tokens=rng.choice([1, 16, 64, 256]), sizes=sizes,
                          cg=rng.random() < 0.5))
    return cases


def golden_split_configs(ref_iface, ref_cfg) -> dict:
    hf = load_policy_module(os.path.join(REFERENCE, "examples/ae/scheduler/hf/nanoflow.py"), "_ref_hf_nanoflow")
    meg = load_policy_module(os.path.join(REFERENCE, "examples/ae/scheduler/megatron/nanoflow.py"), "_ref_meg_nanoflow")
    out = {"nanoflow": [], "equal": []}
    for case in split_cases():
        cfg = ref_cfg.DynaFlowConfig("x:y", 2, ref_cfg.InductorConfig(False), ref_cfg.CUDAGraphConfig(True, case["sizes"]),
                                     {"min_nano_split_tokens": case["min_tokens"]})
        policy = hf.NanoFlowScheduler(cfg)
        info = ref_iface.InputInfo(len(case["num_tokens"]), case["num_tokens"], sum(case["num_tokens"]))
        got = policy.get_split_config(info, case["cg"])
        out["nanoflow"].append({"case": case, "split": dataclasses.asdict(got)})
    rng = random.Random(99)
    for _ in range(30):
        rows = rng.randint(1, 5000)
        n = rng.randint(1, 4)
        mn = rng.choice([1, 64, 512])
        cfg = ref_cfg.DynaFlowConfig("x:y", n, ref_cfg.InductorConfig(False), ref_cfg.CUDAGraphConfig(False, [1]),
                                     {"min_nano_split_tokens": mn, "num_nano_batches": n})
        policy = meg.NanoFlowMegatronScheduler(cfg)
        got = policy.get_split_config(ref_iface.InputInfo(rows, [rows], rows), False)
        out["equal"].append({"case": {"rows": rows, "n": n, "min_tokens": mn}, "split": dataclasses.asdict(got)})
    return out


def make_reference_policy(hf_module, ref_matching, pattern: str, tag: str, cfg):
    """The reference's HF NanoFlow policy with its split / tag rules pointed at an
    operator that exists in a single-process model."""

    class _Policy(hf_module.NanoFlowScheduler):
        def __init__(self, config):
            super().__init__(config)
            self.trace = []

        def get_split_rules(self):
            return [ref_matching.MatchingRule(condition=ref_matching.Op(pattern=pattern))]

        def get_tag_rules(self):
            return {ref_matching.MatchingRule(condition=ref_matching.Op(pattern=pattern)): {tag}}

    return _Policy(cfg)


def run_reference(model, inputs, split, pattern, tag, ref):
    """Executes ``model(*inputs)`` through the reference manager with ``split``."""
    ref_cfg, ref_iface, ref_matching, ref_manager = ref
    hf = load_policy_module(os.path.join(REFERENCE, "examples/ae/scheduler/hf/nanoflow.py"), "_ref_hf_nanoflow2")
    cfg = ref_cfg.DynaFlowConfig("x:y", 2, ref_cfg.InductorConfig(False), ref_cfg.CUDAGraphConfig(False, [64]),
                                 {"min_nano_split_tokens": 1})
    policy = make_reference_policy(hf, ref_matching, pattern, tag, cfg)
    manager = ref_manager.DynaFlowManager()
    trace: list[tuple[str, int]] = []

    def backend(gm, example_inputs):
        manager.initialize(graph_module=gm, config=cfg, scheduler=policy, example_inputs=list(example_inputs))
        # record the dispatch order at the point where the engine calls each subgraph
        import dynaflow.runtime.env as ref_env
        for name in list(manager.engine.module_name_to_node):
            backend_obj = manager.graph_module.__dict__[name]
            inner = backend_obj.callable_dynamic

            def wrapped(*a, _inner=inner, **k):
                h = ref_env.get_op_handle()
                trace.append((h.module_name, h.batch_idx))
                return _inner(*a, **k)

            backend_obj.callable_dynamic = wrapped
        return manager.get_callable()

    torch._dynamo.reset()
    for t in inputs:
        torch._dynamo.mark_dynamic(t, 0)
    compiled = torch.compile(model, backend=backend, fullgraph=True)
    manager.override_split_config(ref_iface.SplitConfig(**split))
    with torch.inference_mode(), contextlib.redirect_stdout(io.StringIO()):
        out = compiled(*inputs)
    tags = {name: sorted(getattr(manager.graph_module.__dict__[name], "tag", set()))
            for name in manager.engine.module_name_to_node}
    return out, trace, tags



def bits(t: torch.Tensor):
    """bf16 tensors are stored as their int16 bit patterns (numpy has no bf16)."""
    return t.detach().contiguous().view(torch.int16).numpy().copy()


class AddRMSNorm(torch.nn.Module):
    """The residual add and the normalisation that follow an all-reduce in a Hugging Face Llama
    decoder layer (``hidden = residual + hidden; hidden = post_attention_layernorm(hidden)``):
    the pair of operators the reference's policies match together with the collective
    (``examples/ae/scheduler/vllm/nanoflow.py:59-69, 171-211``). The normalisation is
    transformers' own ``LlamaRMSNorm``."""

    def __init__(self, hidden: int, eps: float) -> None:
        super().__init__()
        from transformers.models.llama.modeling_llama import LlamaRMSNorm

        self.norm = LlamaRMSNorm(hidden, eps)

    def forward(self, y: torch.Tensor, residual: torch.Tensor):
        r = residual + y
        return self.norm(r), r


class Top2MoE(torch.nn.Module):
    """Mixtral-style block on given router logits: softmax in fp32, top-2, renormalise
    (the arithmetic of transformers' ``MixtralTopKRouter.forward``), every expert a gated MLP
    (``act(gate) * up`` then ``down``, as ``MixtralExperts`` computes one expert), combined as a
    weighted sum in fp32. Written densely (every expert sees every token, unselected ones get
    weight zero) so that it traces into one FX graph with a dynamic token dimension."""

    def __init__(self, hidden: int, inter: int, experts: int) -> None:
        super().__init__()
        self.gate_up = torch.nn.Parameter(torch.empty(experts, 2 * inter, hidden))
        self.down = torch.nn.Parameter(torch.empty(experts, hidden, inter))

    def forward(self, x: torch.Tensor, router_logits: torch.Tensor):
        F = torch.nn.functional
        probs = F.softmax(router_logits.float(), dim=-1)
        top_w, top_i = torch.topk(probs, 2, dim=-1)
        top_w = top_w / top_w.sum(dim=-1, keepdim=True)
        dense = torch.zeros_like(probs).scatter(1, top_i, top_w)
        out = torch.zeros_like(x, dtype=torch.float32)
        for e in range(self.gate_up.shape[0]):
            gate, up = F.linear(x, self.gate_up[e]).chunk(2, dim=-1)
            y = F.linear(F.silu(gate) * up, self.down[e])
            out = out + y.float() * dense[:, e:e + 1]
        return out.to(x.dtype), top_i, top_w


def golden_norm_and_moe(ref) -> None:
    import numpy as np

    split = dict(num_nano_batches=2, batch_sizes=[40, 56], batch_indices=[0, 40, 96], num_tokens=[40, 56],
                 num_tokens_padded=[40, 56], split_indices=[0, 40, 96], is_dryrun=False, use_cudagraph=False)
    gen = torch.Generator().manual_seed(11)
    M, H = 96, 256
    mod = AddRMSNorm(H, 1e-5)
    with torch.no_grad():
        mod.norm.weight.copy_(1 + 0.1 * torch.randn(H, generator=gen))
    mod = mod.to(torch.bfloat16).eval()
    # four ranks' partial sums; the collective itself (NCCL in the reference's hosts) cannot run
    # here, so the module is given their fp32 rank-order sum rounded to bf16
    partials = [torch.randn(M, H, generator=gen).to(torch.bfloat16) for _ in range(4)]
    acc = torch.zeros(M, H)
    for p in partials:
        acc += p.float()
    y = acc.to(torch.bfloat16)
    residual = torch.randn(M, H, generator=gen).to(torch.bfloat16)
    (out, new_res), trace, tags = run_reference(mod, (y, residual), split, r"rsqrt", "norm", ref)
    np.savez_compressed(os.path.join(HERE, "norm_split.npz"), y=bits(y), residual=bits(residual),
                        weight=bits(mod.norm.weight), out=bits(out.clone()), new_residual=bits(new_res.clone()),
                        **{f"partial{r}": bits(p) for r, p in enumerate(partials)})
    with open(os.path.join(HERE, "norm_split.json"), "w") as f:
        json.dump({"split": split, "trace": trace, "tags": tags, "eps": 1e-5, "dtype": "bfloat16 as int16 bits"}, f,
                  indent=1)

    gen = torch.Generator().manual_seed(12)
    H, I, E = 64, 96, 8
    moe = Top2MoE(H, I, E)
    with torch.no_grad():
        for p in moe.parameters():
            p.copy_(torch.randn(p.shape, generator=gen) * 0.08)
    moe = moe.to(torch.bfloat16).eval()
    x = torch.randn(M, H, generator=gen).to(torch.bfloat16)
    # No two experts of a token get equal logits: how torch.topk orders equal values is not
    # specified (on this build it does not prefer the lower index), so ties pin nothing.
    logits = (torch.randn(M, E, generator=gen) + 0.05 * torch.stack([torch.randperm(E, generator=gen).float()
                                                                   for _ in range(M)])).to(torch.bfloat16)
    for t in range(M):
        while logits[t].unique().numel() < E:
            logits[t] = (logits[t].float() + 0.03 * torch.randperm(E, generator=gen).float()).to(torch.bfloat16)
    (out, ids, w), trace, tags = run_reference(moe, (x, logits), split, r"topk", "route", ref)
    np.savez_compressed(os.path.join(HERE, "moe_split.npz"), x=bits(x), logits=bits(logits), gate_up=bits(moe.gate_up),
                        down=bits(moe.down), out=bits(out.clone()), ids=ids.clone().numpy().astype(np.int64),
                        weights=w.clone().numpy().astype(np.float32))
    with open(os.path.join(HERE, "moe_split.json"), "w") as f:
        json.dump({"split": split, "trace": trace, "tags": tags, "dtype": "bfloat16 as int16 bits; ids int64; weights fp32"},
                  f, indent=1)


def golden_dbo_trace(ref_iface, ref_cfg) -> dict:
    """Runs the reference's DBO policy (``examples/ae/scheduler/vllm/dbo.py``, unmodified) against a
    scripted engine that hands out tagged operators in program order, and records the order and
    stream in which the policy executes them. The vLLM names the file imports are provided as
    empty stand-ins (vLLM's forward context only carries per-nano-batch attention metadata)."""
    import asyncio
    import types

    current = {"stream": "default"}

    class _NamedStream:
        def __init__(self, *a, **k):
            self.name = None

    class _StreamCtx:
        def __init__(self, s):
            self.s = s

        def __enter__(self):
            self.prev = current["stream"]
            current["stream"] = self.s.name

        def __exit__(self, *a):
            current["stream"] = self.prev

    torch.cuda.Stream = _NamedStream  # type: ignore[misc]
    torch.cuda.stream = lambda s: _StreamCtx(s)  # type: ignore[assignment]

    fwd = types.ModuleType("vllm.forward_context")
    fwd.DPMetadata = type("DPMetadata", (), {})
    forward_ctx = types.SimpleNamespace(attn_metadata=["meta0", "meta1"], dp_metadata=None)
    fwd.get_forward_context = lambda: forward_ctx
    ln = types.ModuleType("vllm.model_executor.layers.layernorm")
    ln.RMSNorm = type("RMSNorm", (torch.nn.Module,), {})
    ds = types.ModuleType("vllm.model_executor.models.deepseek_v2")
    ds.DeepseekV2MoE = type("DeepseekV2MoE", (torch.nn.Module,), {})
    for name, mod in (("vllm", types.ModuleType("vllm")), ("vllm.forward_context", fwd),
                      ("vllm.model_executor", types.ModuleType("vllm.model_executor")),
                      ("vllm.model_executor.layers", types.ModuleType("vllm.model_executor.layers")),
                      ("vllm.model_executor.layers.layernorm", ln),
                      ("vllm.model_executor.models", types.ModuleType("vllm.model_executor.models")),
                      ("vllm.model_executor.models.deepseek_v2", ds)):
        sys.modules[name] = mod
    dbo = load_policy_module(os.path.join(REFERENCE, "examples/ae/scheduler/vllm/dbo.py"), "_ref_dbo")
    cfg = ref_cfg.DynaFlowConfig("x:y", 2, ref_cfg.InductorConfig(False), ref_cfg.CUDAGraphConfig(False, [64]),
                                 {"min_nano_split_tokens": 1})
    policy = dbo.DBOScheduler(cfg)
    policy.comm_stream.name, policy.comp_stream.name = "comm", "comp"

    def layer(i):
        return [(f"pre{i}", []), (f"attn{i}", ["attention", "no-cudagraph"]),
                (f"disp{i}", ["network", "no-inductor", "dispatch"]), (f"exp{i}", ["no-inductor", "expert"]),
                (f"comb{i}", ["network", "no-inductor", "combine"])]

    cases = []
    for layers, batches in ((1, 2), (3, 2), (2, 1)):
        program = sum((layer(i) for i in range(layers)), []) + [("final", [])]
        trace: list = []
        forward_ctx.attn_metadata = ["meta0", "meta1"]   # the policy overwrites it with one entry per operator

        async def drive():
            op_queue = {b: asyncio.Queue(maxsize=10) for b in range(batches)}
            execute_queue: asyncio.Queue = asyncio.Queue()
            split = ref_iface.SplitConfig(batches, [1] * batches, list(range(batches + 1)), [1] * batches,
                                          [1] * batches, list(range(batches + 1)), False, False)
            context = ref_iface.ExecutionContext(split, op_queue, execute_queue)
            cursor = [0] * batches

            async def push(b):
                if cursor[b] < len(program):
                    name, tags = program[cursor[b]]
                    cursor[b] += 1
                    await op_queue[b].put(ref_iface.OperatorHandle(name, b, 1, set(tags), False, False))
                else:
                    await op_queue[b].put(None)

            async def engine():
                for b in range(batches):
                    await push(b)
                remaining = batches * len(program)
                while remaining:
                    ops, _func, done = await execute_queue.get()
                    op = ops[0]
                    trace.append([op.module_name, op.batch_idx, current["stream"]])
                    remaining -= 1
                    await push(op.batch_idx)
                    done.set()

            await asyncio.gather(engine(), policy.schedule(context))

        asyncio.run(drive())
        cases.append({"layers": layers, "batches": batches, "program": program, "trace": trace})
    return {"cases": cases}


def main() -> None:
    install_cpu_shims()
    sys.path.insert(0, REFERENCE)
    sys.path.insert(0, REPO)
    import dynaflow.config as ref_cfg
    import dynaflow.interface as ref_iface
    import dynaflow.manager as ref_manager
    import dynaflow.matching as ref_matching

    from oracle import llama_oracle

    ref = (ref_cfg, ref_iface, ref_matching, ref_manager)

    with open(os.path.join(HERE, "split_configs.json"), "w") as f:
        json.dump(golden_split_configs(ref_iface, ref_cfg), f, indent=1)

    # ---- 2-layer decoder, CPU fp32, 4 x 256 ids, two nano-batches
    shape = llama_oracle.LlamaShape()
    model = llama_oracle.build(shape, seed=0)
    ids = llama_oracle.make_ids(4, 256, shape.vocab, seed=1)
    with torch.inference_mode():
        unsplit = model(ids)
    c1 = {"shape": dataclasses.asdict(shape), "ids_seed": 1, "weights_seed": 0, "runs": []}
    for cuts in ([0, 2, 4], [0, 1, 4]):
        sizes = [cuts[1] - cuts[0], cuts[2] - cuts[1]]
        split = dict(num_nano_batches=2, batch_sizes=sizes, batch_indices=cuts, num_tokens=sizes,
                     num_tokens_padded=sizes, split_indices=cuts, is_dryrun=False, use_cudagraph=False)
        out, trace, tags = run_reference(model, (ids,), split, r"scaled_dot_product_attention", "attention", ref)
        c1["runs"].append({
            "split": split,
            "equal_to_unsplit": bool(torch.equal(out, unsplit)),
            "max_rel_err_vs_unsplit": float((out - unsplit).abs().max() / unsplit.abs().max()),
            "trace": trace,
            "tags": tags,
        })
    sample = unsplit[:, ::32, ::1000].contiguous()
    c1["logits_sample_index"] = "[:, ::32, ::1000]"
    c1["logits_sample"] = sample.tolist()
    c1["logits_abs_max"] = float(unsplit.abs().max())
    c1["logits_sum"] = float(unsplit.double().sum())
    with open(os.path.join(HERE, "c1_llama.json"), "w") as f:
        json.dump(c1, f, indent=1)

    # ---- bf16 gated MLP executed by the reference in two ragged nano-batches
    gen = torch.Generator().manual_seed(7)
    H, I, M = 128, 384, 96
    mlp = llama_oracle.GatedMLP(H, I)
    with torch.no_grad():
        for p in mlp.parameters():
            p.copy_(torch.randn(p.shape, generator=gen) * 0.02 * 4)
    mlp = mlp.to(torch.bfloat16).eval()
    x = torch.randn(M, H, generator=gen).to(torch.bfloat16)
    split = dict(num_nano_batches=2, batch_sizes=[40, 56], batch_indices=[0, 40, 96], num_tokens=[40, 56],
                 num_tokens_padded=[40, 56], split_indices=[0, 40, 96], is_dryrun=False, use_cudagraph=False)
    out, trace, tags = run_reference(mlp, (x,), split, r"silu", "act", ref)
    import numpy as np

    np.savez_compressed(os.path.join(HERE, "mlp_split.npz"), x=bits(x), w_gate=bits(mlp.gate_proj.weight),
                        w_up=bits(mlp.up_proj.weight), w_down=bits(mlp.down_proj.weight), out=bits(out.clone()))
    with open(os.path.join(HERE, "mlp_split.json"), "w") as f:
        json.dump({"split": split, "trace": trace, "tags": tags, "dtype": "bfloat16 as int16 bits"}, f, indent=1)
    golden_norm_and_moe(ref)
    with open(os.path.join(HERE, "dbo_trace.json"), "w") as f:
        json.dump(golden_dbo_trace(ref_iface, ref_cfg), f, indent=1)
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    main()
