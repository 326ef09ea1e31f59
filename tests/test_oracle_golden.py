"""The oracle against the fixtures the reference package produced (tests/golden/make_golden.py)."""
import json
import os

import numpy as np
import torch

from conftest import GOLDEN
from oracle import ops_oracle, split_oracle


def _load(name):
    with open(os.path.join(GOLDEN, name)) as f:
        return json.load(f)


def test_nanoflow_split_matches_reference():
    for entry in _load("split_configs.json")["nanoflow"]:
        c = entry["case"]
        got = split_oracle.nanoflow_split(c["num_tokens"], c["min_tokens"], c["sizes"], c["cg"])
        assert got == entry["split"], c


def test_equal_split_matches_reference():
    for entry in _load("split_configs.json")["equal"]:
        c = entry["case"]
        got = split_oracle.equal_split(c["rows"], c["n"], c["min_tokens"], False)
        assert got == entry["split"], c


def test_round_robin_trace_matches_reference_dispatch_order():
    c1 = _load("c1_llama.json")
    for run in c1["runs"]:
        names = sorted(run["tags"], key=lambda s: int(s.split("_")[1]))
        got = split_oracle.round_robin_trace([names, names])
        assert [list(t) for t in got] == run["trace"]


def test_round_robin_trace_uneven_programs():
    # nano-batch 0 finishes first; removal during iteration skips nano-batch 1 for one round
    got = split_oracle.round_robin_trace([["a"], ["a", "b", "c"]])
    assert got == [("a", 0), ("a", 1), ("b", 1), ("c", 1)]
    assert split_oracle.skewed_trace([["a", "b"], ["a", "b"]]) == [("a", 0), ("b", 0), ("a", 1), ("b", 1)]


def test_slice_and_merge_round_trip():
    rng = np.random.default_rng(0)
    x = rng.integers(0, 1000, size=(37, 5))
    cuts = [0, 11, 37]
    parts = [split_oracle.slice_rows(x, cuts, b) for b in range(2)]
    assert parts[0].shape[0] == 11 and parts[1].shape[0] == 26
    assert np.array_equal(split_oracle.merge_rows(parts), x)
    empty = split_oracle.slice_rows(x, [0, 0, 37], 0)
    assert empty.shape == (0, 5)


def _bf16(bits):
    return torch.from_numpy(bits).view(torch.bfloat16)


def test_gated_mlp_oracle_matches_reference_execution():
    z = np.load(os.path.join(GOLDEN, "mlp_split.npz"))
    x, wg, wu, wd, ref_out = (_bf16(z[k]) for k in ("x", "w_gate", "w_up", "w_down", "out"))
    # the operator chain the reference executed (HF form), bit for bit, also when split at the golden cut
    assert torch.equal(ops_oracle.gated_mlp_hf(x, wg, wu, wd), ref_out)
    cuts = _load("mlp_split.json")["split"]["split_indices"]
    parts = [ops_oracle.gated_mlp_hf(x[cuts[i]:cuts[i + 1]], wg, wu, wd) for i in range(2)]
    assert torch.equal(torch.cat(parts), ref_out)
    # the fused-epilogue form (one rounding after silu*mul) stays within the bf16 tolerance
    fused = ops_oracle.gated_mlp(x, wg, wu, wd)
    rel = (fused.float() - ref_out.float()).abs().max() / ref_out.float().abs().max()
    assert rel <= 2e-2


def test_allreduce_add_rmsnorm_oracle_matches_reference_execution():
    """The residual add + RMSNorm (transformers' LlamaRMSNorm, bf16, eps 1e-5) that the reference
    engine executed in two ragged nano-batches: the oracle reproduces both outputs bit for bit,
    from the four ranks' partial sums (their fp32 rank-order sum is what the module was fed)."""
    z = np.load(os.path.join(GOLDEN, "norm_split.npz"))
    parts = [_bf16(z[f"partial{r}"]) for r in range(4)]
    residual, weight = _bf16(z["residual"]), _bf16(z["weight"])
    eps = _load("norm_split.json")["eps"]
    out, new_res = ops_oracle.allreduce_add_rmsnorm(parts, residual, weight, eps=eps)
    assert torch.equal(out, _bf16(z["out"])) and torch.equal(new_res, _bf16(z["new_residual"]))
    out1, res1 = ops_oracle.allreduce_add_rmsnorm([_bf16(z["y"])], residual, weight, eps=eps)
    assert torch.equal(out1, out) and torch.equal(res1, new_res)
    cuts = _load("norm_split.json")["split"]["split_indices"]
    for i in range(2):                                   # per nano-batch, as the engine ran it
        sl = slice(cuts[i], cuts[i + 1])
        o, r = ops_oracle.allreduce_add_rmsnorm([p[sl] for p in parts], residual[sl], weight, eps=eps)
        assert torch.equal(o, _bf16(z["out"])[sl]) and torch.equal(r, _bf16(z["new_residual"])[sl])


def test_top2_moe_oracle_matches_reference_execution():
    """The Mixtral-style top-2 block the reference engine executed in two ragged nano-batches:
    expert ids and routing weights bit for bit; the layer output bit for bit with the experts in
    the operator-chain form the fixture ran, and within the bf16 tolerance in the fused-epilogue
    form the CUDA kernels implement."""
    z = np.load(os.path.join(GOLDEN, "moe_split.npz"))
    x, logits, gate_up, down, ref_out = (_bf16(z[k]) for k in ("x", "logits", "gate_up", "down", "out"))
    w, ids = ops_oracle.top2_route(logits)
    assert torch.equal(ids, torch.from_numpy(z["ids"])) and torch.equal(w, torch.from_numpy(z["weights"]))
    inter = gate_up.shape[1] // 2
    wg, wu = gate_up[:, :inter], gate_up[:, inter:]
    assert torch.equal(ops_oracle.moe_layer(x, logits, wg, wu, down, mlp=ops_oracle.gated_mlp_hf), ref_out)
    fused = ops_oracle.moe_layer(x, logits, wg, wu, down)
    assert ((fused.float() - ref_out.float()).abs().max() / ref_out.float().abs().max()).item() <= 2e-2


def test_allreduce_add_rmsnorm_oracle_properties():
    g = torch.Generator().manual_seed(3)
    parts = [torch.randn(5, 64, generator=g).bfloat16() for _ in range(4)]
    res = torch.randn(5, 64, generator=g).bfloat16()
    w = torch.randn(64, generator=g).bfloat16()
    out, new_res = ops_oracle.allreduce_add_rmsnorm(parts, res, w)
    ref_sum = sum(p.float() for p in parts)
    assert torch.allclose(new_res.float(), ref_sum.bfloat16().float() + res.float(), atol=0.07, rtol=1e-2)
    # residual absent == residual of zeros
    out0, res0 = ops_oracle.allreduce_add_rmsnorm(parts, None, w)
    out1, res1 = ops_oracle.allreduce_add_rmsnorm(parts, torch.zeros_like(res), w)
    assert torch.equal(out0, out1) and torch.equal(res0, res1)
    # unit weight: rows have unit RMS
    ones = torch.ones(64).bfloat16()
    out2, _ = ops_oracle.allreduce_add_rmsnorm(parts, res, ones)
    assert torch.allclose(out2.float().pow(2).mean(-1), torch.ones(5), atol=2e-2)


def test_top2_route_and_moe_layer():
    g = torch.Generator().manual_seed(5)
    logits = torch.randn(32, 8, generator=g)
    w, ids = ops_oracle.top2_route(logits)
    assert torch.allclose(w.sum(-1), torch.ones(32)) and (ids[:, 0] != ids[:, 1]).all()
    assert torch.equal(ids[:, 0], logits.argmax(-1))
    x = torch.randn(32, 16, generator=g)
    wg = torch.randn(8, 24, 16, generator=g) * 0.1
    wu = torch.randn(8, 24, 16, generator=g) * 0.1
    wd = torch.randn(8, 16, 24, generator=g) * 0.1
    y = ops_oracle.moe_layer(x, logits, wg, wu, wd)
    t = 7
    manual = sum(w[t, s] * ops_oracle.gated_mlp(x[t:t + 1], wg[ids[t, s]], wu[ids[t, s]], wd[ids[t, s]]) for s in range(2))
    assert torch.allclose(y[t], manual[0], atol=1e-5)


def test_dbo_trace_matches_reference_policy():
    for case in _load("dbo_trace.json")["cases"]:
        program = [(n, t) for n, t in case["program"]]
        got = split_oracle.dbo_trace([program] * case["batches"])
        assert [list(x) for x in got] == case["trace"], (case["layers"], case["batches"])


def test_causal_attention_oracle_matches_pytorch_sdpa():
    """The attention restatement against torch's own scaled_dot_product_attention (the operator
    the CPU parity configuration's decoder calls), ragged sequences, grouped heads, fp32."""
    g = torch.Generator().manual_seed(21)
    lens, hq, hkv, d = [5, 33, 1], 4, 2, 16
    T = sum(lens)
    q, k, v = (torch.randn(T, h, d, generator=g) for h in (hq, hkv, hkv))
    got = ops_oracle.causal_attention(q, k, v, lens)
    start = 0
    for n in lens:
        qs, ks, vs = (t[start:start + n].transpose(0, 1).unsqueeze(0) for t in (q, k, v))
        want = torch.nn.functional.scaled_dot_product_attention(
            qs, ks.repeat_interleave(hq // hkv, dim=1), vs.repeat_interleave(hq // hkv, dim=1), is_causal=True)
        assert torch.allclose(got[start:start + n], want[0].transpose(0, 1), atol=1e-5, rtol=1e-5)
        start += n
