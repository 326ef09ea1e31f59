"""The drop-in path end to end on the GPU: a traced Llama-style decoder is partitioned by a
policy, executed as two nano-batches on two streams, with the gated-MLP subgraphs replaced by
the native kernels; then the same under per-subgraph CUDA-graph capture and replay."""
import pytest
import torch

from helpers import Host, make_config, two_way
from dynaflow_b200.interface import InputInfo, SplitConfig
from dynaflow_b200.matching import MatchingRule, Op
from dynaflow_b200.policies import NanoFlowScheduler, gated_mlp_rule, native_gated_mlp
from oracle import llama_oracle

pytestmark = pytest.mark.gpu

TOL = 2e-2
SHAPE = llama_oracle.LlamaShape(hidden=256, intermediate=512, heads=4, kv_heads=4, head_dim=64, layers=2, vocab=512)


def _rel(a, b):
    return ((a.float() - b.float()).abs().max() / b.float().abs().max()).item()


def _policy(config, native=True):
    attn = MatchingRule(condition=Op(pattern=r"scaled_dot_product_attention"))
    mlp = gated_mlp_rule()
    policy = NanoFlowScheduler(config, split_rules=[mlp, attn],
                               tag_rules={mlp: {"mlp"}, attn: {"attention", "no-cudagraph"}})
    if native:
        policy.substitutions["mlp"] = native_gated_mlp
    return policy


@pytest.fixture(scope="module")
def model(native_lib):
    assert torch.cuda.is_available()
    return llama_oracle.build(SHAPE, seed=0, dtype=torch.bfloat16).cuda()


def test_split_forward_with_native_mlp_matches_unsplit_pytorch(model):
    from dynaflow_b200 import ops

    ids = llama_oracle.make_ids(6, 32, SHAPE.vocab).cuda()
    with torch.inference_mode():
        want = model(ids)
    host = Host(model, _policy(make_config()))
    for cuts in ([0, 3, 6], [0, 1, 6]):
        got = host.run((ids,), two_way(cuts))
        torch.cuda.synchronize()
        ops.check_status()
        assert got.shape == want.shape and _rel(got, want) <= TOL, cuts
    trace = host.manager.engine.last_trace
    assert sum(1 for *_, substituted in trace if substituted) == 2 * SHAPE.layers   # every MLP, both nano-batches
    assert len({stream for _n, _b, stream, _s in trace}) >= 1
    # routing is bit-exact: same dispatch order as the oracle's round-robin restatement
    from oracle import split_oracle

    names = sorted(host.tags, key=lambda s: int(s.split("_")[1]))
    assert [(n, b) for n, b, _s, _f in trace] == split_oracle.round_robin_trace([names, names])


def test_pytorch_subgraphs_only_are_bit_identical_to_unsplit(model):
    """Without substitution the split run executes the very same PyTorch kernels on row
    slices; with an even split of equal-length requests the merge is exact."""
    ids = llama_oracle.make_ids(4, 16, SHAPE.vocab).cuda()
    with torch.inference_mode():
        want = model(ids)
    host = Host(model, _policy(make_config(), native=False))
    got = host.run((ids,), two_way([0, 2, 4]))
    assert _rel(got, want) <= 1e-2  # bf16 GEMMs may pick another kernel for the half batch
    assert got.shape == want.shape


@pytest.mark.parametrize("mixed", [False, True])
def test_cudagraph_capture_and_replay_two_nano_batches(model, mixed):
    """mixed=False: every subgraph is captured and replayed, strict pointer check (the reference's
    contract). mixed=True: attention runs eagerly and the MLPs run on the native kernels between
    captured subgraphs; their fresh outputs are copied into the captured inputs."""
    from dynaflow_b200 import ops

    config = make_config(capture_sizes=(2, 4, 8), cudagraph=True, copy_inputs=mixed, max_static_rows=16,
                         min_nano_split_tokens=1)
    if mixed:
        policy = _policy(config)
    else:
        attn = MatchingRule(condition=Op(pattern=r"scaled_dot_product_attention"))
        policy = NanoFlowScheduler(config, split_rules=[attn], tag_rules={attn: {"attention"}})
    host = Host(model, policy, config)
    manager = host.manager
    seq = 16
    ids = llama_oracle.make_ids(8, seq, SHAPE.vocab, seed=3).cuda()
    with torch.inference_mode():
        want = model(ids)
    # first call traces and initialises; dry runs capture one graph per (subgraph, slot, size)
    for size in (8, 4, 2):
        x = ids[:size].contiguous()
        torch._dynamo.mark_dynamic(x, 0)
        manager.prepare(size, [1] * size, is_dryrun=True, use_cudagraph=True)
        with torch.inference_mode():
            out = host.compiled(x)
        assert out.shape[0] == size
    torch.cuda.synchronize()
    # live: 8 requests -> two nano-batches of 4 (capture size 4), replayed from the graphs
    cfg = policy.get_split_config(InputInfo(8, [1] * 8, 8), use_cudagraph=True)
    assert cfg.num_nano_batches == 2 and cfg.use_cudagraph and cfg.num_tokens_padded == [4, 4]
    manager.override_split_config(cfg)
    torch._dynamo.mark_dynamic(ids, 0)
    with torch.inference_mode():
        got = host.compiled(ids)
    torch.cuda.synchronize()
    ops.check_status()
    assert _rel(got, want) <= TOL
    # ragged: 5 requests -> nano-batches of 2 and 3 rows, padded to capture sizes 2 and 4
    ids5 = ids[:5].contiguous()
    cfg = policy.get_split_config(InputInfo(5, [1] * 5, 5), use_cudagraph=True)
    assert cfg.num_tokens == [2, 3] and cfg.num_tokens_padded == [2, 4]
    manager.override_split_config(cfg)
    torch._dynamo.mark_dynamic(ids5, 0)
    with torch.inference_mode():
        got5 = host.compiled(ids5)
    torch.cuda.synchronize()
    # padded rows are computed too (stale static-buffer rows) and come back with the merge:
    # nano-batch outputs are [2 + 4] rows, of which rows 0-1 and 2-4 are the real ones
    assert got5.shape[0] == 6
    real = torch.cat([got5[:2], got5[2:5]])
    with torch.inference_mode():
        want5 = model(ids5)
    assert _rel(real, want5) <= TOL
    # a size that was never captured must be refused outside a dry run
    bad = SplitConfig(2, [3, 3], [0, 3, 6], [3, 3], [3, 3], [0, 3, 6], is_dryrun=False, use_cudagraph=True)
    manager.override_split_config(bad)
    ids6 = ids[:6].contiguous()
    torch._dynamo.mark_dynamic(ids6, 0)
    with pytest.raises(AssertionError, match="dry run"):
        with torch.inference_mode():
            host.compiled(ids6)


def test_whole_forward_graph_replays_the_recorded_schedule(model):
    """The policy runs live once per split shape, under stream capture; later forwards of that
    shape are one graph launch and must give the same rows; a new shape captures again."""
    import time

    from dynaflow_b200 import ops

    ids = llama_oracle.make_ids(6, 32, SHAPE.vocab, seed=5).cuda()
    ids_b = llama_oracle.make_ids(6, 32, SHAPE.vocab, seed=6).cuda()
    with torch.inference_mode():
        want, want_b = model(ids), model(ids_b)

    eager = Host(model, _policy(make_config()))
    got_eager = eager.run((ids,), two_way([0, 3, 6])).clone()
    eager_trace = [(n, b, s) for n, b, _st, s in eager.manager.engine.last_trace]

    config = make_config(whole_forward_graph=True)
    host = Host(model, _policy(config), config)
    first = host.run((ids,), two_way([0, 3, 6])).clone()          # warm-up + capture + first replay
    graphs = host.manager.forward_graphs
    assert graphs is not None and graphs.captures == 1
    second = host.run((ids_b,), two_way([0, 3, 6])).clone()        # replay with new inputs, no policy run
    assert graphs.captures == 1
    torch.cuda.synchronize()
    ops.check_status()
    assert torch.equal(first, got_eager)                           # same kernels, same order
    assert _rel(first, want) <= TOL and _rel(second, want_b) <= TOL
    entry = next(iter(graphs._entries.values()))
    assert [(n, b, s) for n, b, _st, s in entry.trace] == eager_trace   # the recorded routing
    assert entry.replays == 2
    third = host.run((ids,), two_way([0, 1, 6]))                   # another split shape: second capture
    assert graphs.captures == 2 and _rel(third, want) <= TOL

    # dispatch cost: eager split forward (policy + engine per operator) vs one graph launch
    def avg_ms(h, n=30):
        for _ in range(3):
            h.run((ids,), two_way([0, 3, 6]))
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(n):
            h.run((ids,), two_way([0, 3, 6]))
        torch.cuda.synchronize()
        return (time.perf_counter() - t0) / n * 1e3

    t_eager, t_graph = avg_ms(eager), avg_ms(host)
    print(f"split forward, 2 layers, 2 nano-batches: eager dispatch {t_eager:.3f} ms, graph replay {t_graph:.3f} ms")
    assert t_graph < t_eager


def test_layer_step_through_the_manager_matches_oracle(native_lib):
    """The gated-MLP layer step driven through DynaFlowManager.get_callable(): policy, split into two
    ragged nano-batches, native substitution of the MLP subgraph, merge; eagerly dispatched and as a
    whole-forward graph; against the CPU oracle."""
    from dynaflow_b200 import ops
    from dynaflow_b200.host_step import ManagedLayerStep
    from dynaflow_b200.layer import TensorParallelGatedMLP
    from oracle import ops_oracle

    H, I, rows = 256, 1024, 320
    g = torch.Generator().manual_seed(40)
    w = tuple((torch.randn(s, generator=g) * 0.05).bfloat16() for s in ((I, H), (I, H), (H, I)))
    x = torch.randn(rows, H, generator=g).bfloat16()
    want = ops_oracle.gated_mlp(x, *w)
    layer = TensorParallelGatedMLP(H, I, max_rows=rows, micro_batches=2, weights=w)
    for graph in (False, True):
        step = ManagedLayerStep(layer, whole_forward_graph=graph)
        for cuts in ([0, 128, 320], [0, 200, 320], [0, 128, 320]):
            got = step(x.cuda(), cuts).clone()
            torch.cuda.synchronize()
            ops.check_status()
            assert _rel(got.cpu(), want) <= TOL, (graph, cuts)
            assert step.substituted_per_step == 2          # the MLP subgraph of both nano-batches
