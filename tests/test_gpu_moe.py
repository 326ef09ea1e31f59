"""Top-2 MoE: routing and token movement kernels bit-exact against the oracle, the expert MLP over
a device-side row count, and the whole layer within the bf16 tolerance."""
import pytest
import torch

pytestmark = pytest.mark.gpu

TOL = 2e-2


def _rel(got, want):
    return ((got.float().cpu() - want.float()).abs().max() / want.float().abs().max()).item()


@pytest.fixture(scope="module")
def lib(native_lib):
    assert torch.cuda.is_available()
    return native_lib


def test_routing_and_selection_are_bit_exact(lib):
    from oracle import ops_oracle

    g = torch.Generator().manual_seed(0)
    T, E = 3000, 8
    logits = torch.randn(T, E, generator=g).bfloat16()
    logits[5] = logits[5, 0]                      # an all-equal row: ties resolve to the lowest indices
    logits[7, 3] = logits[7, 6] = 4.0             # a tie for first place
    want_w, want_ids = ops_oracle.top2_route(logits)
    dev = logits.cuda()
    ids = torch.empty(T, 2, dtype=torch.int32, device="cuda")
    w = torch.empty(T, 2, dtype=torch.float32, device="cuda")
    assert lib.df_moe_route_top2(dev.data_ptr(), T, E, ids.data_ptr(), w.data_ptr(), None) == 0
    torch.cuda.synchronize()
    assert torch.equal(ids.cpu().long(), want_ids)                       # routing: bit-exact
    assert torch.allclose(w.cpu(), want_w, rtol=1e-5, atol=1e-6)
    assert ids[5].tolist() == [0, 1] and ids[7].tolist() == [3, 6]
    rows = torch.empty(T, dtype=torch.int32, device="cuda")
    slot = torch.empty(T, dtype=torch.int32, device="cuda")
    pos = torch.empty(T, dtype=torch.int32, device="cuda")
    count = torch.zeros(1, dtype=torch.int32, device="cuda")
    total = 0
    for e in range(E):
        assert lib.df_moe_select_rows(ids.data_ptr(), T, e, rows.data_ptr(), slot.data_ptr(), pos.data_ptr(),
                                      count.data_ptr(), None) == 0
        torch.cuda.synchronize()
        want_rows, want_slot = torch.nonzero(want_ids == e, as_tuple=True)
        n = int(count.item())
        assert n == want_rows.numel()
        assert torch.equal(rows[:n].cpu().long(), want_rows) and torch.equal(slot[:n].cpu().long(), want_slot)
        inv = torch.full((T,), -1, dtype=torch.long)
        inv[want_rows] = torch.arange(n)
        assert torch.equal(pos.cpu().long(), inv)
        total += n
    assert total == 2 * T                                                  # every token went to two experts


def test_gather_mlp_scatter_with_device_row_count(lib):
    from dynaflow_b200 import ops
    from oracle import ops_oracle

    g = torch.Generator().manual_seed(1)
    T, H, I = 500, 256, 512
    x = torch.randn(T, H, generator=g).bfloat16()
    wg, wu, wd = [(torch.randn(s, generator=g) * 0.05).bfloat16() for s in ((I, H), (I, H), (H, I))]
    picked = torch.sort(torch.randperm(T, generator=g)[:137]).values
    rows = torch.zeros(T, dtype=torch.int32)
    rows[:137] = picked.int()
    count = torch.tensor([137], dtype=torch.int32)
    xd, rd, cd = x.cuda(), rows.cuda(), count.cuda()
    wgd, wud, wdd = wg.cuda(), wu.cuda(), wd.cuda()     # kept alive: the calls below only see raw pointers
    packed = torch.full((T, H), float("nan"), dtype=torch.bfloat16, device="cuda")
    assert lib.df_moe_gather_rows(xd.data_ptr(), rd.data_ptr(), cd.data_ptr(), T, H, packed.data_ptr(), None) == 0
    torch.cuda.synchronize()
    assert torch.equal(packed[:137].cpu(), x[picked])
    assert torch.isnan(packed[137:].float()).all()                        # rows beyond the count are not touched
    out = torch.full((T, H), float("nan"), dtype=torch.bfloat16, device="cuda")
    ws = torch.empty(ops.mlp_workspace_bytes(T, H, I), dtype=torch.uint8, device="cuda")
    st = ops.status_block()
    rc = lib.df_mlp_gated_bf16_rows_on_device(packed.data_ptr(), wgd.data_ptr(), wud.data_ptr(), wdd.data_ptr(),
                                              out.data_ptr(), ws.data_ptr(), T, cd.data_ptr(), H, I, 0, st.data_ptr(), None)
    assert rc == 0
    torch.cuda.synchronize()
    ops.check_status()
    want = ops_oracle.gated_mlp(x[picked], wg, wu, wd)
    assert _rel(out[:137], want) <= TOL
    assert torch.isnan(out[256:].float()).all()                            # tiles past the count never ran
    # a count of zero is a no-op
    cd.zero_()
    out.fill_(float("nan"))
    lib.df_mlp_gated_bf16_rows_on_device(packed.data_ptr(), wgd.data_ptr(), wud.data_ptr(), wdd.data_ptr(),
                                         out.data_ptr(), ws.data_ptr(), T, cd.data_ptr(), H, I, 0, st.data_ptr(), None)
    torch.cuda.synchronize()
    ops.check_status()
    assert torch.isnan(out.float()).all()


@pytest.mark.parametrize("T,H,I,E", [(256, 256, 512, 8), (1000, 512, 1024, 8)])
def test_single_rank_moe_layer_matches_oracle(lib, T, H, I, E):
    from dynaflow_b200 import ops
    from dynaflow_b200.moe import ExpertParallelMoE
    from oracle import ops_oracle

    g = torch.Generator().manual_seed(2)
    x = torch.randn(T, H, generator=g).bfloat16()
    logits = torch.randn(T, E, generator=g).bfloat16()
    w_gate = (torch.randn(E, I, H, generator=g) * 0.05).bfloat16()
    w_up = (torch.randn(E, I, H, generator=g) * 0.05).bfloat16()
    w_down = (torch.randn(E, H, I, generator=g) * 0.05).bfloat16()
    layer = ExpertParallelMoE(H, I, E, T, weights=(w_gate, w_up, w_down), slots=1)
    got = layer.forward(x.cuda(), logits.cuda()).clone()
    again = layer.forward(x.cuda(), logits.cuda())
    torch.cuda.synchronize()
    ops.check_status()
    assert torch.equal(got, again)
    want = ops_oracle.moe_layer(x, logits, w_gate, w_up, w_down)
    assert _rel(got, want) <= TOL


def test_moe_layer_against_reference_executed_fixture(lib):
    """The Mixtral-style top-2 block the reference engine executed in two ragged nano-batches
    (tests/golden/moe_split.npz): expert ids bit-exact, routing weights to fp32 rounding, layer
    output within the bf16 tolerance, nano-batch by nano-batch."""
    import json
    import os

    import numpy as np

    from conftest import GOLDEN
    from dynaflow_b200 import ops
    from dynaflow_b200.moe import ExpertParallelMoE

    z = np.load(os.path.join(GOLDEN, "moe_split.npz"))
    cuts = json.load(open(os.path.join(GOLDEN, "moe_split.json")))["split"]["split_indices"]
    x, logits, gate_up, down, ref_out = (torch.from_numpy(z[k]).view(torch.bfloat16)
                                         for k in ("x", "logits", "gate_up", "down", "out"))
    E, inter, H = gate_up.shape[0], gate_up.shape[1] // 2, gate_up.shape[2]
    weights = (gate_up[:, :inter].contiguous(), gate_up[:, inter:].contiguous(), down)
    for i in range(2):
        sl = slice(cuts[i], cuts[i + 1])
        T = cuts[i + 1] - cuts[i]
        layer = ExpertParallelMoE(H, inter, E, T, weights=weights, slots=1)
        got = layer.forward(x[sl].cuda(), logits[sl].cuda())
        torch.cuda.synchronize()
        ops.check_status()
        assert torch.equal(layer.ids[0].cpu().long(), torch.from_numpy(z["ids"])[sl])
        assert torch.allclose(layer.route_w[0].cpu(), torch.from_numpy(z["weights"])[sl], rtol=1e-5, atol=1e-6)
        assert _rel(got, ref_out[sl]) <= TOL


@pytest.mark.parametrize("world,T,H", [(2, 64, 256), (8, 800, 1024), (4, 36, 64)])
def test_emulated_all_gather_and_reduce_scatter(lib, world, T, H):
    """The two halves of the all-reduce as collectives of their own (expert parallelism)."""
    from dynaflow_b200 import ops
    from dynaflow_b200.comm import EmulatedComm
    from dynaflow_b200._native import df_comm_rank_t

    g = torch.Generator().manual_seed(3)
    data = [torch.randn(T, H, generator=g).bfloat16() for _ in range(world)]
    em = EmulatedComm(world, max_rows=max(T, 64), hidden=H, n_ctas=4)

    def run(code):
        views = (df_comm_rank_t * world)()
        for r in range(world):
            views[r] = em._view(r, em.ptrs)
        rc = lib.df_allreduce_emulated_bf16(views, world, em.max_rows, H, T, None, 0.0, code, em.n_ctas,
                                            ops.status_block().data_ptr(), torch.cuda.current_stream().cuda_stream)
        assert rc == 0
        torch.cuda.synchronize()
        ops.check_status()

    # all-gather: rank r contributes its slice of data[r]
    full = torch.zeros(T, H).bfloat16()
    for r in range(world):
        lo, hi = T * r // world, T * (r + 1) // world
        em.partial(r, T).copy_(data[r])
        em.result(r, T).zero_()
        full[lo:hi] = data[r][lo:hi]
    run(4)
    for r in range(world):
        assert torch.equal(em.result(r, T).cpu(), full), r
    # reduce-scatter: every rank contributes T rows; rank r receives the sum of slice r
    acc = torch.zeros(T, H)
    for r in range(world):
        em.partial(r, T).copy_(data[r])
        em.result(r, T).zero_()
        acc += data[r].float()
    want = acc.bfloat16()
    run(3)
    for r in range(world):
        lo, hi = T * r // world, T * (r + 1) // world
        got = em.result(r, T).cpu()
        assert torch.equal(got[lo:hi], want[lo:hi]), r
        keep = torch.ones(T, dtype=torch.bool)
        keep[lo:hi] = False
        assert got[keep].abs().sum() == 0                                   # nothing written outside the own slice


# ------------------------------------------------------------------ all-to-all form
def test_a2a_plan_positions_and_counts(lib):
    g = torch.Generator().manual_seed(50)
    T, E = 1000, 8
    ids = torch.stack([torch.randperm(E, generator=g)[:2] for _ in range(T)]).int()
    dev = ids.cuda()
    pos = torch.empty(T, 2, dtype=torch.int32, device="cuda")
    counts = torch.zeros(E, dtype=torch.int32, device="cuda")
    assert lib.df_a2a_plan(dev.data_ptr(), T, E, pos.data_ptr(), counts.data_ptr(), None) == 0
    torch.cuda.synchronize()
    flat = ids.flatten()
    want_pos = torch.empty_like(flat)
    seen = [0] * E
    for i, e in enumerate(flat.tolist()):
        want_pos[i] = seen[e]
        seen[e] += 1
    assert torch.equal(pos.cpu().flatten(), want_pos) and counts.cpu().tolist() == seen


@pytest.mark.parametrize("world,Tr,H,E", [(2, 64, 256, 8), (8, 100, 512, 8), (4, 37, 64, 16)])
def test_emulated_a2a_dispatch_and_combine(lib, world, Tr, H, E):
    """All ranks of the all-to-all as one cooperative launch on one GPU: every routed row lands in the
    owner's packed input grouped by source rank in token order (bit-exact), the arrived-row counts are
    right, and the combine pulls each token's two expert rows back with its routing weights."""
    import ctypes

    from dynaflow_b200 import ops
    from dynaflow_b200._native import df_a2a_rank_t
    from oracle import ops_oracle

    g = torch.Generator().manual_seed(51 + world)
    cap, per = Tr * world, E // world
    xs = [torch.randn(Tr, H, generator=g).bfloat16() for _ in range(world)]
    routed = [ops_oracle.top2_route(torch.randn(Tr, E, generator=g).bfloat16()) for _ in range(world)]
    nbytes = lib.df_a2a_region_bytes(world, E, cap, H)
    in_off, out_off = lib.df_a2a_packed_in_offset(world, E, cap, H), lib.df_a2a_packed_out_offset(world, E, cap, H)
    rows_off = lib.df_a2a_rows_total_offset()
    regions = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(world)]
    views = (df_a2a_rank_t * world)()
    for r in range(world):
        views[r].rank = r
        for q in range(world):
            views[r].regions[q] = regions[q].data_ptr()
    x_dev = [x.cuda() for x in xs]
    ids_dev = [ids.int().cuda() for _w, ids in routed]
    w_dev = [w.float().cuda() for w, _ids in routed]
    pos_dev = [torch.empty(Tr, 2, dtype=torch.int32, device="cuda") for _ in range(world)]
    cnt_dev = [torch.zeros(E, dtype=torch.int32, device="cuda") for _ in range(world)]
    out_dev = [torch.zeros(Tr, H, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    for r in range(world):
        assert lib.df_a2a_plan(ids_dev[r].data_ptr(), Tr, E, pos_dev[r].data_ptr(), cnt_dev[r].data_ptr(), None) == 0

    def ptrs(ts):
        return (ctypes.c_void_p * world)(*[t.data_ptr() for t in ts])

    st = ops.status_block()
    for call in range(2):                                            # the flags carry a sequence number: twice
        rc = lib.df_a2a_emulated_bf16(views, world, E, cap, H, Tr, ptrs(x_dev), ptrs(ids_dev), ptrs(pos_dev), ptrs(cnt_dev),
                                      None, None, 0, 4, st.data_ptr(), None)
        assert rc == 0
        torch.cuda.synchronize()
        ops.check_status()
        for e in range(E):
            d, el = e // per, e % per
            want_rows = torch.cat([xs[s][(routed[s][1] == e).any(dim=1)] for s in range(world)])
            n = want_rows.shape[0]
            total = regions[d][rows_off + 4 * el: rows_off + 4 * el + 4].view(torch.int32).item()
            assert total == n, (e, total, n)
            got = regions[d][in_off + el * cap * H * 2: in_off + (el * cap + n) * H * 2].view(torch.bfloat16).view(n, H)
            assert torch.equal(got.cpu(), want_rows), e
            # stand-in for the expert: its output rows are the input rows scaled by (e + 1) / 8
            out_rows = regions[d][out_off + el * cap * H * 2: out_off + (el * cap + n) * H * 2].view(torch.bfloat16).view(n, H)
            out_rows.copy_((got.float() * ((e + 1) / 8)).bfloat16())
        rc = lib.df_a2a_emulated_bf16(views, world, E, cap, H, Tr, None, ptrs(ids_dev), ptrs(pos_dev), None, ptrs(w_dev),
                                      ptrs(out_dev), 1, 4, st.data_ptr(), None)
        assert rc == 0
        torch.cuda.synchronize()
        ops.check_status()
        for r in range(world):
            w, ids = routed[r]
            y = [(xs[r].float() * ((ids[:, c].float() + 1) / 8).unsqueeze(1)).bfloat16().float() for c in range(2)]
            want = (y[0] * w[:, 0:1] + y[1] * w[:, 1:2]).bfloat16()
            assert _rel(out_dev[r], want) <= 1e-2, (call, r)


@pytest.mark.parametrize("T,H,I,E", [(300, 256, 512, 8), (64, 128, 256, 16)])
def test_single_rank_moe_layer_all_to_all_form(lib, T, H, I, E):
    from dynaflow_b200 import ops
    from dynaflow_b200.moe import ExpertParallelMoE
    from oracle import ops_oracle

    g = torch.Generator().manual_seed(52)
    x = torch.randn(T, H, generator=g).bfloat16()
    logits = torch.randn(T, E, generator=g).bfloat16()
    w = tuple((torch.randn(*s, generator=g) * 0.05).bfloat16() for s in ((E, I, H), (E, I, H), (E, H, I)))
    layer = ExpertParallelMoE(H, I, E, T, weights=w, slots=1, exchange="a2a", n_ctas=8)
    got = layer.forward(x.cuda(), logits.cuda()).clone()
    again = layer.forward(x.cuda(), logits.cuda())
    torch.cuda.synchronize()
    ops.check_status()
    assert torch.equal(got, again)
    assert _rel(got, ops_oracle.moe_layer(x, logits, *w)) <= TOL
    layer.close()
