"""The peer-memory all-reduce (+ residual + RMSNorm) kernel against the CPU oracle.

On one GPU the ranks are emulated as one cooperative launch over all ranks' regions
(blocks of different ranks wait on one another, so they must be co-resident); the
multi-process form is covered by tests/test_gpu_multi.py.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu

TOL = 2e-2


def _rel(got, want):
    return ((got.float().cpu() - want.float()).abs().max() / want.float().abs().max()).item()


@pytest.fixture(scope="module")
def comm_mod(native_lib):
    from dynaflow_b200 import comm

    return comm


@pytest.mark.parametrize("world,T,H,n_ctas", [(2, 64, 256, 4), (4, 100, 512, 8), (8, 37, 4096, 8), (3, 5, 64, 2),
                                               (8, 1024, 4096, 16), (1, 16, 128, 2)])
def test_emulated_allreduce_matches_oracle(comm_mod, world, T, H, n_ctas):
    from dynaflow_b200 import ops

    g = torch.Generator().manual_seed(world * 1000 + T)
    parts = [torch.randn(T, H, generator=g).bfloat16() for _ in range(world)]
    em = comm_mod.EmulatedComm(world, max_rows=max(T, 128), hidden=H, n_ctas=n_ctas)
    acc = torch.zeros(T, H)
    for p in parts:
        acc += p.float()
    want = acc.bfloat16()
    for call in range(3):  # repeated calls reuse the flags with a growing sequence number
        for r in range(world):
            em.partial(r, T).copy_(parts[r])
            em.result(r, T).zero_()
        em.run(T)
        torch.cuda.synchronize()
        ops.check_status()
        for r in range(world):
            assert torch.equal(em.result(r, T).cpu(), want), (call, r)   # fp32 sum in rank order: bit-exact


@pytest.mark.parametrize("world,T,H", [(2, 48, 256), (8, 200, 4096), (4, 33, 1024)])
@pytest.mark.parametrize("with_residual", [True, False])
def test_emulated_fused_rmsnorm_matches_oracle(comm_mod, world, T, H, with_residual):
    from dynaflow_b200 import ops
    from oracle import ops_oracle

    g = torch.Generator().manual_seed(7 * world + T)
    parts = [torch.randn(T, H, generator=g).bfloat16() for _ in range(world)]
    residual = torch.randn(T, H, generator=g).bfloat16() if with_residual else None
    weight = (1.0 + 0.1 * torch.randn(H, generator=g)).bfloat16()
    want_out, want_res = ops_oracle.allreduce_add_rmsnorm(parts, residual, weight, eps=1e-5)
    em = comm_mod.EmulatedComm(world, max_rows=256, hidden=H, n_ctas=8)
    for r in range(world):
        em.partial(r, T).copy_(parts[r])
    res_in = [residual.cuda() for _ in range(world)] if with_residual else None
    res_out = [torch.empty(T, H, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    outs = [torch.empty(T, H, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    em.run(T, weight=weight.cuda(), residual_in=res_in, residual_out=res_out, out=outs)
    torch.cuda.synchronize()
    ops.check_status()
    for r in range(world):
        assert torch.equal(res_out[r].cpu(), want_res), r          # bf16 add of bit-exact sums
        assert _rel(outs[r], want_out) <= TOL
        assert torch.equal(outs[r], outs[0])                      # every rank computes the same


def test_missing_peer_times_out_and_reports(comm_mod, native_lib):
    """A peer that never raises its flag: the wait runs out after the (shortened)
    deadline, the status block says DF_ERR_PEER and the context stays usable."""
    import ctypes

    from dynaflow_b200 import _native, ops

    ops.set_timeout_ms(30)
    try:
        em = comm_mod.EmulatedComm(2, max_rows=64, hidden=128, n_ctas=2)
        # launch rank 0 alone through the real (non-emulated) entry point: rank 1 never runs
        view = em._view(0, em.ptrs)
        st = ops.status_block()
        rc = native_lib.df_allreduce_bf16(ctypes.byref(view), 2, 64, 128, 16, 2, st.data_ptr(),
                                          torch.cuda.current_stream().cuda_stream)
        assert rc == 0, _native.last_error()
        with pytest.raises(ops.DeviceStatusError, match="DF_ERR_PEER"):
            ops.check_status()
        ops.check_status()                                         # cleared; context alive
        x = torch.ones(4, device="cuda")
        assert float((x + 1).sum()) == 8.0
    finally:
        ops.set_timeout_ms(2000)


@pytest.mark.parametrize("T", [300, 2000])
def test_standalone_add_rmsnorm_equals_the_fused_second_half(comm_mod, T):
    """2000 rows: a warp per row, the same arithmetic in the same order as the fused kernel's epilogue, so the same
    bits. 300 rows: fewer warps than SMs, so a whole CTA takes a row (the sum of squares is then added up in another
    order: the same residual bits, the normalised rows within one bf16 step)."""
    from dynaflow_b200 import ops
    from oracle import ops_oracle

    g = torch.Generator().manual_seed(21)
    H = 4096
    y = torch.randn(T, H, generator=g).bfloat16()
    res = torch.randn(T, H, generator=g).bfloat16()
    w = (1 + 0.1 * torch.randn(H, generator=g)).bfloat16()
    want_out, want_res = ops_oracle.allreduce_add_rmsnorm([y], res, w)
    out = torch.empty(T, H, dtype=torch.bfloat16, device="cuda")
    res_dev = res.cuda()
    comm_mod.add_rmsnorm(y.cuda(), res_dev, w.cuda(), out, res_dev)
    torch.cuda.synchronize()
    assert torch.equal(res_dev.cpu(), want_res)
    assert _rel(out, want_out) <= TOL
    # bit-identical to the fused kernel's epilogue on the same sum
    em = comm_mod.EmulatedComm(1, max_rows=2048, hidden=H, n_ctas=4)
    em.partial(0, T).copy_(y)
    out2 = [torch.empty(T, H, dtype=torch.bfloat16, device="cuda")]
    res2 = [res.cuda()]
    em.run(T, weight=w.cuda(), residual_in=res2, residual_out=res2, out=out2)
    torch.cuda.synchronize()
    ops.check_status()
    assert torch.equal(res2[0], res_dev)
    if T >= 2000:
        assert torch.equal(out2[0], out)
    else:
        assert torch.allclose(out2[0].float(), out.float(), rtol=2.0 ** -7, atol=1e-3)
    out0 = torch.empty(T, H, dtype=torch.bfloat16, device="cuda")
    res0 = torch.empty(T, H, dtype=torch.bfloat16, device="cuda")
    comm_mod.add_rmsnorm(y.cuda(), None, w.cuda(), out0, res0)   # no residual: r' = y
    assert torch.equal(res0.cpu(), y)


@pytest.mark.parametrize("world,T,H", [(2, 48, 256), (8, 203, 4096), (4, 33, 1024), (1, 16, 128)])
@pytest.mark.parametrize("with_residual", [True, False])
def test_emulated_sharded_residual_form(comm_mod, world, T, H, with_residual):
    """Residual stream sharded by rows: the owner of a row slice adds the residual and normalises
    between the two shots; every rank receives the normalised rows of all slices, and only the
    owner's residual rows change."""
    from dynaflow_b200 import ops
    from oracle import ops_oracle

    g = torch.Generator().manual_seed(13 * world + T)
    parts = [torch.randn(T, H, generator=g).bfloat16() for _ in range(world)]
    residual = torch.randn(T, H, generator=g).bfloat16()
    weight = (1.0 + 0.1 * torch.randn(H, generator=g)).bfloat16()
    want_out, want_res = ops_oracle.allreduce_add_rmsnorm(parts, residual if with_residual else None, weight)
    em = comm_mod.EmulatedComm(world, max_rows=256, hidden=H, n_ctas=8)
    for r in range(world):
        em.partial(r, T).copy_(parts[r])
    sentinel = 7.0
    res_bufs = [(residual.clone() if with_residual else torch.full((T, H), sentinel).bfloat16()).cuda()
                for _ in range(world)]
    em.run(T, weight=weight.cuda(), residual_in=res_bufs if with_residual else None, residual_out=res_bufs,
           sharded=True)
    torch.cuda.synchronize()
    ops.check_status()
    for r in range(world):
        assert _rel(em.result(r, T), want_out) <= TOL
        assert torch.equal(em.result(r, T), em.result(0, T))
        lo, hi = T * r // world, T * (r + 1) // world
        assert torch.equal(res_bufs[r][lo:hi].cpu(), want_res[lo:hi])            # own slice updated
        before = residual if with_residual else torch.full((T, H), sentinel).bfloat16()
        keep = torch.ones(T, dtype=torch.bool)
        keep[lo:hi] = False
        assert torch.equal(res_bufs[r].cpu()[keep], before[keep])                # other rows untouched


@pytest.mark.parametrize("sharded", [False, True])
def test_fused_reduction_against_reference_executed_fixture(comm_mod, sharded):
    """Four ranks' partial sums, residual and weight of the fixture the reference engine produced
    (transformers' LlamaRMSNorm after the residual add, two ragged nano-batches): the kernel's new
    residual is bit-identical and its normalised output within the bf16 tolerance, per nano-batch."""
    import json
    import os

    import numpy as np

    from conftest import GOLDEN
    from dynaflow_b200 import ops

    z = np.load(os.path.join(GOLDEN, "norm_split.npz"))
    meta = json.load(open(os.path.join(GOLDEN, "norm_split.json")))
    t = {k: torch.from_numpy(z[k]).view(torch.bfloat16) for k in z.files}
    world, H = 4, t["y"].shape[1]
    cuts = meta["split"]["split_indices"]
    em = comm_mod.EmulatedComm(world, max_rows=128, hidden=H, n_ctas=4)
    for i in range(2):
        sl = slice(cuts[i], cuts[i + 1])
        T = cuts[i + 1] - cuts[i]
        res_in = [t["residual"][sl].cuda() for _ in range(world)]
        res_out = [torch.zeros(T, H, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
        outs = [torch.zeros(T, H, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
        for r in range(world):
            em.partial(r, T).copy_(t[f"partial{r}"][sl])
        em.run(T, weight=t["weight"].cuda(), residual_in=res_in, residual_out=res_out, out=outs, eps=meta["eps"],
               sharded=sharded)
        torch.cuda.synchronize()
        ops.check_status()
        want_out, want_res = t["out"][sl], t["new_residual"][sl]
        for r in range(world):
            lo, hi = (T * r // world, T * (r + 1) // world) if sharded else (0, T)
            assert torch.equal(res_out[r][lo:hi].cpu(), want_res[lo:hi]), (i, r)
            got = em.result(r, T) if sharded else outs[r]
            assert _rel(got, want_out) <= TOL, (i, r)
