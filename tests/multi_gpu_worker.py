"""Worker of tests/test_gpu_multi.py: launched by torch.distributed.run, one rank per GPU."""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))


def main() -> None:
    from dynaflow_b200 import ops
    from dynaflow_b200.comm import PeerComm
    from dynaflow_b200.layer import TensorParallelGatedMLP
    from oracle import ops_oracle

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    T, H, I = 1000, 1024, 2048
    comm = PeerComm(rank, world, max_rows=1024, hidden=H, slots=2, n_ctas=16, device=dev)

    # ---- plain all-reduce: bit-exact against the fp32 rank-order sum, three calls in a row
    parts = [torch.randn(T, H, generator=torch.Generator().manual_seed(100 + r)).bfloat16() for r in range(world)]
    acc = torch.zeros(T, H)
    for p in parts:
        acc += p.float()
    want = acc.bfloat16()
    for call in range(3):
        comm.partial(0, T).copy_(parts[rank])
        got = comm.all_reduce(0, T)
        torch.cuda.synchronize()
        ops.check_status()
        assert torch.equal(got.cpu(), want), f"rank {rank} call {call}: all-reduce differs"
        dist.barrier()

    # ---- fused residual + RMSNorm
    g = torch.Generator().manual_seed(5)
    residual = torch.randn(T, H, generator=g).bfloat16()
    weight = (1 + 0.1 * torch.randn(H, generator=g)).bfloat16()
    want_out, want_res = ops_oracle.allreduce_add_rmsnorm(parts, residual, weight)
    comm.partial(1, T).copy_(parts[rank])
    res_dev = residual.to(dev)
    out = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
    comm.all_reduce_add_rmsnorm(1, T, res_dev, weight.to(dev), out, res_dev)   # residual updated in place
    torch.cuda.synchronize()
    ops.check_status()
    assert torch.equal(res_dev.cpu(), want_res), f"rank {rank}: residual differs"
    rel = ((out.float().cpu() - want_out.float()).abs().max() / want_out.float().abs().max()).item()
    assert rel <= 2e-2, f"rank {rank}: fused RMSNorm rel err {rel}"
    dist.barrier()

    # ---- tensor-parallel gated MLP, two micro-batches, reduction overlapped with the next GEMMs
    g = torch.Generator().manual_seed(9)
    w_gate = (torch.randn(I, H, generator=g) * 0.05).bfloat16()
    w_up = (torch.randn(I, H, generator=g) * 0.05).bfloat16()
    w_down = (torch.randn(H, I, generator=g) * 0.05).bfloat16()
    x = torch.randn(2 * T, H, generator=g).bfloat16()
    layer = TensorParallelGatedMLP(H, I, rank=rank, world=world, max_rows=1024, micro_batches=2, device=dev,
                                   weights=(w_gate, w_up, w_down), comm=comm)
    results = []
    layer.forward_device(x.to(dev), None, [0, T, 2 * T], results=results)
    torch.cuda.synchronize()
    ops.check_status()
    got = torch.cat([r.cpu() for r in results])
    want = ops_oracle.gated_mlp(x, w_gate, w_up, w_down)
    rel = ((got.float() - want.float()).abs().max() / want.float().abs().max()).item()
    assert rel <= 2e-2, f"rank {rank}: TP layer rel err {rel}"
    out_host = torch.empty(2 * T, H, dtype=torch.bfloat16).pin_memory()
    layer.forward_host(x.pin_memory(), out_host, [0, T, 2 * T])
    torch.cuda.synchronize()
    ops.check_status()
    assert torch.equal(out_host, got), f"rank {rank}: host-staged step differs from the device-resident one"
    dist.barrier()

    # ---- two TP blocks back to back with the fused reduction + residual + RMSNorm between them
    norm_w = (1 + 0.1 * torch.randn(H, generator=g)).bfloat16()
    res0 = torch.randn(2 * T, H, generator=g).bfloat16()
    res_dev = res0.to(dev)
    outs = layer.forward_chain(x.to(dev), [0, T, 2 * T], 2, norm_w.to(dev), res_dev)
    torch.cuda.synchronize()
    ops.check_status()
    xo, ro = x, res0
    for _ in range(2):                          # oracle: shard, reduce in rank order, add, normalise
        parts = []
        for r in range(world):
            lo, hi = r * (I // world), (r + 1) * (I // world)
            parts.append(ops_oracle.gated_mlp(xo, w_gate[lo:hi], w_up[lo:hi], w_down[:, lo:hi]))
        xo, ro = ops_oracle.allreduce_add_rmsnorm(parts, ro, norm_w)
    got = torch.cat([o.cpu() for o in outs])
    rel = ((got.float() - xo.float()).abs().max() / xo.float().abs().max()).item()
    assert rel <= 2e-2, f"rank {rank}: chained TP blocks rel err {rel}"
    rel = ((res_dev.cpu().float() - ro.float()).abs().max() / ro.float().abs().max()).item()
    assert rel <= 2e-2, f"rank {rank}: chained residual rel err {rel}"
    dist.barrier()

    # ---- the same chain with the residual stream sharded by rows (add + norm between the two shots)
    res_dev = res0.to(dev)
    outs = layer.forward_chain(x.to(dev), [0, T, 2 * T], 2, norm_w.to(dev), res_dev, sharded_residual=True)
    torch.cuda.synchronize()
    ops.check_status()
    got = torch.cat([o.cpu() for o in outs])
    rel = ((got.float() - xo.float()).abs().max() / xo.float().abs().max()).item()
    assert rel <= 2e-2, f"rank {rank}: sharded-residual chain rel err {rel}"
    for mb in range(2):                                   # this rank's residual rows of each micro-batch
        lo, hi = comm.slice_bounds(T)
        mine = res_dev[mb * T + lo: mb * T + hi].cpu().float()
        ref = ro[mb * T + lo: mb * T + hi].float()
        assert ((mine - ref).abs().max() / ro.float().abs().max()).item() <= 2e-2, f"rank {rank}: residual slice"
    dist.barrier()

    # ---- the same layer step through DynaFlowManager.get_callable(): all-gather, MLP, reduce-scatter as subgraphs
    from dynaflow_b200.host_step import ManagedLayerStep

    comm_in = PeerComm(rank, world, max_rows=1024, hidden=H, slots=2, n_ctas=16, device=dev)
    lo, hi = comm.slice_bounds(T)
    x_local = torch.cat([x[lo:hi], x[T + lo:T + hi]]).to(dev)                 # this rank's rows of both nano-batches
    want_local = torch.cat([want[lo:hi], want[T + lo:T + hi]])
    for graph in (False, True):
        step = ManagedLayerStep(layer, comm_in=comm_in, whole_forward_graph=graph)
        for _ in range(2):
            got = step(x_local, [0, hi - lo, 2 * (hi - lo)]).clone()
            torch.cuda.synchronize()
            ops.check_status()
            rel = ((got.float().cpu() - want_local.float()).abs().max() / want.float().abs().max()).item()
            assert rel <= 2e-2, f"rank {rank}: managed TP step rel err {rel} (graph={graph})"
        dist.barrier()
    comm_in.close()
    dist.barrier()

    # ---- expert-parallel top-2 MoE layer: dispatch (all-gather) / expert / combine (reduce-scatter)
    from dynaflow_b200.moe import ExpertParallelMoE

    E, Hm, Im, per_rank = 8, 256, 512, 96
    g = torch.Generator().manual_seed(31)
    xg = torch.randn(per_rank * world, Hm, generator=g).bfloat16()
    lg = torch.randn(per_rank * world, E, generator=g).bfloat16()
    mg = (torch.randn(E, Im, Hm, generator=g) * 0.05).bfloat16()
    mu = (torch.randn(E, Im, Hm, generator=g) * 0.05).bfloat16()
    md = (torch.randn(E, Hm, Im, generator=g) * 0.05).bfloat16()
    if E % world == 0:
        moe = ExpertParallelMoE(Hm, Im, E, per_rank, rank=rank, world=world, weights=(mg, mu, md), slots=1, n_ctas=8,
                                device=dev)
        lo = rank * per_rank
        for _ in range(2):
            mine = moe.forward(xg[lo:lo + per_rank].to(dev), lg[lo:lo + per_rank].to(dev)).clone()
        torch.cuda.synchronize()
        ops.check_status()
        want_all = ops_oracle.moe_layer(xg, lg, mg, mu, md)
        rel = ((mine.float().cpu() - want_all[lo:lo + per_rank].float()).abs().max() / want_all.float().abs().max()).item()
        assert rel <= 2e-2, f"rank {rank}: expert-parallel MoE rel err {rel}"
        dist.barrier()
        moe.close()
        # the same layer with the all-to-all exchange: only the routed rows cross the links
        moe = ExpertParallelMoE(Hm, Im, E, per_rank, rank=rank, world=world, weights=(mg, mu, md), slots=1, n_ctas=8,
                                device=dev, exchange="a2a")
        for _ in range(2):
            mine = moe.forward(xg[lo:lo + per_rank].to(dev), lg[lo:lo + per_rank].to(dev)).clone()
        torch.cuda.synchronize()
        ops.check_status()
        rel = ((mine.float().cpu() - want_all[lo:lo + per_rank].float()).abs().max() / want_all.float().abs().max()).item()
        assert rel <= 2e-2, f"rank {rank}: all-to-all MoE rel err {rel}"
        dist.barrier()
        moe.close()
    dist.barrier()

    # ---- tensor-parallel decoder stack (attention + MLP halves, reductions overlapped) vs PyTorch
    from dynaflow_b200.decoder import DecoderShape, TensorParallelDecoder, reference_weights
    from test_gpu_decoder import load_oracle_model, oracle_hidden

    dshape = DecoderShape(hidden=256, intermediate=512, heads=8, kv_heads=8, head_dim=128, layers=2, vocab=256)
    dweights = reference_weights(dshape, seed=8)
    dids = torch.randint(0, dshape.vocab, (4, 64), generator=torch.Generator().manual_seed(9))
    dec = TensorParallelDecoder(dshape, rank=rank, world=world, max_rows=2 * 64, micro_batches=2, weights=dweights,
                                device=dev, n_ctas=8)
    hidden = dec.forward(dids.to(dev))
    torch.cuda.synchronize()
    ops.check_status()
    model = load_oracle_model(dshape, dweights).to(dev)
    want_h = oracle_hidden(model, dids.to(dev)).reshape(-1, dshape.hidden)
    rel = ((hidden.float() - want_h.float()).abs().max() / want_h.float().abs().max()).item()
    assert rel <= 2e-2, f"rank {rank}: TP decoder rel err {rel}"
    dist.barrier()
    dec.close()
    dist.barrier()
    comm.close()
    dist.destroy_process_group()
    if rank == 0:
        print("MULTI_GPU_OK")


if __name__ == "__main__":
    main()
