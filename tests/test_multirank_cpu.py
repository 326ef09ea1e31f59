"""Host-side logic of the multi-rank path on CPU: two gloo ranks."""
import os
import subprocess
import sys
import textwrap

from conftest import ROOT

WORKER = textwrap.dedent("""
    import os, sys
    import torch, torch.distributed as dist
    sys.path.insert(0, {root!r})
    from dynaflow_b200.interface import InputInfo, SplitConfig
    from dynaflow_b200.layer import shard_bounds
    from dynaflow_b200.policies import agree_on_split
    from oracle import ops_oracle, split_oracle

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo")

    # 1. tensor-parallel sharding of the gated MLP: the sum of the ranks' partial outputs is the
    #    unsharded layer (fp32: exact up to summation order)
    g = torch.Generator().manual_seed(0)
    H, I, M = 32, 64, 10
    x = torch.randn(M, H, generator=g)
    wg, wu, wd = torch.randn(I, H, generator=g) * 0.2, torch.randn(I, H, generator=g) * 0.2, torch.randn(H, I, generator=g) * 0.2
    lo, hi = shard_bounds(I, rank, world)
    assert (hi - lo) * world == I and lo == rank * (I // world)
    partial = ops_oracle.gated_mlp(x, wg[lo:hi], wu[lo:hi], wd[:, lo:hi])
    total = partial.clone()
    dist.all_reduce(total)
    want = ops_oracle.gated_mlp(x, wg, wu, wd)
    assert torch.allclose(total, want, rtol=1e-5, atol=1e-6), (total - want).abs().max()

    # 2. the reduction the peer-memory kernel implements: rank-order fp32 sum, then residual + RMSNorm
    parts = [None] * world
    dist.all_gather_object(parts, partial.bfloat16())
    res = torch.randn(M, H, generator=g).bfloat16()
    w = torch.ones(H).bfloat16()
    out, new_res = ops_oracle.allreduce_add_rmsnorm(parts, res, w)
    gathered = [None] * world
    dist.all_gather_object(gathered, out)
    assert all(torch.equal(gathered[0], o) for o in gathered)      # every rank holds the same rows

    # 3. agreement on the split: rank 1 cannot split (one request), so nobody does
    def cfg_for(tokens):
        d = split_oracle.nanoflow_split(tokens, 4, [64], False)
        return SplitConfig(**d)
    mine = cfg_for([8, 8]) if rank == 0 else cfg_for([16])
    agreed, rows = agree_on_split(mine, len([8, 8] if rank == 0 else [16]))
    assert agreed.num_nano_batches == 1 and rows == [[16, 16]], (agreed, rows)
    # both can split: configs stay, per-nano-batch rows of every rank are known everywhere
    mine = cfg_for([8, 8]) if rank == 0 else cfg_for([6, 10])
    agreed, rows = agree_on_split(mine, 2)
    assert agreed.num_nano_batches == 2 and rows == [[8, 6], [8, 10]], rows
    dist.barrier()
    dist.destroy_process_group()
    if rank == 0:
        print("CPU_MULTIRANK_OK")
""")


def test_two_gloo_ranks(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER.format(root=ROOT))
    env = dict(os.environ, OMP_NUM_THREADS="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29733", str(script)]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env)
    assert proc.returncode == 0, (proc.stdout[-2000:], proc.stderr[-3000:])
    assert "CPU_MULTIRANK_OK" in proc.stdout


EXIT_WORKER = textwrap.dedent("""
    import os, sys, time
    import torch, torch.distributed as dist
    sys.path.insert(0, {root!r})
    import bench

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    mode = sys.argv[1]
    dist.init_process_group("gloo")
    sync = bench.RankSync(world, torch.device("cpu"))
    log = []
    closers = [lambda: log.append(("closed", time.time()))]
    error, learned = None, False
    try:
        assert sync.max_ms(1.0 + rank) == float(world)            # ordinary use: the maximum over ranks
        assert sync.all_equal(7.0) and not sync.all_equal(float(rank))
        if mode == "fail" and rank == 1:
            raise RuntimeError("rank 1 breaks here")                # the others are on their way to the next meeting point
        time.sleep(0.2 * rank)
        sync.barrier()
        sync.barrier()
        if mode == "soft":
            # the LAST block of a run fails on rank 2 after one of its synchronisation points: every rank gets
            # {{"error": ...}} in place of the block's figures, and the run then leaves clean
            def block():
                sync.barrier()
                if rank == 2:
                    raise ValueError("rank 2 breaks in the last block")
                time.sleep(0.1 * rank)
                sync.barrier()
                sync.max_ms(1.0)
                return {{"figure": 1}}
            got = bench.last_block(sync, block)
            assert "error" in got and "figure" not in got, got
            assert ("rank 2 breaks" in got["error"]) == (rank == 2), got
    except bench.PeerFailed as exc:
        error, learned = str(exc), True
    except Exception as exc:
        error = str(exc)
    error = bench.leave_together(sync, closers, error, learned)
    assert len(log) == 1                                             # every rank unmapped exactly once
    # nobody unmapped before everybody had stopped: the closers ran after the second meeting point on all ranks
    stamps = [None] * world
    dist.all_gather_object(stamps, (log[0][1], error))
    dist.destroy_process_group()
    if mode == "fail":
        assert all(e is not None for _t, e in stamps), stamps        # the failure reached every rank
        assert (error == "rank 1 breaks here") == (rank == 1)
        print(f"RANK{{rank}}_LEFT_WITH_ERROR")
        sys.exit(1)
    assert all(e is None for _t, e in stamps), stamps
    print(f"RANK{{rank}}_LEFT_CLEAN")
""")


def _run_exit_worker(tmp_path, mode, port):
    script = tmp_path / f"exit_{mode}.py"
    script.write_text(EXIT_WORKER.format(root=ROOT))
    env = dict(os.environ, OMP_NUM_THREADS="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=3", "--master-addr",
           "127.0.0.1", "--master-port", str(port), str(script), mode]
    return subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env)


def test_ranks_leave_together_clean_and_after_a_failure(tmp_path):
    """bench.py's exit protocol on three gloo ranks: every host-side collective has one shape, so a rank
    that fails still pairs with the synchronisation its peers reach next; they learn of it there, and all
    ranks run their closers between the same two meeting points and exit non-zero. A failure inside the
    run's last block (``last_block``) instead costs only that block: all ranks agree on it and leave clean."""
    ok = _run_exit_worker(tmp_path, "clean", 29741)
    assert ok.returncode == 0, (ok.stdout[-2000:], ok.stderr[-3000:])
    assert all(f"RANK{r}_LEFT_CLEAN" in ok.stdout for r in range(3))
    soft = _run_exit_worker(tmp_path, "soft", 29743)
    assert soft.returncode == 0, (soft.stdout[-2000:], soft.stderr[-3000:])
    assert all(f"RANK{r}_LEFT_CLEAN" in soft.stdout for r in range(3))
    bad = _run_exit_worker(tmp_path, "fail", 29742)
    assert bad.returncode != 0
    assert all(f"RANK{r}_LEFT_WITH_ERROR" in bad.stdout for r in range(3)), (bad.stdout[-2000:], bad.stderr[-3000:])
