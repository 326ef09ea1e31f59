"""Parity of the sm_100a gated-MLP kernels (through the C ABI) against the CPU oracle.

Tolerance (bf16, as the task states it): max|a-b| / max|b| <= 2e-2.
"""
import json
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN

pytestmark = pytest.mark.gpu

TOL = 2e-2


def rel_err(got: torch.Tensor, want: torch.Tensor) -> float:
    return ((got.float().cpu() - want.float().cpu()).abs().max() / want.float().abs().max()).item()


@pytest.fixture(scope="module")
def ops(native_lib):
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    from dynaflow_b200 import ops as _ops

    return _ops


def _rand(shape, scale, seed):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).bfloat16()


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (1, 8, 8), (16, 256, 4096), (257, 520, 200), (100, 4096, 1024),
                                    (384, 264, 14336 // 8)])
def test_gemm_matches_oracle(ops, M, N, K):
    a, b = _rand((M, K), 1.0, 1), _rand((N, K), 0.05, 2)
    got = ops.gemm_bf16(a.cuda(), b.cuda())
    ops.check_status()
    want = torch.nn.functional.linear(a.float(), b.float())
    assert rel_err(got, want) <= TOL


def test_gemm_strided_operands_and_output(ops):
    a_full, b_full = _rand((96, 512), 1.0, 3).cuda(), _rand((264, 512), 0.05, 4).cuda()
    out_full = torch.zeros(96, 512, dtype=torch.bfloat16, device="cuda")
    a, b, out = a_full[:, 128:384], b_full[:, 64:320], out_full[:, 8:272]
    ops.gemm_bf16(a, b, out=out)
    ops.check_status()
    want = a.float() @ b.float().T
    assert rel_err(out, want) <= TOL
    assert out_full[:, :8].abs().sum() == 0 and out_full[:, 272:].abs().sum() == 0  # nothing outside the view


@pytest.mark.parametrize("M,H,I", [(128, 64, 128), (1, 64, 128), (16, 256, 256), (300, 512, 1032), (1000, 1024, 2816)])
def test_gated_mlp_matches_oracle(ops, M, H, I):
    from oracle import ops_oracle

    x = _rand((M, H), 1.0, 5)
    wg, wu, wd = _rand((I, H), 0.05, 6), _rand((I, H), 0.05, 7), _rand((H, I), 0.05, 8)
    h = ops.gateup_silu(x.cuda(), wg.cuda(), wu.cuda())
    out = ops.gated_mlp(x.cuda(), wg.cuda(), wu.cuda(), wd.cuda())
    ops.check_status()
    g = torch.nn.functional.linear(x, wg)
    u = torch.nn.functional.linear(x, wu)
    assert rel_err(h, ops_oracle.silu_mul(g, u)) <= TOL
    assert rel_err(out, ops_oracle.gated_mlp(x, wg, wu, wd)) <= TOL
    assert rel_err(out, ops_oracle.gated_mlp_hf(x, wg, wu, wd)) <= TOL


def test_gated_mlp_against_reference_golden(ops):
    z = np.load(os.path.join(GOLDEN, "mlp_split.npz"))
    t = {k: torch.from_numpy(z[k]).view(torch.bfloat16) for k in z.files}
    cuts = json.load(open(os.path.join(GOLDEN, "mlp_split.json")))["split"]["split_indices"]
    dev = {k: v.cuda() for k, v in t.items()}
    # the reference executed this MLP as two nano-batches cut at `cuts` and concatenated the results
    parts = [ops.gated_mlp(dev["x"][cuts[i]:cuts[i + 1]], dev["w_gate"], dev["w_up"], dev["w_down"]) for i in range(2)]
    ops.check_status()
    assert rel_err(torch.cat(parts), t["out"]) <= TOL


def test_empty_nano_batch(ops):
    x = torch.empty(0, 64, dtype=torch.bfloat16, device="cuda")
    w = _rand((128, 64), 0.05, 1).cuda()
    wd = _rand((64, 128), 0.05, 2).cuda()
    assert ops.gated_mlp(x, w, w, wd).shape == (0, 64)
    assert ops.gemm_bf16(x, w).shape == (0, 128)


def test_micro_batch_split_is_bit_exact_at_full_size(ops):
    """Size-independent property at the benchmark shape: every output row depends on
    its own input row only and tiles accumulate in a fixed order, so running the two
    micro-batches separately gives bit-identical rows to one full-batch run."""
    M, H, I = 4096, 4096, 14336
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(M, H, device="cuda", generator=g).bfloat16()
    wg = (torch.randn(I, H, device="cuda", generator=g) * 0.02).bfloat16()
    wu = (torch.randn(I, H, device="cuda", generator=g) * 0.02).bfloat16()
    wd = (torch.randn(H, I, device="cuda", generator=g) * 0.02).bfloat16()
    full = ops.gated_mlp(x, wg, wu, wd)
    for cut in (M // 2, 1000):
        parts = torch.cat([ops.gated_mlp(x[:cut].contiguous(), wg, wu, wd), ops.gated_mlp(x[cut:].contiguous(), wg, wu, wd)])
        if cut == M // 2:
            assert torch.equal(parts, full)      # both sides run whole tiles: identical accumulation order
        else:
            # a 1000-row nano-batch has fewer tiles than SMs in the down projection and takes the
            # stream-K path (partial sums combined in fp32): equal within rounding, and identical
            # again once that path is switched off
            assert rel_err(parts, full.cpu()) <= 1e-2
            ops.set_launch_option("stream_k", False)
            try:
                parts = torch.cat([ops.gated_mlp(x[:cut].contiguous(), wg, wu, wd),
                                   ops.gated_mlp(x[cut:].contiguous(), wg, wu, wd)])
            finally:
                ops.set_launch_option("stream_k", True)
            assert torch.equal(parts, full)
    ops.check_status()
    # scaling the input by 2 scales the gate pre-activation: check linearity of the down projection instead
    h = ops.gateup_silu(x[:256].contiguous(), wg, wu)
    y1 = ops.gemm_bf16(h, wd)
    y2 = ops.gemm_bf16((h.float() * 2).bfloat16(), wd)
    assert torch.equal((y1.float() * 2).bfloat16(), y2)  # power-of-two scaling is exact in bf16/fp32
    # sampled rows against the CPU oracle at this size
    from oracle import ops_oracle

    rows = torch.tensor([0, 1, 127, 128, 2047, 2048, 4095])
    want = ops_oracle.gated_mlp(x[rows].cpu(), wg.cpu(), wu.cpu(), wd.cpu())
    assert rel_err(full[rows], want) <= TOL


def test_limited_grid_gives_identical_results(ops):
    x, w, wd = _rand((512, 256), 1.0, 1).cuda(), _rand((1024, 256), 0.05, 2).cuda(), _rand((256, 1024), 0.05, 3).cuda()
    ops.set_launch_option("stream_k", False)   # whole tiles on both sides: the grid size must not change a bit
    try:
        a = ops.gated_mlp(x, w, w, wd)
        b = ops.gated_mlp(x, w, w, wd, max_ctas=7)
    finally:
        ops.set_launch_option("stream_k", True)
    ops.check_status()
    assert torch.equal(a, b)
    c = ops.gated_mlp(x, w, w, wd, max_ctas=40)   # stream-K may engage: same values within rounding
    ops.check_status()
    assert rel_err(c, a.cpu()) <= 1e-2


def test_argument_errors(ops):
    x = torch.zeros(8, 64, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError):
        ops.gemm_bf16(x, torch.zeros(8, 32, dtype=torch.bfloat16, device="cuda"))
    with pytest.raises(ValueError):
        ops.gemm_bf16(x.float(), x)
    with pytest.raises(RuntimeError, match="multiples of 8"):
        ops.gemm_bf16(x, torch.zeros(12, 64, dtype=torch.bfloat16, device="cuda"))


@pytest.mark.parametrize("M,H,I", [(16, 4096, 14336), (128, 4096, 1792), (256, 4096, 14336), (40, 1024, 2816)])
def test_small_m_stream_k_path(ops, M, H, I):
    """Decode-sized nano-batches: fewer output tiles than SMs, so the k-blocks are spread over
    all SMs and partial sums are combined in k order. Checked against the oracle, and for
    run-to-run bit reproducibility (the combination order is fixed)."""
    from oracle import ops_oracle

    x = _rand((M, H), 1.0, 11)
    wg, wu, wd = _rand((I, H), 0.02, 12), _rand((I, H), 0.02, 13), _rand((H, I), 0.02, 14)
    dev = [t.cuda() for t in (x, wg, wu, wd)]
    out1 = ops.gated_mlp(*dev)
    h1 = ops.gateup_silu(dev[0], dev[1], dev[2])
    out2 = ops.gated_mlp(*dev)
    ops.check_status()
    assert torch.equal(out1, out2)
    g = torch.nn.functional.linear(x, wg)
    u = torch.nn.functional.linear(x, wu)
    assert rel_err(h1, ops_oracle.silu_mul(g, u)) <= TOL
    assert rel_err(out1, ops_oracle.gated_mlp(x, wg, wu, wd)) <= TOL
    # the plain entry point without a workspace (whole tiles only) agrees within tolerance
    ops.set_launch_option("stream_k", False)
    try:
        out3 = ops.gated_mlp(*dev)
    finally:
        ops.set_launch_option("stream_k", True)
    ops.check_status()
    assert rel_err(out3, out1) <= 1e-2


@pytest.mark.parametrize("M,H,I", [(256, 4096, 14336), (1000, 1024, 2816), (4096, 4096, 14336), (8192, 4096, 1792)])
def test_one_launch_mlp_equals_two_launches(ops, M, H, I):
    """df_mlp_gated_bf16 runs gate/up and down as ONE persistent launch (down tiles wait on
    per-panel counters for their rows of the intermediate). Same tiles, same accumulation
    order: the result must be bit-identical to the two separate launches, every time."""
    g = torch.Generator(device="cuda").manual_seed(M + I)
    x = torch.randn(M, H, device="cuda", generator=g).bfloat16()
    wg = (torch.randn(I, H, device="cuda", generator=g) * 0.02).bfloat16()
    wu = (torch.randn(I, H, device="cuda", generator=g) * 0.02).bfloat16()
    wd = (torch.randn(H, I, device="cuda", generator=g) * 0.02).bfloat16()
    ops.set_launch_option("mlp_one_launch", False)
    ops.set_launch_option("stream_k", False)      # whole tiles, as the single launch computes them
    try:
        two = ops.gated_mlp(x, wg, wu, wd)
    finally:
        ops.set_launch_option("mlp_one_launch", True)
        ops.set_launch_option("stream_k", True)
    for _ in range(5):
        one = ops.gated_mlp(x, wg, wu, wd)
        if ((M + 127) // 128) * ((H + 127) // 128) >= 128:   # fewer down tiles take the stream-K path
            assert torch.equal(one, two)
        else:
            assert rel_err(one, two) <= 1e-2
    ops.check_status()
    small = ops.gated_mlp(x, wg, wu, wd, max_ctas=5)     # few CTAs: long waits on the panel counters
    ops.check_status()
    assert torch.equal(small, two)


@pytest.fixture(params=[True, False], ids=["split_k_small", "operand_swap"])
def small_rows_form(request, ops):
    """Both forms a launch of at most 128 rows can take: the split-K kernel (default) and, with it
    switched off, the operand-swapped form of the general kernel."""
    ops.set_launch_option("split_k_small", request.param)
    yield request.param
    ops.set_launch_option("split_k_small", True)


@pytest.mark.parametrize("M", [1, 7, 16, 17, 48, 64, 65, 100, 127, 128])
@pytest.mark.parametrize("H,I", [(4096, 14336), (1024, 2816)])
def test_decode_rows_operand_swapped_form(ops, M, H, I, small_rows_form):
    """Launches of at most 128 rows take the split-K kernel or the operand-swapped form of the GEMM
    kernel (weight rows on the accumulator lanes, token rows on its columns, stream-K partial sums
    finished cooperatively). Against the oracle, against the regular form, bit-reproducible, and
    nothing written past row M."""
    from oracle import ops_oracle

    x = _rand((M, H), 1.0, 21)
    wg, wu, wd = _rand((I, H), 0.02, 22), _rand((I, H), 0.02, 23), _rand((H, I), 0.02, 24)
    dev = [t.cuda() for t in (x, wg, wu, wd)]
    canvas = torch.full((M + 2, H), 7.0, dtype=torch.bfloat16, device="cuda")   # guard rows after the output
    out = canvas[:M]
    ops.gated_mlp(*dev, out=out)
    first = out.clone()
    ops.gated_mlp(*dev, out=out)
    ops.check_status()
    assert torch.equal(out, first)
    assert torch.all(canvas[M:] == 7.0)
    assert rel_err(out, ops_oracle.gated_mlp(x, wg, wu, wd)) <= TOL
    h = ops.gateup_silu(dev[0], dev[1], dev[2])          # the entry point without a workspace: whole tiles
    g = torch.nn.functional.linear(x, wg)
    u = torch.nn.functional.linear(x, wu)
    assert rel_err(h, ops_oracle.silu_mul(g, u)) <= TOL
    ops.set_launch_option("operand_swap", False)
    try:
        regular = ops.gated_mlp(*dev)
    finally:
        ops.set_launch_option("operand_swap", True)
    ops.check_status()
    assert rel_err(out, regular) <= 1e-2


@pytest.mark.parametrize("M", [1, 8, 50, 128])
@pytest.mark.parametrize("N,K", [(768, 4096), (4096, 512), (4096, 1792), (200, 72), (16032, 4096)])
def test_split_k_small_gemm(ops, M, N, K):
    """The projections of a decode step (at most 128 rows): (tile, k range) CTAs that exchange fp32
    partial tiles with bulk copies and sum them in k order. Against an fp32 product, bit-reproducible,
    nothing written outside the output view, and in agreement with the one-CTA-per-tile form and
    with the general kernel."""
    a, b = _rand((M, K), 1.0, 31).cuda(), _rand((N, K), 0.03, 32).cuda()
    canvas = torch.full((M + 2, N + 16), 7.0, dtype=torch.bfloat16, device="cuda")
    out = canvas[:M, 8:8 + N]
    ops.gemm_bf16(a, b, out=out)
    first = out.clone()
    for _ in range(3):
        ops.gemm_bf16(a, b, out=out)
        assert torch.equal(out, first)
    ops.check_status()
    assert torch.all(canvas[M:] == 7.0) and torch.all(canvas[:, :8] == 7.0) and torch.all(canvas[:, 8 + N:] == 7.0)
    want = a.float() @ b.float().T
    assert rel_err(out, want) <= TOL
    for option in ("stream_k", "split_k_small"):
        ops.set_launch_option(option, False)
        try:
            other = ops.gemm_bf16(a, b)
        finally:
            ops.set_launch_option(option, True)
        ops.check_status()
        assert rel_err(other, out) <= 1e-2


def test_split_k_small_random_shapes(ops):
    """Forty seeded random shapes (1..128 rows, N and K any multiples of 8, strided operands and output, both the
    plain and the gate/up form, a limited grid every fourth case) against fp32 products."""
    rng = np.random.default_rng(41)
    for case in range(40):
        M = int(rng.integers(1, 129))
        N = int(rng.integers(1, 600)) * 8
        K = int(rng.integers(1, 400)) * 8
        pad_a, pad_b, pad_c = (int(rng.integers(0, 3)) * 8 for _ in range(3))
        a_full = _rand((M, K + pad_a), 1.0, 1000 + case).cuda()
        b_full = _rand((N, K + pad_b), 0.05, 2000 + case).cuda()
        a, b = a_full[:, pad_a:], b_full[:, :K]
        canvas = torch.full((M + 1, N + pad_c + 8), 3.0, dtype=torch.bfloat16, device="cuda")
        out = canvas[:M, pad_c:pad_c + N]
        max_ctas = 0 if case % 4 else int(rng.integers(1, 60))
        ops.gemm_bf16(a, b, out=out, max_ctas=max_ctas)
        ops.check_status()
        want = a.float() @ b.float().T
        assert rel_err(out, want) <= TOL, (case, M, N, K, max_ctas)
        assert torch.all(canvas[M:] == 3.0) and torch.all(canvas[:, :pad_c] == 3.0) and torch.all(canvas[:, pad_c + N:] == 3.0), (case, M, N, K)
        if case % 2 == 0:
            b2 = _rand((N, K), 0.05, 3000 + case).cuda()
            h = ops.gateup_silu(a.contiguous(), b.contiguous(), b2, max_ctas=max_ctas)
            ops.check_status()
            g = (a.float() @ b.float().T).bfloat16().float()
            u = (a.float() @ b2.float().T).bfloat16().float()
            assert rel_err(h, torch.nn.functional.silu(g) * u) <= TOL, (case, M, N, K)


@pytest.mark.parametrize("M", [2048, 8192, 16384])
def test_benchmark_shapes_against_oracle_on_sampled_rows(ops, M):
    """The shapes every benchmark number is quoted on (hidden 4096, intermediate 14336; M rows in
    two micro-batches of M/2, each ONE persistent launch): 24 sampled rows of every micro-batch,
    among them the first and last row of the first and last 128-row panel, against the CPU oracle."""
    from oracle import ops_oracle

    H, I = 4096, 14336
    g = torch.Generator(device="cuda").manual_seed(M)
    x = torch.randn(M, H, device="cuda", generator=g).bfloat16()
    wg = (torch.randn(I, H, device="cuda", generator=g) * 0.02).bfloat16()
    wu = (torch.randn(I, H, device="cuda", generator=g) * 0.02).bfloat16()
    wd = (torch.randn(H, I, device="cuda", generator=g) * 0.02).bfloat16()
    half = M // 2
    out = torch.empty(M, H, dtype=torch.bfloat16, device="cuda")
    ws = torch.empty(ops.mlp_workspace_bytes(half, H, I), dtype=torch.uint8, device="cuda")
    for mb in range(2):
        ops.gated_mlp(x[mb * half:(mb + 1) * half], wg, wu, wd, out=out[mb * half:(mb + 1) * half], workspace=ws)
    torch.cuda.synchronize()
    ops.check_status()
    pick = torch.randint(0, half, (16,), generator=torch.Generator().manual_seed(M + 1))
    edge = torch.tensor([0, 127, 128, half // 2, half - 128, half - 1, 1, half - 2])
    rows = torch.cat([torch.cat([pick, edge]) + mb * half for mb in range(2)])
    want = ops_oracle.gated_mlp(x[rows].cpu(), wg.cpu(), wu.cpu(), wd.cpu())
    assert rel_err(out[rows], want) <= TOL
    # elementwise as well: no row may be off by more than the tolerance times its own magnitude scale
    per_row = (out[rows].float().cpu() - want.float()).abs().amax(1) / want.float().abs().amax(1)
    assert per_row.max().item() <= 2 * TOL
