"""Parity of the sm_100a prefill attention kernel (through the C ABI) against the CPU oracle.

Tolerance (bf16): max|a-b| / max|b| <= 2e-2.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu

TOL = 2e-2
HD = 128


def _qkv(T, hq, hkv, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(T, (hq + 2 * hkv) * HD, generator=g).bfloat16()


def _run(ops, qkv, hq, hkv, batch, seq_len, lens=None, max_ctas=0):
    dev = qkv.cuda()
    q, k, v = dev[:, :hq * HD], dev[:, hq * HD:(hq + hkv) * HD], dev[:, (hq + hkv) * HD:]
    out = torch.zeros(qkv.shape[0], hq * HD, dtype=torch.bfloat16, device="cuda")
    cu = None
    if lens is not None:
        cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device="cuda")
    ops.attention_prefill(q, k, v, out, batch=batch, seq_len=seq_len, cu_seqlens=cu, max_ctas=max_ctas)
    torch.cuda.synchronize()
    ops.check_status()
    return out.cpu()


def _want(qkv, hq, hkv, lens):
    from oracle import ops_oracle

    T = qkv.shape[0]
    q = qkv[:, :hq * HD].reshape(T, hq, HD)
    k = qkv[:, hq * HD:(hq + hkv) * HD].reshape(T, hkv, HD)
    v = qkv[:, (hq + hkv) * HD:].reshape(T, hkv, HD)
    return ops_oracle.causal_attention(q, k, v, lens).reshape(T, hq * HD)


def _rel(got, want):
    return ((got.float() - want.float()).abs().max() / want.float().abs().max()).item()


@pytest.fixture(scope="module")
def ops(native_lib):
    from dynaflow_b200 import ops as _ops

    return _ops


@pytest.mark.parametrize("batch,seq,hq,hkv", [(1, 128, 1, 1), (1, 256, 2, 1), (2, 384, 4, 2), (3, 512, 4, 1), (1, 1024, 2, 2)])
def test_uniform_sequences_match_oracle(ops, batch, seq, hq, hkv):
    qkv = _qkv(batch * seq, hq, hkv, 11)
    got = _run(ops, qkv, hq, hkv, batch, seq)
    assert _rel(got, _want(qkv, hq, hkv, [seq] * batch)) <= TOL


@pytest.mark.parametrize("lens", [[1], [7, 129], [100, 300, 5, 128], [257, 64, 511]])
def test_ragged_sequences_match_oracle(ops, lens):
    hq, hkv = 4, 2
    qkv = _qkv(sum(lens), hq, hkv, 12)
    got = _run(ops, qkv, hq, hkv, len(lens), max(lens), lens=lens)
    assert _rel(got, _want(qkv, hq, hkv, lens)) <= TOL


def test_large_scores_keep_the_running_maximum_exact(ops):
    """Scores that grow along the keys force the accumulator to be rescaled several times."""
    batch, seq, hq, hkv = 1, 640, 1, 1
    qkv = _qkv(seq, hq, hkv, 13)
    ramp = torch.linspace(0.2, 3.0, seq).unsqueeze(1)
    qkv[:, HD:2 * HD] = (qkv[:, HD:2 * HD].float() * ramp).bfloat16()      # later keys have larger norms
    got = _run(ops, qkv, hq, hkv, batch, seq)
    assert _rel(got, _want(qkv, hq, hkv, [seq])) <= TOL


def test_grid_limit_does_not_change_the_result(ops):
    """The launch on a few CTAs (SMs left to the reduction kernel) is bit-identical."""
    batch, seq, hq, hkv = 2, 512, 4, 1
    qkv = _qkv(batch * seq, hq, hkv, 14)
    assert torch.equal(_run(ops, qkv, hq, hkv, batch, seq), _run(ops, qkv, hq, hkv, batch, seq, max_ctas=5))


def test_llama3_8b_shape_sampled_rows(ops):
    """One micro-batch of the Llama-3-8B-shaped prefill on one GPU: 4 sequences of 2048, 32 query and 8
    key/value heads; the oracle is evaluated on two heads of one sequence (it is O(S^2) on the CPU)."""
    batch, seq, hq, hkv = 4, 2048, 32, 8
    qkv = _qkv(batch * seq, hq, hkv, 15)
    got = _run(ops, qkv, hq, hkv, batch, seq)
    b = 2
    rows = slice(b * seq, (b + 1) * seq)
    for h in (5, 30):
        kvh = h // (hq // hkv)
        sub = torch.cat([qkv[rows, h * HD:(h + 1) * HD], qkv[rows, (hq + kvh) * HD:(hq + kvh + 1) * HD],
                         qkv[rows, (hq + hkv + kvh) * HD:(hq + hkv + kvh + 1) * HD]], dim=1)
        want = _want(sub, 1, 1, [seq])
        assert _rel(got[rows, h * HD:(h + 1) * HD], want) <= TOL


def test_rejects_unsupported_head_dim(native_lib):
    x = torch.zeros(128, 64, dtype=torch.bfloat16, device="cuda")
    st = torch.zeros(4, dtype=torch.int32, device="cuda")
    rc = native_lib.df_attention_prefill_bf16(x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), 128, 1, 128, None, 1, 1,
                                              64, 64, 64, 64, 64, 0.125, 0, st.data_ptr(), None)
    assert rc == -3


# ------------------------------------------------------------------ decode (split-KV)
@pytest.fixture(params=[True, False], ids=["keys_on_lanes", "heads_on_rows"])
def decode_form(request, ops):
    """Both forms of the decode kernel: the transposed products (default) and the query heads on the
    accumulator rows."""
    ops.set_launch_option("decode_keys_on_lanes", request.param)
    yield request.param
    ops.set_launch_option("decode_keys_on_lanes", True)


def _decode_case(ops, batch, max_len, hq, hkv, lens, seed, max_ctas=0, poison=False):
    from oracle import ops_oracle

    g = torch.Generator().manual_seed(seed)
    q = torch.randn(batch, hq * HD, generator=g).bfloat16()
    kc = torch.randn(batch, max_len, hkv * HD, generator=g).bfloat16()
    vc = torch.randn(batch, max_len, hkv * HD, generator=g).bfloat16()
    if poison:   # what an allocator hands out: anything, NaN patterns included, past the end of a sequence
        for b, n in enumerate(lens):
            kc[b, n:] = float("nan")
            vc[b, n:] = float("nan")
    out = torch.full((batch, hq * HD), float("nan"), dtype=torch.bfloat16, device="cuda")
    ws = ops.attention_decode_workspace(batch, hq, hkv, max_len)
    sl = torch.tensor(lens, dtype=torch.int32, device="cuda")
    ops.attention_decode(q.cuda(), kc.cuda(), vc.cuda(), sl, out, ws, max_ctas=max_ctas)
    first = out.clone()
    out.fill_(float("nan"))
    ops.attention_decode(q.cuda(), kc.cuda(), vc.cuda(), sl, out, ws, max_ctas=max_ctas)   # bit-reproducible
    torch.cuda.synchronize()
    ops.check_status()
    assert torch.equal(out, first)
    want = ops_oracle.decode_attention(q.view(batch, hq, HD), torch.nan_to_num(kc).view(batch, max_len, hkv, HD),
                                       torch.nan_to_num(vc).view(batch, max_len, hkv, HD), lens).reshape(batch, hq * HD)
    return out.cpu(), want


@pytest.mark.parametrize("batch,max_len,hq,hkv,lens", [
    (1, 128, 4, 1, [128]), (2, 256, 4, 1, [1, 256]), (3, 640, 8, 2, [640, 129, 300]), (5, 1024, 4, 4, [7, 1000, 512, 513, 1]),
    (4, 4096, 4, 1, [4096, 4095, 2049, 100]), (2, 300, 3, 1, [300, 77]), (2, 384, 16, 2, [384, 130])])
def test_decode_attention_matches_oracle(ops, batch, max_len, hq, hkv, lens, decode_form):
    got, want = _decode_case(ops, batch, max_len, hq, hkv, lens, 31)
    assert torch.isfinite(got.float()).all()
    assert _rel(got, want) <= TOL


def test_decode_attention_ignores_what_lies_past_the_end_of_a_sequence(ops):
    """Cache rows past seq_lens[b] are not the kernel's to read into the result: filled with NaN,
    the output stays finite and equal to the oracle's."""
    got, want = _decode_case(ops, 4, 1024, 8, 2, [1, 130, 1000, 513], 34, poison=True)
    assert torch.isfinite(got.float()).all()
    assert _rel(got, want) <= TOL


def test_decode_attention_with_sixteen_heads_per_key_value_head(ops):
    got, want = _decode_case(ops, 3, 512, 32, 2, [512, 65, 300], 35)
    assert _rel(got, want) <= TOL


def test_decode_attention_large_scores_rescale(ops):
    """Scores that grow along the cache force the running reference maximum to move (the O^T rescale path)."""
    from oracle import ops_oracle

    batch, max_len, hq, hkv = 2, 1024, 4, 1
    g = torch.Generator().manual_seed(36)
    q = torch.randn(batch, hq * HD, generator=g).bfloat16()
    ramp = torch.linspace(0.2, 3.0, max_len).view(1, max_len, 1)
    kc = (q.view(batch, 1, hq, HD)[:, :, 0, :] * ramp).bfloat16().contiguous()     # keys aligned with head 0's query, growing
    vc = torch.randn(batch, max_len, hkv * HD, generator=g).bfloat16()
    lens = [1024, 700]
    out = torch.empty(batch, hq * HD, dtype=torch.bfloat16, device="cuda")
    ws = ops.attention_decode_workspace(batch, hq, hkv, max_len)
    sl = torch.tensor(lens, dtype=torch.int32, device="cuda")
    ops.attention_decode(q.cuda(), kc.cuda(), vc.cuda(), sl, out, ws, max_ctas=2)   # long chunks: many blocks per item
    torch.cuda.synchronize()
    ops.check_status()
    want = ops_oracle.decode_attention(q.view(batch, hq, HD), kc.view(batch, max_len, hkv, HD),
                                       vc.view(batch, max_len, hkv, HD), lens).reshape(batch, hq * HD)
    assert torch.isfinite(out.float()).all()
    assert _rel(out.cpu(), want) <= TOL


def test_decode_attention_random_shapes(ops):
    """Twelve seeded random cases: batch, cache length, head grouping, ragged lengths, grid limit."""
    import numpy as np

    rng = np.random.default_rng(43)
    for case in range(12):
        hkv = int(rng.integers(1, 4))
        group = int(rng.choice([1, 2, 3, 4, 5, 8, 12, 16]))
        batch = int(rng.integers(1, 9))
        max_len = int(rng.integers(1, 1200))
        lens = [int(rng.integers(1, max_len + 1)) for _ in range(batch)]
        max_ctas = 0 if case % 3 else int(rng.integers(1, 40))
        got, want = _decode_case(ops, batch, max_len, hkv * group, hkv, lens, 500 + case, max_ctas=max_ctas, poison=case % 2 == 0)
        assert torch.isfinite(got.float()).all(), (case, batch, max_len, hkv, group)
        assert _rel(got, want) <= TOL, (case, batch, max_len, hkv, group, lens)


def test_decode_attention_on_few_ctas_is_within_tolerance(ops):
    """Fewer CTAs cut the cache into fewer, longer chunks: another summation order, same result
    within tolerance."""
    lens = [900, 1024, 333, 64, 1, 512]
    a, want = _decode_case(ops, 6, 1024, 8, 2, lens, 32)
    b, _ = _decode_case(ops, 6, 1024, 8, 2, lens, 32, max_ctas=3)
    assert _rel(a, want) <= TOL and _rel(b, want) <= TOL


def test_rope_append_equals_rope_then_append(ops, native_lib):
    g = torch.Generator().manual_seed(38)
    B, max_len, hq, hkv = 5, 40, 4, 2
    qkv = torch.randn(B, (hq + 2 * hkv) * HD, generator=g).bfloat16().cuda()
    lens = [1, 40, 17, 2, 33]
    sl = torch.tensor(lens, dtype=torch.int32, device="cuda")
    ref = qkv.clone()
    kc_ref = torch.zeros(B, max_len, hkv * HD, dtype=torch.bfloat16, device="cuda")
    vc_ref = torch.zeros_like(kc_ref)
    pos = (sl - 1).contiguous()
    rc = native_lib.df_rope_bf16(ref.data_ptr(), pos.data_ptr(), B, hq + hkv, HD, ref.stride(0), 500000.0, None)
    assert rc == 0
    ops.kv_cache_append(ref[:, hq * HD:(hq + hkv) * HD], ref[:, (hq + hkv) * HD:], kc_ref, vc_ref, sl)
    kc, vc = torch.zeros_like(kc_ref), torch.zeros_like(vc_ref)
    ops.rope_append(qkv, sl, hq, hkv, kc, vc, 500000.0)
    torch.cuda.synchronize()
    assert torch.equal(qkv, ref) and torch.equal(kc, kc_ref) and torch.equal(vc, vc_ref)


def test_kv_cache_append_writes_the_last_valid_position(ops):
    g = torch.Generator().manual_seed(33)
    B, max_len, cols = 5, 40, 2 * HD
    qkv = torch.randn(B, 6 * HD, generator=g).bfloat16().cuda()
    kc = torch.zeros(B, max_len, cols, dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    lens = [1, 40, 17, 2, 33]
    sl = torch.tensor(lens, dtype=torch.int32, device="cuda")
    k_new, v_new = qkv[:, 2 * HD:4 * HD], qkv[:, 4 * HD:]
    ops.kv_cache_append(k_new, v_new, kc, vc, sl)
    torch.cuda.synchronize()
    for b, n in enumerate(lens):
        assert torch.equal(kc[b, n - 1], k_new[b]) and torch.equal(vc[b, n - 1], v_new[b])
        keep = torch.ones(max_len, dtype=torch.bool)
        keep[n - 1] = False
        assert kc[b, keep].abs().sum() == 0 and vc[b, keep].abs().sum() == 0
