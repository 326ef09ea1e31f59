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
