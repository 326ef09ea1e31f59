"""The Llama-style decoder stack on the native kernels (single rank) against the plain PyTorch
decoder of the oracle with the same weights."""
import pytest
import torch

pytestmark = pytest.mark.gpu

TOL = 2e-2


def load_oracle_model(shape, weights):
    from oracle import llama_oracle

    ls = llama_oracle.LlamaShape(hidden=shape.hidden, intermediate=shape.intermediate, heads=shape.heads,
                                 kv_heads=shape.kv_heads, head_dim=shape.head_dim, layers=shape.layers, vocab=shape.vocab,
                                 eps=shape.eps, rope_theta=shape.rope_theta)
    model = llama_oracle.LlamaDecoder(ls).to(torch.bfloat16).eval()
    with torch.no_grad():
        model.embed.weight.copy_(weights["embed"])
        model.lm_head.weight.copy_(weights["lm_head"])
        model.norm.weight.copy_(weights["final_norm"])
        for i, blk in enumerate(model.blocks):
            blk.attn.q_proj.weight.copy_(weights[f"l{i}.q"])
            blk.attn.k_proj.weight.copy_(weights[f"l{i}.k"])
            blk.attn.v_proj.weight.copy_(weights[f"l{i}.v"])
            blk.attn.o_proj.weight.copy_(weights[f"l{i}.o"])
            blk.mlp.gate_proj.weight.copy_(weights[f"l{i}.gate"])
            blk.mlp.up_proj.weight.copy_(weights[f"l{i}.up"])
            blk.mlp.down_proj.weight.copy_(weights[f"l{i}.down"])
            blk.input_norm.weight.copy_(weights[f"l{i}.norm1"])
            blk.post_norm.weight.copy_(weights[f"l{i}.norm2"])
    return model


def oracle_hidden(model, ids):
    from oracle import llama_oracle

    with torch.inference_mode():
        cos, sin = llama_oracle.rope_tables(ids.shape[1], model.s.head_dim, model.s.rope_theta, device=ids.device)
        x = model.embed(ids)
        for blk in model.blocks:
            x = blk(x, cos, sin)
        return model.norm(x)


def test_decoder_stack_matches_pytorch_decoder(native_lib):
    from dynaflow_b200 import ops
    from dynaflow_b200.decoder import DecoderShape, TensorParallelDecoder, reference_weights

    shape = DecoderShape(hidden=256, intermediate=512, heads=4, kv_heads=2, head_dim=128, layers=3, vocab=512)
    weights = reference_weights(shape, seed=4)
    ids = torch.randint(0, shape.vocab, (6, 32), generator=torch.Generator().manual_seed(5))
    model = load_oracle_model(shape, weights).cuda()
    want = oracle_hidden(model, ids.cuda()).reshape(-1, shape.hidden)
    for micro_batches in (2, 1, 3):
        dec = TensorParallelDecoder(shape, max_rows=6 * 32, micro_batches=micro_batches, weights=weights)
        got = dec.forward(ids.cuda())
        torch.cuda.synchronize()
        ops.check_status()
        rel = ((got.float() - want.float()).abs().max() / want.float().abs().max()).item()
        assert got.shape == want.shape and rel <= TOL, (micro_batches, rel)
        logits = dec.logits_last_token(got, 6, 32)
        with torch.inference_mode():
            want_logits = model.lm_head(want.view(6, 32, -1)[:, -1])
        rel = ((logits.float() - want_logits.float()).abs().max() / want_logits.float().abs().max()).item()
        assert rel <= TOL


def test_rope_kernel_matches_rotate_half(native_lib):
    from oracle import llama_oracle

    g = torch.Generator().manual_seed(6)
    T, heads, hd = 70, 6, 64
    extra = 2 * hd                                    # trailing v columns that must stay untouched
    x = torch.randn(T, heads * hd + extra, generator=g).bfloat16()
    pos = torch.randint(0, 500, (T,), generator=g, dtype=torch.int32)
    dev = x.cuda()
    rc = native_lib.df_rope_bf16(dev.data_ptr(), pos.cuda().data_ptr(), T, heads, hd, dev.stride(0), 10000.0, None)
    assert rc == 0
    torch.cuda.synchronize()
    cos_all, sin_all = llama_oracle.rope_tables(500, hd, 10000.0)
    cos, sin = cos_all[pos.long()], sin_all[pos.long()]             # [T, hd]
    heads_in = x[:, :heads * hd].view(T, heads, hd).transpose(0, 1).unsqueeze(0)   # [1, heads, T, hd]
    want = llama_oracle.apply_rope(heads_in, cos, sin)[0].transpose(0, 1).reshape(T, heads * hd)
    got = dev.cpu()
    assert torch.equal(got[:, heads * hd:], x[:, heads * hd:])
    rel = ((got[:, :heads * hd].float() - want.float()).abs().max() / want.float().abs().max()).item()
    assert rel <= 1e-2


def test_decode_step_matches_pytorch_decoder(native_lib):
    """One decode step (new token against a key/value cache, two micro-batches) on the native kernels,
    eagerly and replayed from one CUDA graph, against the PyTorch decoder run over the whole sequences:
    the cache is filled with the oracle's own rotated keys and values of the earlier positions."""
    from dynaflow_b200 import ops
    from dynaflow_b200.decoder import DecoderShape, TensorParallelDecoder, reference_weights
    from oracle import llama_oracle

    shape = DecoderShape(hidden=256, intermediate=512, heads=4, kv_heads=2, head_dim=128, layers=2, vocab=512)
    weights = reference_weights(shape, seed=14)
    B, L, max_len = 6, 150, 200
    ids = torch.randint(0, shape.vocab, (B, L), generator=torch.Generator().manual_seed(15)).cuda()
    model = load_oracle_model(shape, weights).cuda()
    keys, values = [], []
    with torch.inference_mode():
        cos, sin = llama_oracle.rope_tables(L, shape.head_dim, shape.rope_theta, device=ids.device)
        x = model.embed(ids)
        for blk in model.blocks:
            h = blk.input_norm(x)
            k = blk.attn.k_proj(h).view(B, L, shape.kv_heads, shape.head_dim).transpose(1, 2)
            v = blk.attn.v_proj(h).view(B, L, shape.kv_heads, shape.head_dim).transpose(1, 2)
            keys.append(llama_oracle.apply_rope(k, cos, sin).transpose(1, 2).reshape(B, L, -1))
            values.append(v.transpose(1, 2).reshape(B, L, -1))
            x = blk(x, cos, sin)
        want = model.lm_head(model.norm(x)[:, -1])
    dec = TensorParallelDecoder(shape, max_rows=B, micro_batches=2, weights=weights)
    dec.init_decode(B, max_len, context_len=L, fill_seed=None)
    for li in range(shape.layers):
        dec.k_cache[li, :, :L - 1].copy_(keys[li][:, :L - 1])
        dec.v_cache[li, :, :L - 1].copy_(values[li][:, :L - 1])
    last = ids[:, -1].contiguous()
    got = torch.cat(dec.decode_step(last)).clone()
    torch.cuda.synchronize()
    ops.check_status()
    rel = ((got.float() - want.float()).abs().max() / want.float().abs().max()).item()
    assert got.shape == want.shape and rel <= TOL, rel
    # the step wrote the new token's keys and values where the oracle has them
    assert ((dec.k_cache[0, :, L - 1].float() - keys[0][:, L - 1].float()).abs().max()
            / keys[0].float().abs().max()).item() <= TOL
    # the same step as one CUDA graph, replayed twice
    replay, logits = dec.capture_decode(last)
    for _ in range(2):
        for lg in logits:
            lg.zero_()
        replay()
        torch.cuda.synchronize()
        ops.check_status()
        again = torch.cat(logits)
        assert torch.equal(again, got)
    # without programmatic dependent launches (every kernel waits for its predecessor to drain before
    # it starts): the same bits, eagerly and from a graph captured in that mode
    ops.set_launch_option("dependent_launch", False)
    try:
        plain = torch.cat(dec.decode_step(last)).clone()
        replay2, logits2 = dec.capture_decode(last)
        replay2()
        torch.cuda.synchronize()
        ops.check_status()
        assert torch.equal(plain, got) and torch.equal(torch.cat(logits2), got)
    finally:
        ops.set_launch_option("dependent_launch", True)
