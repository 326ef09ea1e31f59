"""CPU restatement of the reference's algorithms for the hot path.

TEST INFRASTRUCTURE ONLY. Nothing in the ``dynaflow_b200`` package imports this
directory; only ``tests/``, ``__graft_entry__.smoke()`` and the ``cpu_baseline`` /
``--impl reference`` legs of ``bench.py`` do, and only as the checker or as the
timed CPU baseline.

Pinning status
  * split / merge indexing, ``get_split_config`` arithmetic, graph partitioning and
    the dispatch order of the round-robin policy: PINNED against the reference
    package itself, executed on CPU in the build container
    (``tests/golden/make_golden.py`` wrote ``tests/golden/*.json|*.pt`` from it).
  * gated MLP: PINNED to the reference's own PyTorch execution of the split MLP
    graph on CPU (same fixtures); the GPU kernels are compared within 2e-2.
  * residual add + RMSNorm after the all-reduce: PINNED. The reference engine executed
    ``residual + y`` followed by transformers' ``LlamaRMSNorm`` (bf16, eps 1e-5) in two
    ragged nano-batches (``tests/golden/norm_split.*``); the oracle reproduces output and
    new residual bit for bit. The cross-rank sum itself (NCCL / flashinfer / NVLS in the
    reference's hosts) cannot run in the build container: the fixture feeds the module the
    fp32 rank-order sum of four stored partials, which is the oracle's definition of it.
  * top-2 MoE: PINNED to the reference engine's execution of a Mixtral-style block whose
    router arithmetic is transformers' ``MixtralTopKRouter`` (``tests/golden/moe_split.*``):
    expert ids and routing weights bit for bit, the layer output bit for bit with the
    operator-chain expert form and within 2e-2 in the fused-epilogue form. The fixture has
    no tied logits (``torch.topk`` does not specify their order); ties resolve to the lower
    expert index here and in the CUDA kernel.
  * causal attention: the reference treats it as an opaque subgraph run by the host's
    kernels; the oracle states ``scaled_dot_product_attention(is_causal=True)`` in fp32 and
    is checked against PyTorch's own implementation in ``tests/test_oracle_golden.py``.
"""
