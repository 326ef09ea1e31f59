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
  * all-reduce + residual + RMSNorm and the top-2 MoE routing: the arithmetic lives
    in third-party code that is not part of the reference tree (flashinfer,
    unpinned; vLLM @2dda3e35 ``RMSNorm``; vLLM fused-MoE routing), and the reference
    has no vectors for it: PARITY UNPINNED. The restatement follows the call sites
    and the in-tree kernel ``tokenweave.cu:38-113``.
"""
