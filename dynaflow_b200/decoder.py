"""A Llama-style decoder stack on the batch-split, overlapped schedule, tensor parallel.

Everything on the hot path runs on this library's kernels: fused qkv projection and output
projection (``ops.gemm_bf16``), rotary embedding (``df_rope_bf16``), causal attention
(``ops.attention_prefill``, reading q, k, v as column ranges of the fused qkv rows and writing
the rows the output projection reads -- no transposes; the reference leaves this subgraph to the
host model's kernels, ``examples/ae/scheduler/vllm/nanoflow.py:91-94``), the gated MLP
(``ops.gated_mlp``), and between the blocks the reduce-scatter / residual add / RMSNorm /
all-gather kernel on the communication stream (single rank: the stand-alone add + RMSNorm
kernel). Head dimension 128 only.

Schedule: the requests are cut into micro-batches; for every half-block (attention part,
MLP part) the micro-batches run in order on the compute stream, and the reduction of
micro-batch ``i`` runs on the communication stream under the GEMMs of micro-batch ``i+1``
(NanoFlow's round-robin, ``examples/ae/scheduler/hf/nanoflow.py:123-146``, at the granularity
of the subgraphs its split rules produce).

Sharding (Megatron): q/k/v heads and the MLP intermediate by columns, o and down by rows;
activations between blocks are replicated, the residual stream is sharded by rows.
"""
from __future__ import annotations

import dataclasses

import torch

from . import _native, ops
from .comm import MulticastComm, PeerComm, add_rmsnorm


@dataclasses.dataclass
class DecoderShape:
    hidden: int = 4096
    intermediate: int = 14336
    heads: int = 32
    kv_heads: int = 8
    head_dim: int = 128
    layers: int = 32
    vocab: int = 128256
    eps: float = 1e-5
    rope_theta: float = 10000.0


class TensorParallelDecoder:
    def __init__(self, shape: DecoderShape, *, rank: int = 0, world: int = 1, max_rows: int, micro_batches: int = 2,
                 seed: int = 0, device: torch.device | None = None, weights: dict | None = None, n_ctas: int = 32,
                 multicast: bool = False, gemm_max_ctas: int = 0) -> None:
        s = shape
        if s.heads % world or s.kv_heads % world or s.intermediate % world:
            raise ValueError("heads, kv heads and the intermediate size must divide evenly across ranks")
        if s.head_dim != 128:
            raise ValueError("the attention kernel is built for a head dimension of 128")
        self.s, self.rank, self.world = s, rank, world
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.micro_batches = micro_batches
        self.max_rows = max_rows
        self.qh, self.kvh = s.heads // world, s.kv_heads // world
        self.q_cols, self.kv_cols = self.qh * s.head_dim, self.kvh * s.head_dim
        self.inter = s.intermediate // world
        self.lib = _native.load()
        dev = self.device
        # random weights are drawn on the device (same seed => same full matrices on every rank)
        gen = torch.Generator(device=dev).manual_seed(seed)

        def full(name, *shp):
            if weights is not None:
                return weights[name]
            return (torch.randn(*shp, generator=gen, device=dev) * 0.02).bfloat16()

        self.embed = full("embed", s.vocab, s.hidden).to(dev)
        self.lm_head = full("lm_head", s.vocab, s.hidden).to(dev)
        self.layers = []
        r = rank
        for i in range(s.layers):
            wq = full(f"l{i}.q", s.heads * s.head_dim, s.hidden)
            wk = full(f"l{i}.k", s.kv_heads * s.head_dim, s.hidden)
            wv = full(f"l{i}.v", s.kv_heads * s.head_dim, s.hidden)
            wo = full(f"l{i}.o", s.hidden, s.heads * s.head_dim)
            wg = full(f"l{i}.gate", s.intermediate, s.hidden)
            wu = full(f"l{i}.up", s.intermediate, s.hidden)
            wd = full(f"l{i}.down", s.hidden, s.intermediate)
            qs, ks, ms = slice(r * self.q_cols, (r + 1) * self.q_cols), slice(r * self.kv_cols, (r + 1) * self.kv_cols), \
                slice(r * self.inter, (r + 1) * self.inter)
            self.layers.append({
                "wqkv": torch.cat([wq[qs], wk[ks], wv[ks]], 0).contiguous().to(dev),
                "wo": wo[:, qs].contiguous().to(dev),
                "wg": wg[ms].contiguous().to(dev), "wu": wu[ms].contiguous().to(dev), "wd": wd[:, ms].contiguous().to(dev),
                "norm1": (weights[f"l{i}.norm1"] if weights else torch.ones(s.hidden).bfloat16()).to(dev),
                "norm2": (weights[f"l{i}.norm2"] if weights else torch.ones(s.hidden).bfloat16()).to(dev),
            })
        self.final_norm = (weights["final_norm"] if weights else torch.ones(s.hidden).bfloat16()).to(dev)
        n = micro_batches
        qkv_cols = self.q_cols + 2 * self.kv_cols
        self.qkv = [torch.empty(max_rows, qkv_cols, dtype=torch.bfloat16, device=dev) for _ in range(n)]
        self.attn_out = [torch.empty(max_rows, self.q_cols, dtype=torch.bfloat16, device=dev) for _ in range(n)]
        self.workspace = [torch.empty(ops.mlp_workspace_bytes(max_rows, s.hidden, self.inter), dtype=torch.uint8,
                                      device=dev) for _ in range(n)]
        self.x = [torch.empty(max_rows, s.hidden, dtype=torch.bfloat16, device=dev) for _ in range(n)]
        self.residual = [torch.empty(max_rows, s.hidden, dtype=torch.bfloat16, device=dev) for _ in range(n)]
        self.partial_local = [torch.empty(max_rows, s.hidden, dtype=torch.bfloat16, device=dev) for _ in range(n)]
        comm_cls = MulticastComm if multicast else PeerComm   # in-switch or peer-memory reduction
        self.comm = comm_cls(rank, world, max_rows, s.hidden, slots=n, n_ctas=n_ctas, device=dev) if world > 1 else None
        self.gemm_max_ctas = gemm_max_ctas                    # CTAs the GEMMs may use (0 = one per SM)
        self.launch_count = 0

    # ------------------------------------------------------------------ pieces
    def _partial(self, mb: int, rows: int) -> torch.Tensor:
        return self.comm.partial(mb, rows) if self.comm is not None else self.partial_local[mb][:rows]

    def _attention_half(self, layer: dict, x: torch.Tensor, mb: int, batch: int, seq: int, pos: torch.Tensor) -> None:
        s = self.s
        rows = batch * seq
        qkv = self.qkv[mb][:rows]
        ops.gemm_bf16(x, layer["wqkv"], out=qkv, max_ctas=self.gemm_max_ctas)
        rc = self.lib.df_rope_bf16(qkv.data_ptr(), pos.data_ptr(), rows, self.qh + self.kvh, s.head_dim, qkv.stride(0),
                                   s.rope_theta, torch.cuda.current_stream(self.device).cuda_stream)
        if rc != 0:
            raise RuntimeError(_native.last_error())
        attn = self.attn_out[mb][:rows]
        ops.attention_prefill(qkv[:, :self.q_cols], qkv[:, self.q_cols:self.q_cols + self.kv_cols],
                              qkv[:, self.q_cols + self.kv_cols:], attn, batch=batch, seq_len=seq,
                              max_ctas=self.gemm_max_ctas)
        ops.gemm_bf16(attn, layer["wo"], out=self._partial(mb, rows), max_ctas=self.gemm_max_ctas)
        self.launch_count += 4

    def _mlp_half(self, layer: dict, x: torch.Tensor, mb: int, rows: int) -> None:
        ops.gated_mlp(x, layer["wg"], layer["wu"], layer["wd"], out=self._partial(mb, rows), workspace=self.workspace[mb],
                      max_ctas=self.gemm_max_ctas)
        self.launch_count += 2

    def _reduce_norm(self, mb: int, rows: int, weight: torch.Tensor, first: bool = False) -> torch.Tensor:
        """Sum the ranks' partials, add the residual, normalise: the next half-block's input."""
        self.launch_count += 1
        if self.comm is None:
            x = self.x[mb][:rows]
            add_rmsnorm(self.partial_local[mb][:rows], None if first else self.residual[mb][:rows], weight, x,
                        self.residual[mb][:rows], self.s.eps)
            return x
        return self.comm.all_reduce_add_rmsnorm_sharded(mb, rows, self.residual[mb][:rows], weight, self.s.eps,
                                                        first=first)

    # ----------------------------------------------------------------- forward
    def forward(self, ids: torch.Tensor, skip_comm: bool = False, skip_compute: bool = False) -> torch.Tensor:
        """``ids`` [requests, seq] -> hidden states after the final norm, [requests * seq, hidden],
        as per-micro-batch views concatenated. Requests are cut evenly into micro-batches.
        ``skip_comm`` / ``skip_compute`` leave out the reductions, resp. the GEMMs and attention
        (timing of the two halves of the overlap; the values are then meaningless)."""
        s = self.s
        batch, seq = ids.shape
        n = min(self.micro_batches, batch)
        cuts = [batch * i // n for i in range(n + 1)]
        main = torch.cuda.current_stream(self.device)
        comm_stream = self.comm.stream if self.comm is not None else main
        pos = torch.arange(seq, device=self.device, dtype=torch.int32).repeat(cuts[1] - cuts[0] + 1)
        xs: list[torch.Tensor] = []
        rows_of = []
        for mb in range(n):
            b = cuts[mb + 1] - cuts[mb]
            rows = b * seq
            rows_of.append((b, rows))
            emb = self.embed[ids[cuts[mb]:cuts[mb + 1]].reshape(-1)]
            self.partial_local[mb][:rows].copy_(emb) if self.comm is None else self.comm.partial(mb, rows).copy_(emb)
            xs.append(None)
        if self.comm is not None:
            start = torch.cuda.Event()
            start.record(main)
            comm_stream.wait_event(start)
        done: list = [None] * n

        def reduce_after(mb: int, weight: torch.Tensor, first: bool = False) -> None:
            rows = rows_of[mb][1]
            if self.comm is None:
                xs[mb] = self._reduce_norm(mb, rows, weight, first)
                return
            ready = torch.cuda.Event()
            ready.record(main)
            if skip_comm:
                xs[mb] = self.comm.partial(mb, rows)
                return
            comm_stream.wait_event(ready)
            with torch.cuda.stream(comm_stream):
                xs[mb] = self._reduce_norm(mb, rows, weight, first)
                ev = torch.cuda.Event()
                ev.record(comm_stream)
            done[mb] = ev

        # the embedding is the first residual; with several ranks every rank only contributes 1/world of it
        for mb in range(n):
            if self.comm is not None:
                self.comm.partial(mb, rows_of[mb][1]).mul_(1.0 / self.world)
            reduce_after(mb, self.layers[0]["norm1"], first=True)
        for li, layer in enumerate(self.layers):
            for mb in range(n):
                if done[mb] is not None:
                    main.wait_event(done[mb])
                b, rows = rows_of[mb]
                if not skip_compute:
                    self._attention_half(layer, xs[mb], mb, b, seq, pos[:rows])
                reduce_after(mb, layer["norm2"])
            nxt = self.layers[li + 1]["norm1"] if li + 1 < len(self.layers) else self.final_norm
            for mb in range(n):
                if done[mb] is not None:
                    main.wait_event(done[mb])
                if not skip_compute:
                    self._mlp_half(layer, xs[mb], mb, rows_of[mb][1])
                reduce_after(mb, nxt)
        if self.comm is not None:
            main.wait_stream(comm_stream)
        return torch.cat([xs[mb] for mb in range(n)], 0)

    # ------------------------------------------------------------------ decode
    def init_decode(self, batch: int, max_len: int, context_len: int, fill_seed: int | None = 0) -> None:
        """Allocates what a decode step needs: per layer a key and a value cache
        ``[batch, max_len, kv_cols]`` (this rank's key/value heads), filled N(0, 1) from
        ``fill_seed`` (``None``: zeros), the sequence lengths (every sequence holds ``context_len``
        keys AFTER the new token has been appended), and the split-KV workspace."""
        s, dev = self.s, self.device
        n = min(self.micro_batches, batch)
        self.d_batch, self.d_max_len = batch, max_len
        self.d_cuts = [batch * i // n for i in range(n + 1)]
        gen = torch.Generator(device=dev).manual_seed(fill_seed if fill_seed is not None else 0)
        shape = (s.layers, batch, max_len, self.kv_cols)
        if fill_seed is None:
            self.k_cache = torch.zeros(shape, dtype=torch.bfloat16, device=dev)
            self.v_cache = torch.zeros(shape, dtype=torch.bfloat16, device=dev)
        else:
            self.k_cache = torch.empty(shape, dtype=torch.bfloat16, device=dev)
            self.v_cache = torch.empty(shape, dtype=torch.bfloat16, device=dev)
            for li in range(s.layers):           # layer by layer: no fp32 copy of the whole cache
                self.k_cache[li].copy_(torch.randn(shape[1:], generator=gen, device=dev))
                self.v_cache[li].copy_(torch.randn(shape[1:], generator=gen, device=dev))
        self.seq_lens = torch.full((batch,), context_len, dtype=torch.int32, device=dev)
        rows = max(self.d_cuts[i + 1] - self.d_cuts[i] for i in range(n))
        self.attn_ws = [ops.attention_decode_workspace(rows, self.qh, self.kvh, max_len, dev) for _ in range(n)]
        self.decode_streams = [torch.cuda.Stream(device=dev) for _ in range(max(n - 1, 0))]
        # One compute stream per micro-batch pays without reductions (one GPU: 6.02 -> 5.17 ms on one rank's share of the
        # 8-rank step, the projections of one micro-batch run beside the attention of the other). With reductions the
        # two chains each wait for their own reductions and the gain is gone (2 ranks 17.5 vs 17.3 ms, 4 ranks 10.2 vs
        # 10.3 ms), so the single compute stream, whose stagger hides the reductions, stays the tensor-parallel default.
        self.decode_streams_per_micro_batch = self.comm is None
        per = s.vocab // self.world
        self.lm_head_shard = self.lm_head[self.rank * per:(self.rank + 1) * per].contiguous()
        self.logits = [torch.empty(rows, per, dtype=torch.bfloat16, device=dev) for _ in range(n)]

    def _attention_half_decode(self, li: int, layer: dict, x: torch.Tensor, mb: int) -> None:
        """qkv projection, RoPE at the sequences' last positions, the new keys and values into the
        cache, split-KV attention over the cache, output projection into the partial buffer."""
        s = self.s
        lo, hi = self.d_cuts[mb], self.d_cuts[mb + 1]
        rows = hi - lo
        qkv = self.qkv[mb][:rows]
        ops.gemm_bf16(x, layer["wqkv"], out=qkv, max_ctas=self.gemm_max_ctas)
        kc, vc = self.k_cache[li, lo:hi], self.v_cache[li, lo:hi]
        ops.rope_append(qkv, self.seq_lens[lo:hi], self.qh, self.kvh, kc, vc, s.rope_theta)
        attn = self.attn_out[mb][:rows]
        ops.attention_decode(qkv[:, :self.q_cols], kc, vc, self.seq_lens[lo:hi], attn, self.attn_ws[mb],
                             max_ctas=self.gemm_max_ctas)
        ops.gemm_bf16(attn, layer["wo"], out=self._partial(mb, rows), max_ctas=self.gemm_max_ctas)
        self.launch_count += 4

    def decode_step(self, ids: torch.Tensor, skip_comm: bool = False, skip_compute: bool = False) -> list[torch.Tensor]:
        """One new token per sequence: ``ids [batch]`` -> per micro-batch this rank's slice of the
        logits ``[rows, vocab / world]``. Same schedule as ``forward``: the micro-batches' compute on
        the current stream, the reduction of micro-batch i on the communication stream under the
        kernels of micro-batch i+1 (attention of one under the reduction of the other). Allocates
        nothing and never synchronises with the host, so it can be captured into one CUDA graph
        (``capture_decode``); the sequence lengths stay in device memory."""
        n = len(self.d_cuts) - 1
        main = torch.cuda.current_stream(self.device)
        comm_stream = self.comm.stream if self.comm is not None else main
        # one compute stream per micro-batch (``decode_streams_per_micro_batch``): the chains of the micro-batches only
        # meet in the communication stream, so the latency-bound projections of one run beside the attention of the other
        cs = [main] + [self.decode_streams[i] if self.decode_streams_per_micro_batch else main for i in range(n - 1)]
        xs: list = [None] * n
        rows_of = [self.d_cuts[i + 1] - self.d_cuts[i] for i in range(n)]
        for mb in range(n):
            target = self.partial_local[mb][:rows_of[mb]] if self.comm is None else self.comm.partial(mb, rows_of[mb])
            torch.index_select(self.embed, 0, ids[self.d_cuts[mb]:self.d_cuts[mb + 1]], out=target)
            if self.comm is not None:
                target.mul_(1.0 / self.world)
        start = torch.cuda.Event()
        start.record(main)
        for stream in {id(s): s for s in cs[1:] + ([comm_stream] if self.comm is not None else [])}.values():
            if stream is not main:
                stream.wait_event(start)
        done: list = [None] * n

        def reduce_after(mb: int, weight: torch.Tensor, first: bool = False) -> None:
            rows = rows_of[mb]
            if self.comm is None:
                with torch.cuda.stream(cs[mb]):
                    xs[mb] = self._reduce_norm(mb, rows, weight, first)
                return
            ready = torch.cuda.Event()
            ready.record(cs[mb])
            if skip_comm:
                xs[mb] = self.comm.partial(mb, rows)
                return
            comm_stream.wait_event(ready)
            with torch.cuda.stream(comm_stream):
                xs[mb] = self._reduce_norm(mb, rows, weight, first)
                ev = torch.cuda.Event()
                ev.record(comm_stream)
            done[mb] = ev

        for mb in range(n):
            reduce_after(mb, self.layers[0]["norm1"], first=True)
        for li, layer in enumerate(self.layers):
            for mb in range(n):
                if done[mb] is not None:
                    cs[mb].wait_event(done[mb])
                if li == 0 and mb > 0 and cs[mb] is not cs[mb - 1] and self.comm is not None:
                    # start half a layer behind the micro-batch before: its reductions then fall under this one's
                    # kernels and the other way round, instead of both chains waiting at the same time
                    stagger = torch.cuda.Event()
                    stagger.record(cs[mb - 1])
                    cs[mb].wait_event(stagger)
                if not skip_compute:
                    with torch.cuda.stream(cs[mb]):
                        self._attention_half_decode(li, layer, xs[mb], mb)
                reduce_after(mb, layer["norm2"])
            nxt = self.layers[li + 1]["norm1"] if li + 1 < len(self.layers) else self.final_norm
            for mb in range(n):
                if done[mb] is not None:
                    cs[mb].wait_event(done[mb])
                if not skip_compute:
                    with torch.cuda.stream(cs[mb]):
                        self._mlp_half(layer, xs[mb], mb, rows_of[mb])
                reduce_after(mb, nxt)
        out = []
        for mb in range(n):
            if done[mb] is not None:
                cs[mb].wait_event(done[mb])
            lg = self.logits[mb][:rows_of[mb]]
            if not skip_compute:
                with torch.cuda.stream(cs[mb]):
                    ops.gemm_bf16(xs[mb], self.lm_head_shard, out=lg, max_ctas=self.gemm_max_ctas)
            out.append(lg)
        for stream in cs[1:]:
            if stream is not main:
                main.wait_stream(stream)
        if self.comm is not None:
            main.wait_stream(comm_stream)
        self.last_hidden = xs
        return out

    def capture_decode(self, ids: torch.Tensor, **kw):
        """Runs one decode step eagerly (kernels loaded, workspaces created), then captures the step
        -- both streams, every kernel and reduction -- into ONE CUDA graph. Returns
        ``(replay, logits)``: ``replay()`` launches the graph on the current stream; ``ids`` is
        read at replay time from the tensor passed here, the sequence lengths from
        ``self.seq_lens``."""
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):          # the eager run on the capture stream: its scratch is created here
            self.decode_step(ids, **kw)
        torch.cuda.synchronize(self.device)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side, capture_error_mode="thread_local"):
                logits = self.decode_step(ids, **kw)
        torch.cuda.current_stream(self.device).wait_stream(side)
        return graph.replay, logits

    def logits_last_token(self, hidden: torch.Tensor, batch: int, seq: int) -> torch.Tensor:
        """Prefill only needs the logits of each request's last token."""
        last = hidden.view(batch, seq, -1)[:, -1, :].contiguous()
        return ops.gemm_bf16(last, self.lm_head)

    def close(self) -> None:
        if self.comm is not None:
            self.comm.close()


def reference_weights(shape: DecoderShape, seed: int = 0) -> dict:
    """Full (unsharded) bf16 weights N(0, 0.02) by name, for parity tests."""
    gen = torch.Generator().manual_seed(seed)
    s = shape
    w = {"embed": (torch.randn(s.vocab, s.hidden, generator=gen) * 0.02).bfloat16(),
         "lm_head": (torch.randn(s.vocab, s.hidden, generator=gen) * 0.02).bfloat16(),
         "final_norm": (1 + 0.1 * torch.randn(s.hidden, generator=gen)).bfloat16()}
    for i in range(s.layers):
        w[f"l{i}.q"] = (torch.randn(s.heads * s.head_dim, s.hidden, generator=gen) * 0.02).bfloat16()
        w[f"l{i}.k"] = (torch.randn(s.kv_heads * s.head_dim, s.hidden, generator=gen) * 0.02).bfloat16()
        w[f"l{i}.v"] = (torch.randn(s.kv_heads * s.head_dim, s.hidden, generator=gen) * 0.02).bfloat16()
        w[f"l{i}.o"] = (torch.randn(s.hidden, s.heads * s.head_dim, generator=gen) * 0.02).bfloat16()
        w[f"l{i}.gate"] = (torch.randn(s.intermediate, s.hidden, generator=gen) * 0.02).bfloat16()
        w[f"l{i}.up"] = (torch.randn(s.intermediate, s.hidden, generator=gen) * 0.02).bfloat16()
        w[f"l{i}.down"] = (torch.randn(s.hidden, s.intermediate, generator=gen) * 0.02).bfloat16()
        w[f"l{i}.norm1"] = (1 + 0.1 * torch.randn(s.hidden, generator=gen)).bfloat16()
        w[f"l{i}.norm2"] = (1 + 0.1 * torch.randn(s.hidden, generator=gen)).bfloat16()
    return w
