"""Top-2 mixture-of-experts layer as the reference's operator triple dispatch / expert / combine
(``examples/ae/patch/vllm.patch:308-379, 423-527``), on the native kernels.

* ``dispatch``: all-gather of the ranks' token rows and router logits (the reference's
  all-gather based manager, ``vllm.patch:87-100``), over peer memory;
* ``expert``: top-2 routing on all tokens, then for every LOCAL expert: select its tokens
  (count stays on the device), gather them into a dense matrix, run the fused gated MLP over
  exactly that many rows, scale by the routing weight and scatter back -- the rank's
  contribution to every token;
* ``combine``: reduce-scatter of the contributions, each rank receiving its own tokens
  (``vllm.patch:103-115``).

``exchange="a2a"`` selects the all-to-all form of the same triple (the reference's all2all managers,
``vllm.patch:145-191``): routing happens on the token owner, ``dispatch`` exchanges per-(source,
expert) counts and PUTS only the routed rows into the owner's packed expert input over peer memory,
``expert`` runs each local expert over exactly the rows that arrived, ``combine`` PULLS the two
expert outputs of every token back and applies the routing weights (``df_a2a_*``).

With one rank the collectives are the identity and the layer is a single-GPU MoE. The three
methods launch on the current stream and never synchronise with the host, so a policy (the
DBO schedule) can place dispatch / combine on the communication stream under the expert GEMMs
of the other nano-batch.
"""
from __future__ import annotations

import ctypes

import torch

from . import _native, ops
from ._native import df_a2a_rank_t
from .comm import PeerComm, _bf16_view, _check


class A2ARegions:
    """One all-to-all region per nano-batch slot on every rank (flags, exchanged counts, per local
    expert the arrived row count and the packed input / output buffers), allocated through the C ABI
    and mapped by every peer over CUDA IPC (handles exchanged with ``all_gather_object``)."""

    def __init__(self, rank: int, world: int, experts: int, capacity: int, hidden: int, slots: int,
                 device: torch.device, group=None) -> None:
        import torch.distributed as dist

        self.lib = _native.load()
        self.rank, self.world, self.experts, self.capacity, self.hidden = rank, world, experts, capacity, hidden
        self.device = device
        self.local_experts = experts // world
        self.bytes = int(self.lib.df_a2a_region_bytes(world, experts, capacity, hidden))
        self.in_off = int(self.lib.df_a2a_packed_in_offset(world, experts, capacity, hidden))
        self.out_off = int(self.lib.df_a2a_packed_out_offset(world, experts, capacity, hidden))
        self.rows_off = int(self.lib.df_a2a_rows_total_offset())
        self.local: list[int] = []
        self._opened: list[int] = []
        handles = []
        with torch.cuda.device(device):
            for _ in range(slots):
                ptr, handle = ctypes.c_void_p(), (ctypes.c_ubyte * 64)()
                _check(self.lib.df_comm_region_alloc(self.bytes, ctypes.byref(ptr), ctypes.byref(handle)), "df_comm_region_alloc")
                self.local.append(ptr.value)
                handles.append(bytes(handle))
        gathered = [None] * world
        if world > 1:
            dist.all_gather_object(gathered, handles, group=group)
        else:
            gathered[0] = handles
        self.views = []
        with torch.cuda.device(device):
            for slot in range(slots):
                view = df_a2a_rank_t()
                view.rank = rank
                for r in range(world):
                    if r == rank:
                        view.regions[r] = self.local[slot]
                        continue
                    ptr = ctypes.c_void_p()
                    handle = (ctypes.c_ubyte * 64).from_buffer_copy(gathered[r][slot])
                    _check(self.lib.df_comm_region_open(ctypes.byref(handle), ctypes.byref(ptr)), "df_comm_region_open")
                    view.regions[r] = ptr.value
                    self._opened.append(ptr.value)
                self.views.append(view)
        if world > 1:
            dist.barrier(group=group)

    def packed(self, slot: int, local_expert: int, out: bool) -> torch.Tensor:
        base = self.local[slot] + (self.out_off if out else self.in_off) + local_expert * self.capacity * self.hidden * 2
        return _bf16_view(base, self.capacity, self.hidden, self.device)

    def rows_total_ptr(self, slot: int, local_expert: int) -> int:
        return self.local[slot] + self.rows_off + 4 * local_expert

    def close(self) -> None:
        torch.cuda.synchronize(self.device)
        with torch.cuda.device(self.device):
            for ptr in self._opened:
                self.lib.df_comm_region_close(ptr)
            for ptr in self.local:
                self.lib.df_comm_region_free(ptr)
        self._opened, self.local = [], []


class ExpertParallelMoE:
    def __init__(self, hidden: int, intermediate: int, num_experts: int, tokens_per_rank: int, *, rank: int = 0,
                 world: int = 1, weights: tuple[torch.Tensor, torch.Tensor, torch.Tensor] | None = None, seed: int = 0,
                 slots: int = 2, n_ctas: int = 32, device: torch.device | None = None, exchange: str = "agrs") -> None:
        if exchange not in ("agrs", "a2a"):
            raise ValueError("exchange must be 'agrs' (all-gather / reduce-scatter) or 'a2a' (all-to-all puts and pulls)")
        self.exchange = exchange
        if num_experts % world != 0:
            raise ValueError("experts must divide evenly across ranks")
        if num_experts % 8 != 0:
            raise ValueError("the router width must be a multiple of 8 (16-byte rows)")
        self.lib = _native.load()
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.hidden, self.intermediate, self.num_experts = hidden, intermediate, num_experts
        self.rank, self.world = rank, world
        self.tokens_per_rank = tokens_per_rank
        self.total_tokens = tokens_per_rank * world
        per = num_experts // world
        self.local_experts = list(range(rank * per, (rank + 1) * per))
        if weights is None:
            g = torch.Generator().manual_seed(seed)
            w_gate = (torch.randn(num_experts, intermediate, hidden, generator=g) * 0.02).bfloat16()
            w_up = (torch.randn(num_experts, intermediate, hidden, generator=g) * 0.02).bfloat16()
            w_down = (torch.randn(num_experts, hidden, intermediate, generator=g) * 0.02).bfloat16()
        else:
            w_gate, w_up, w_down = weights
        sel = slice(self.local_experts[0], self.local_experts[-1] + 1)
        self.w_gate = w_gate[sel].contiguous().to(self.device)
        self.w_up = w_up[sel].contiguous().to(self.device)
        self.w_down = w_down[sel].contiguous().to(self.device)
        self.slots = slots
        T = self.total_tokens
        dev = self.device
        # per nano-batch slot: routing results, per-expert selection, packed expert input / output
        self.ids = [torch.empty(T, 2, dtype=torch.int32, device=dev) for _ in range(slots)]
        self.route_w = [torch.empty(T, 2, dtype=torch.float32, device=dev) for _ in range(slots)]
        self.rows = [torch.empty(T, dtype=torch.int32, device=dev) for _ in range(slots)]
        self.slot_of = [torch.empty(T, dtype=torch.int32, device=dev) for _ in range(slots)]
        self.pos = [torch.empty(T, dtype=torch.int32, device=dev) for _ in range(slots)]
        self.count = [torch.zeros(1, dtype=torch.int32, device=dev) for _ in range(slots)]
        self.packed_in = [torch.empty(T, hidden, dtype=torch.bfloat16, device=dev) for _ in range(slots)]
        self.packed_out = [torch.empty(T, hidden, dtype=torch.bfloat16, device=dev) for _ in range(slots)]
        self.scratch = [torch.empty(T, hidden, dtype=torch.bfloat16, device=dev) for _ in range(slots)]
        ws = ops.mlp_workspace_bytes(T, hidden, intermediate)
        self.workspace = [torch.empty(ws, dtype=torch.uint8, device=dev) for _ in range(slots)]
        self.n_ctas = n_ctas
        self.a2a = None
        if exchange == "a2a":
            # only routed rows move: per slot the local routing (ids, weights of this rank's tokens), the
            # positions of its pairs, and the regions the peers put into / pull from
            self.a2a = A2ARegions(rank, world, num_experts, T, hidden, slots, dev)
            Tr = tokens_per_rank
            self.l_ids = [torch.empty(Tr, 2, dtype=torch.int32, device=dev) for _ in range(slots)]
            self.l_w = [torch.empty(Tr, 2, dtype=torch.float32, device=dev) for _ in range(slots)]
            self.l_pos = [torch.empty(Tr, 2, dtype=torch.int32, device=dev) for _ in range(slots)]
            self.l_counts = [torch.zeros(num_experts, dtype=torch.int32, device=dev) for _ in range(slots)]
            self.l_out = [torch.empty(Tr, hidden, dtype=torch.bfloat16, device=dev) for _ in range(slots)]
            self.comm_x = self.comm_logits = self.comm_out = None
        elif world > 1:
            self.comm_x = PeerComm(rank, world, T, hidden, slots=slots, n_ctas=n_ctas, device=dev)
            self.comm_logits = PeerComm(rank, world, T, num_experts, slots=slots, n_ctas=4, device=dev)
            self.comm_out = PeerComm(rank, world, T, hidden, slots=slots, n_ctas=n_ctas, device=dev)
        else:
            self.comm_x = self.comm_logits = self.comm_out = None
            self.local_contrib = [torch.empty(T, hidden, dtype=torch.bfloat16, device=dev) for _ in range(slots)]

    def _stream(self) -> int:
        return torch.cuda.current_stream(self.device).cuda_stream

    def _collective(self, comm: PeerComm, slot: int, fn_name: str) -> None:
        fn = getattr(self.lib, fn_name)
        rc = fn(ctypes.byref(comm._plain_views[slot]), comm.world, comm.max_rows, comm.hidden, self.total_tokens,
                comm.n_ctas, comm._status_ptr, self._stream())
        if rc != 0:
            _check(rc, fn_name)

    # ---------------------------------------------------------------- the operator triple
    def dispatch(self, x_local: torch.Tensor, logits_local: torch.Tensor, slot: int = 0):
        """``[tokens_per_rank, H]`` and ``[tokens_per_rank, E]`` of this rank -> all ranks' rows."""
        if self.exchange == "a2a":
            return self._dispatch_a2a(x_local, logits_local, slot)
        if self.world == 1:
            return x_local, logits_local
        lo = self.rank * self.tokens_per_rank
        self.comm_x.partial(slot, self.total_tokens)[lo:lo + self.tokens_per_rank].copy_(x_local)
        self.comm_logits.partial(slot, self.total_tokens)[lo:lo + self.tokens_per_rank].copy_(logits_local)
        self._collective(self.comm_x, slot, "df_all_gather_bf16")
        self._collective(self.comm_logits, slot, "df_all_gather_bf16")
        return self.comm_x.result(slot, self.total_tokens), self.comm_logits.result(slot, self.total_tokens)

    def expert(self, x_all: torch.Tensor, logits_all: torch.Tensor, slot: int = 0) -> torch.Tensor:
        """This rank's experts' contribution to every token: ``[total_tokens, H]``, zeros where
        none of the local experts was chosen."""
        if self.exchange == "a2a":
            return self._expert_a2a(slot)
        T, H, I = self.total_tokens, self.hidden, self.intermediate
        st = ops.status_block(self.device).data_ptr()
        s = self._stream()
        lib = self.lib
        _check(lib.df_moe_route_top2(logits_all.data_ptr(), T, self.num_experts, self.ids[slot].data_ptr(),
                                     self.route_w[slot].data_ptr(), s), "df_moe_route_top2")
        target = (self.comm_out.partial(slot, T) if self.world > 1 else self.local_contrib[slot])
        for j, e in enumerate(self.local_experts):
            _check(lib.df_moe_select_rows(self.ids[slot].data_ptr(), T, e, self.rows[slot].data_ptr(),
                                          self.slot_of[slot].data_ptr(), self.pos[slot].data_ptr(),
                                          self.count[slot].data_ptr(), s), "df_moe_select_rows")
            _check(lib.df_moe_gather_rows(x_all.data_ptr(), self.rows[slot].data_ptr(), self.count[slot].data_ptr(), T, H,
                                          self.packed_in[slot].data_ptr(), s), "df_moe_gather_rows")
            _check(lib.df_mlp_gated_bf16_rows_on_device(
                self.packed_in[slot].data_ptr(), self.w_gate[j].data_ptr(), self.w_up[j].data_ptr(),
                self.w_down[j].data_ptr(), self.packed_out[slot].data_ptr(), self.workspace[slot].data_ptr(), T,
                self.count[slot].data_ptr(), H, I, 0, st, s), "df_mlp_gated_bf16_rows_on_device")
            # the first local expert writes its contribution (zeros included), later ones are summed in
            dst = target if j == 0 else self.scratch[slot]
            _check(lib.df_moe_scatter_rows(self.packed_out[slot].data_ptr(), self.pos[slot].data_ptr(),
                                           self.slot_of[slot].data_ptr(), self.route_w[slot].data_ptr(), T, H,
                                           dst.data_ptr(), s), "df_moe_scatter_rows")
            if j > 0:
                target.add_(dst)
        return target

    def combine(self, contrib: torch.Tensor, slot: int = 0) -> torch.Tensor:
        """Sum of all ranks' contributions for this rank's own tokens: ``[tokens_per_rank, H]``."""
        if self.exchange == "a2a":
            return self._combine_a2a(slot)
        if self.world == 1:
            return contrib
        self._collective(self.comm_out, slot, "df_reduce_scatter_bf16")
        lo = self.rank * self.tokens_per_rank
        return self.comm_out.result(slot, self.total_tokens)[lo:lo + self.tokens_per_rank]

    # ---------------------------------------------------------------- the all-to-all form
    def _dispatch_a2a(self, x_local: torch.Tensor, logits_local: torch.Tensor, slot: int):
        """Routes this rank's tokens, exchanges the per-(source, expert) counts and puts every routed
        row into the packed input of the rank that owns its expert."""
        lib, a, s = self.lib, self.a2a, self._stream()
        Tr, E = self.tokens_per_rank, self.num_experts
        st = ops.status_block(self.device).data_ptr()
        _check(lib.df_moe_route_top2(logits_local.data_ptr(), Tr, E, self.l_ids[slot].data_ptr(), self.l_w[slot].data_ptr(), s),
               "df_moe_route_top2")
        _check(lib.df_a2a_plan(self.l_ids[slot].data_ptr(), Tr, E, self.l_pos[slot].data_ptr(),
                               self.l_counts[slot].data_ptr(), s), "df_a2a_plan")
        _check(lib.df_a2a_dispatch_bf16(ctypes.byref(a.views[slot]), self.world, E, a.capacity, self.hidden, x_local.data_ptr(),
                                        self.l_ids[slot].data_ptr(), self.l_pos[slot].data_ptr(),
                                        self.l_counts[slot].data_ptr(), Tr, self.n_ctas, st, s), "df_a2a_dispatch_bf16")
        return None, None

    def _expert_a2a(self, slot: int):
        """The gated MLP of every local expert over exactly the rows that arrived for it."""
        lib, a, s = self.lib, self.a2a, self._stream()
        st = ops.status_block(self.device).data_ptr()
        for j in range(len(self.local_experts)):
            _check(lib.df_mlp_gated_bf16_rows_on_device(
                a.packed(slot, j, False).data_ptr(), self.w_gate[j].data_ptr(), self.w_up[j].data_ptr(),
                self.w_down[j].data_ptr(), a.packed(slot, j, True).data_ptr(), self.workspace[slot].data_ptr(), a.capacity,
                a.rows_total_ptr(slot, j), self.hidden, self.intermediate, 0, st, s), "df_mlp_gated_bf16_rows_on_device")
        return None

    def _combine_a2a(self, slot: int) -> torch.Tensor:
        """Pulls the two expert outputs of each of this rank's tokens and sums them with the routing weights."""
        lib, a, s = self.lib, self.a2a, self._stream()
        st = ops.status_block(self.device).data_ptr()
        _check(lib.df_a2a_combine_bf16(ctypes.byref(a.views[slot]), self.world, self.num_experts, a.capacity, self.hidden,
                                       self.l_ids[slot].data_ptr(), self.l_pos[slot].data_ptr(), self.l_w[slot].data_ptr(),
                                       self.tokens_per_rank, self.l_out[slot].data_ptr(), self.n_ctas, st, s),
               "df_a2a_combine_bf16")
        return self.l_out[slot]

    def forward(self, x_local: torch.Tensor, logits_local: torch.Tensor, slot: int = 0) -> torch.Tensor:
        x_all, logits_all = self.dispatch(x_local, logits_local, slot)
        return self.combine(self.expert(x_all, logits_all, slot), slot)

    def close(self) -> None:
        for c in (self.comm_x, self.comm_logits, self.comm_out, self.a2a):
            if c is not None:
                c.close()
