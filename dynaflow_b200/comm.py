"""Peer-memory communicator for the tensor-parallel reduction of a micro-batch.

``PeerComm`` is the multi-process form (one process per GPU): every rank allocates
one region per micro-batch slot through the C ABI, the 64-byte CUDA IPC handles are
exchanged with ``torch.distributed.all_gather_object`` (plumbing only), and each
rank maps its peers' regions. ``MulticastComm`` is the same communicator over an
NVLink multicast mapping (the regions come from ``torch.distributed._symmetric_memory``,
again plumbing only): the all-reduce and the sharded-residual fused form then reduce
inside the switch (``multimem.ld_reduce`` / ``multimem.st`` in the library's own
kernel). ``EmulatedComm`` keeps all ranks' regions on one GPU and runs them as one
cooperative launch (tests without a second GPU).

The all-reduce replaces the ``network``-tagged all-reduce (+ RMSNorm) subgraph of a
TP model (``examples/ae/scheduler/vllm/nanoflow.py:59-69, 171-211``); a policy
substitutes it with ``PeerComm.all_reduce`` / ``all_reduce_add_rmsnorm`` on its
communication stream.
"""
from __future__ import annotations

import ctypes
from typing import Any

import torch

from . import _native, ops
from ._native import df_comm_rank_t


class _DevicePointer:
    """Adapter exposing raw device memory to torch through ``__cuda_array_interface__``."""

    def __init__(self, ptr: int, nbytes: int) -> None:
        self.__cuda_array_interface__ = {"shape": (nbytes // 2,), "typestr": "<i2", "data": (ptr, False),
                                         "version": 2}


def _bf16_view(ptr: int, rows: int, hidden: int, device: torch.device) -> torch.Tensor:
    t = torch.as_tensor(_DevicePointer(ptr, rows * hidden * 2), device=device)
    return t.view(torch.bfloat16).view(rows, hidden)


def _check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what} failed ({rc}): {_native.last_error()}")


def set_exclusive_sms(on: bool) -> None:
    """Process-wide: with ``True`` every reduction CTA claims 40 KB of shared memory it does not
    use, which keeps it off the SMs that hold a GEMM CTA (and GEMM CTAs off its SM). Together with
    GEMMs launched on fewer CTAs than SMs (``TensorParallelGatedMLP.gemm_max_ctas``) the reduction
    then runs on SMs of its own, two CTAs per free SM."""
    _check(_native.load().df_comm_set_exclusive_smem(40960 if on else 0), "df_comm_set_exclusive_smem")


def multicast_supported(device: int | None = None) -> bool:
    """Whether the current (or given) device offers NVLink multicast mappings (driver attribute
    CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED)."""
    try:
        from cuda.bindings import driver as cu
    except ImportError:                      # older cuda-python layout
        from cuda import cuda as cu
    dev = torch.cuda.current_device() if device is None else device
    torch.cuda.init()
    err, value = cu.cuDeviceGetAttribute(cu.CUdevice_attribute.CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev)
    return int(err) == 0 and int(value) == 1


class _Regions:
    """Layout bookkeeping shared by the two communicators."""

    def __init__(self, world: int, max_rows: int, hidden: int, slots: int, n_ctas: int, device: torch.device) -> None:
        if not 1 <= world <= _native.MAX_WORLD:
            raise ValueError(f"world size {world} is outside [1, {_native.MAX_WORLD}]")
        if hidden % 8 != 0:
            raise ValueError("hidden must be a multiple of 8")
        self.lib = _native.load()
        self.world, self.max_rows, self.hidden, self.slots = world, max_rows, hidden, slots
        self.n_ctas = n_ctas
        self.device = device
        self.region_bytes = int(self.lib.df_comm_region_bytes(max_rows, hidden))
        self.partial_off = int(self.lib.df_comm_partial_offset(max_rows, hidden))
        self.sum_off = int(self.lib.df_comm_sum_offset(max_rows, hidden))
        self.launches = 0
        self.bytes_reduced = 0

    def _view(self, rank: int, regions: list[int], residual_in=None, residual_out=None, out=None) -> df_comm_rank_t:
        v = df_comm_rank_t()
        v.rank = rank
        for r, ptr in enumerate(regions):
            v.regions[r] = ptr
        v.residual_in = residual_in.data_ptr() if residual_in is not None else None
        v.residual_out = residual_out.data_ptr() if residual_out is not None else None
        v.out = out.data_ptr() if out is not None else None
        return v


class PeerComm(_Regions):
    def __init__(self, rank: int, world: int, max_rows: int, hidden: int, *, slots: int = 2, n_ctas: int = 32,
                 device: torch.device | None = None, group: Any = None) -> None:
        import torch.distributed as dist

        device = device or torch.device("cuda", torch.cuda.current_device())
        super().__init__(world, max_rows, hidden, slots, n_ctas, device)
        self.rank = rank
        self.local: list[int] = []
        self._opened: list[int] = []
        self.regions: list[list[int]] = []
        self._map_regions(group)
        if world > 1:
            dist.barrier(group=group)  # every rank has mapped every region before anyone launches
        self._partials = [_bf16_view(self.local[s] + self.partial_off, max_rows, hidden, device) for s in range(slots)]
        self._sums = [_bf16_view(self.local[s] + self.sum_off, max_rows, hidden, device) for s in range(slots)]
        self.stream = torch.cuda.Stream(device=device)
        # per-slot argument blocks of the plain all-reduce, built once (the launch path stays short)
        self._plain_views = [self._view(rank, self.regions[s]) for s in range(slots)]
        self._status_ptr = ops.status_block(device).data_ptr()

    def _map_regions(self, group: Any) -> None:
        """Fills ``self.local[slot]`` and ``self.regions[slot][r]`` (rank r's region of that slot as
        mapped in this process): allocation through the C ABI, CUDA IPC handles for the peers."""
        import torch.distributed as dist

        world, rank, slots, device = self.world, self.rank, self.slots, self.device
        handles: list[bytes] = []
        with torch.cuda.device(device):
            for _ in range(slots):
                ptr = ctypes.c_void_p()
                handle = (ctypes.c_ubyte * 64)()
                _check(self.lib.df_comm_region_alloc(self.region_bytes, ctypes.byref(ptr), ctypes.byref(handle)),
                       "df_comm_region_alloc")
                self.local.append(ptr.value)
                handles.append(bytes(handle))
        gathered: list[Any] = [None] * world
        if world > 1:
            dist.all_gather_object(gathered, handles, group=group)
        else:
            gathered[0] = handles
        with torch.cuda.device(device):
            for slot in range(slots):
                row = []
                for r in range(world):
                    if r == rank:
                        row.append(self.local[slot])
                        continue
                    ptr = ctypes.c_void_p()
                    handle = (ctypes.c_ubyte * 64).from_buffer_copy(gathered[r][slot])
                    _check(self.lib.df_comm_region_open(ctypes.byref(handle), ctypes.byref(ptr)), "df_comm_region_open")
                    row.append(ptr.value)
                    self._opened.append(ptr.value)
                self.regions.append(row)

    def partial(self, slot: int, rows: int) -> torch.Tensor:
        """Where this rank's partial sums of micro-batch slot ``slot`` must be written."""
        return self._partials[slot][:rows]

    def result(self, slot: int, rows: int) -> torch.Tensor:
        """The reduced rows after ``all_reduce`` (identical on every rank)."""
        return self._sums[slot][:rows]

    def all_reduce(self, slot: int, rows: int) -> torch.Tensor:
        """Launches on the current stream; returns ``result(slot, rows)``."""
        rc = self.lib.df_allreduce_bf16(ctypes.byref(self._plain_views[slot]), self.world, self.max_rows, self.hidden,
                                        rows, self.n_ctas, self._status_ptr,
                                        torch.cuda.current_stream(self.device).cuda_stream)
        if rc != 0:
            _check(rc, "df_allreduce_bf16")
        self.launches += 1
        self.bytes_reduced += rows * self.hidden * 2
        return self._sums[slot][:rows]

    def all_reduce_add_rmsnorm(self, slot: int, rows: int, residual: torch.Tensor | None, weight: torch.Tensor,
                               out: torch.Tensor, residual_out: torch.Tensor, eps: float = 1e-5,
                               fused: bool = True) -> torch.Tensor:
        """``out = rmsnorm(allreduce(partial) + residual) * weight``; ``residual_out`` gets the sum.
        ``fused=True``: one launch, the normalisation runs on the reduction's few CTAs.
        ``fused=False``: the reduction, then the normalisation as a second launch over all SMs
        (same bits; faster when the message is large)."""
        if not fused:
            y = self.all_reduce(slot, rows)
            add_rmsnorm(y, residual, weight, out, residual_out, eps)
            return out
        view = self._view(self.rank, self.regions[slot], residual, residual_out, out)
        st = ops.status_block(self.device)
        _check(self.lib.df_allreduce_add_rmsnorm_bf16(ctypes.byref(view), self.world, self.max_rows, self.hidden, rows,
                                                      weight.data_ptr(), eps, self.n_ctas, st.data_ptr(),
                                                      torch.cuda.current_stream(self.device).cuda_stream),
               "df_allreduce_add_rmsnorm_bf16")
        self.launches += 1
        self.bytes_reduced += rows * self.hidden * 2
        return out

    def all_reduce_add_rmsnorm_sharded(self, slot: int, rows: int, residual: torch.Tensor, weight: torch.Tensor,
                                       eps: float = 1e-5, first: bool = False) -> torch.Tensor:
        """Reduce-scatter, residual add + RMSNorm on this rank's row slice, all-gather. ``residual``
        is ``[rows, hidden]`` on every rank but only the rows ``slice_bounds(rows)`` are read and
        updated here (the residual stream is sharded by rows); ``first=True`` treats it as zeros.
        Returns the normalised rows of all ranks (``result(slot, rows)``)."""
        view = self._view(self.rank, self.regions[slot], None if first else residual, residual, None)
        rc = self.lib.df_allreduce_add_rmsnorm_sharded_bf16(ctypes.byref(view), self.world, self.max_rows, self.hidden,
                                                            rows, weight.data_ptr(), eps, self.n_ctas, self._status_ptr,
                                                            torch.cuda.current_stream(self.device).cuda_stream)
        if rc != 0:
            _check(rc, "df_allreduce_add_rmsnorm_sharded_bf16")
        self.launches += 1
        self.bytes_reduced += rows * self.hidden * 2
        return self._sums[slot][:rows]

    def _half(self, fn_name: str, slot: int, rows: int) -> None:
        rc = getattr(self.lib, fn_name)(ctypes.byref(self._plain_views[slot]), self.world, self.max_rows, self.hidden,
                                        rows, self.n_ctas, self._status_ptr,
                                        torch.cuda.current_stream(self.device).cuda_stream)
        if rc != 0:
            _check(rc, fn_name)
        self.launches += 1

    def all_gather(self, slot: int, rows: int) -> torch.Tensor:
        """Every rank has written ITS row slice (``slice_bounds(rows)``) into ``partial(slot, rows)``;
        afterwards ``result(slot, rows)`` holds all rows on every rank. Current stream."""
        self._half("df_all_gather_bf16", slot, rows)
        return self._sums[slot][:rows]

    def reduce_scatter(self, slot: int, rows: int) -> torch.Tensor:
        """Every rank's ``partial(slot, rows)`` holds ``rows`` rows of contributions; afterwards
        this rank's slice of ``result(slot, rows)`` holds their sum over ranks (fp32 in rank order,
        rounded once). Returns that slice. Current stream."""
        self._half("df_reduce_scatter_bf16", slot, rows)
        lo, hi = self.slice_bounds(rows)
        return self._sums[slot][lo:hi]

    def slice_bounds(self, rows: int) -> tuple[int, int]:
        """Rows of a ``rows``-row message that this rank owns."""
        return rows * self.rank // self.world, rows * (self.rank + 1) // self.world

    def summary(self) -> dict:
        return {"kind": "peer-memory two-shot all-reduce (hand-written, no NCCL on the data path)",
                "n_ctas": self.n_ctas, "launches": self.launches, "payload_bytes": self.bytes_reduced}

    def close(self) -> None:
        torch.cuda.synchronize(self.device)
        self._partials, self._sums = [], []
        with torch.cuda.device(self.device):
            for ptr in self._opened:
                self.lib.df_comm_region_close(ptr)
            for ptr in self.local:
                self.lib.df_comm_region_free(ptr)
        self._opened, self.local = [], []


class MulticastComm(PeerComm):
    """``PeerComm`` whose regions are bound to an NVLink multicast object, so that the all-reduce
    and the sharded-residual fused form reduce inside the switch (``df_allreduce_multicast_bf16``).
    The regions are one ``torch.distributed._symmetric_memory`` allocation per rank, which also
    provides every peer's mapping (the flag barriers and the replicated-residual form keep using
    those). Raises if the devices offer no multicast mapping. All ranks must leave together: a
    rank that dies while its memory is bound to the multicast object can fault its peers' GPUs."""

    def _map_regions(self, group: Any) -> None:
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm

        pg = group if group is not None else dist.group.WORLD
        stride = (self.region_bytes + 4095) // 4096 * 4096
        self._symm = symm.empty(stride * self.slots, dtype=torch.uint8, device=self.device)
        self._symm.zero_()                    # flag words and sequence numbers start at zero
        torch.cuda.synchronize(self.device)
        self._handle = symm.rendezvous(self._symm, pg.group_name)
        mc = int(getattr(self._handle, "multicast_ptr", 0) or 0)
        if mc == 0:
            raise RuntimeError("these devices expose no NVLink multicast mapping; use PeerComm")
        ptrs = [int(p) for p in self._handle.buffer_ptrs]
        self.local = [ptrs[self.rank] + s * stride for s in range(self.slots)]
        self.regions = [[ptrs[r] + s * stride for r in range(self.world)] for s in range(self.slots)]
        self.multicast = [mc + s * stride for s in range(self.slots)]

    def all_reduce(self, slot: int, rows: int) -> torch.Tensor:
        rc = self.lib.df_allreduce_multicast_bf16(ctypes.byref(self._plain_views[slot]), self.multicast[slot], self.world,
                                                  self.max_rows, self.hidden, rows, 0, None, 0.0, self.n_ctas,
                                                  self._status_ptr, torch.cuda.current_stream(self.device).cuda_stream)
        if rc != 0:
            _check(rc, "df_allreduce_multicast_bf16")
        self.launches += 1
        self.bytes_reduced += rows * self.hidden * 2
        return self._sums[slot][:rows]

    def all_reduce_add_rmsnorm_sharded(self, slot: int, rows: int, residual: torch.Tensor, weight: torch.Tensor,
                                       eps: float = 1e-5, first: bool = False) -> torch.Tensor:
        view = self._view(self.rank, self.regions[slot], None if first else residual, residual, None)
        rc = self.lib.df_allreduce_multicast_bf16(ctypes.byref(view), self.multicast[slot], self.world, self.max_rows,
                                                  self.hidden, rows, 1, weight.data_ptr(), eps, self.n_ctas,
                                                  self._status_ptr, torch.cuda.current_stream(self.device).cuda_stream)
        if rc != 0:
            _check(rc, "df_allreduce_multicast_bf16")
        self.launches += 1
        self.bytes_reduced += rows * self.hidden * 2
        return self._sums[slot][:rows]

    def summary(self) -> dict:
        return {"kind": "in-switch all-reduce over an NVLink multicast mapping (hand-written multimem kernel, "
                        "no NCCL on the data path)",
                "n_ctas": self.n_ctas, "launches": self.launches, "payload_bytes": self.bytes_reduced}

    def close(self) -> None:
        """Collective: every rank must call it, with none of its kernels in flight; the ranks meet
        at a barrier before any of them releases its binding to the multicast object."""
        import torch.distributed as dist

        torch.cuda.synchronize(self.device)
        if self.world > 1 and dist.is_initialized():
            dist.barrier()
        self._partials, self._sums = [], []
        self.local, self.regions, self.multicast = [], [], []
        self._handle = None
        self._symm = None


def add_rmsnorm(y: torch.Tensor, residual: torch.Tensor | None, weight: torch.Tensor, out: torch.Tensor,
                residual_out: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    """``r' = y + residual; out = rmsnorm(r') * weight; residual_out = r'`` on the current stream."""
    T, H = y.shape
    for t in (y, out, residual_out) + ((residual,) if residual is not None else ()):
        if t.dtype != torch.bfloat16 or not t.is_contiguous() or tuple(t.shape) != (T, H):
            raise ValueError("add_rmsnorm takes contiguous bf16 [T, H] tensors")
    rc = _native.load().df_add_rmsnorm_bf16(y.data_ptr(), residual.data_ptr() if residual is not None else None,
                                            residual_out.data_ptr(), out.data_ptr(), weight.data_ptr(), eps, T, H,
                                            torch.cuda.current_stream(y.device).cuda_stream)
    _check(rc, "df_add_rmsnorm_bf16")
    return out


class EmulatedComm(_Regions):
    """All ranks on one GPU, one cooperative launch (grid.y = rank)."""

    def __init__(self, world: int, max_rows: int, hidden: int, n_ctas: int = 8, device: torch.device | None = None) -> None:
        device = device or torch.device("cuda", torch.cuda.current_device())
        super().__init__(world, max_rows, hidden, 1, n_ctas, device)
        self.buffers = [torch.zeros(self.region_bytes, dtype=torch.uint8, device=device) for _ in range(world)]
        self.ptrs = [b.data_ptr() for b in self.buffers]

    def partial(self, rank: int, rows: int) -> torch.Tensor:
        b = self.buffers[rank][self.partial_off:self.partial_off + self.max_rows * self.hidden * 2]
        return b.view(torch.bfloat16).view(self.max_rows, self.hidden)[:rows]

    def result(self, rank: int, rows: int) -> torch.Tensor:
        b = self.buffers[rank][self.sum_off:self.sum_off + self.max_rows * self.hidden * 2]
        return b.view(torch.bfloat16).view(self.max_rows, self.hidden)[:rows]

    def run(self, rows: int, *, weight: torch.Tensor | None = None, residual_in: list | None = None,
            residual_out: list | None = None, out: list | None = None, eps: float = 1e-5,
            sharded: bool = False) -> None:
        fuse = weight is not None
        views = (df_comm_rank_t * self.world)()
        for r in range(self.world):
            v = self._view(r, self.ptrs, residual_in[r] if (fuse and residual_in) else None,
                           residual_out[r] if fuse else None, out[r] if (fuse and not sharded) else None)
            views[r] = v
        st = ops.status_block(self.device)
        _check(self.lib.df_allreduce_emulated_bf16(views, self.world, self.max_rows, self.hidden, rows,
                                                   weight.data_ptr() if fuse else None, eps,
                                                   (2 if sharded else 1) if fuse else 0,
                                                   self.n_ctas, st.data_ptr(),
                                                   torch.cuda.current_stream(self.device).cuda_stream),
               "df_allreduce_emulated_bf16")
