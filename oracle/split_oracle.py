"""Integer side of the hot path: how a batch is cut into nano-batches, how inputs
are sliced and outputs merged, and in what order a round-robin policy dispatches.

Plain Python / numpy restatement; each function cites the reference lines it follows.
"""
from __future__ import annotations

import itertools

import numpy as np


def pack_tokens(num_tokens: int, capture_sizes: list[int]) -> tuple[int, bool]:
    """``dynaflow/utils.py:1-5``."""
    if num_tokens <= max(capture_sizes):
        return min(s for s in capture_sizes if s >= num_tokens), True
    return num_tokens, False


def nanoflow_split(num_tokens: list[int], min_nano_split_tokens: int, capture_sizes: list[int],
                   use_cudagraph: bool) -> dict:
    """Balanced two-way split at a request boundary
    (``examples/ae/scheduler/vllm/nanoflow.py:98-151``, identical in ``hf/nanoflow.py:66-120``).
    Returns the fields of a SplitConfig as a dict."""
    batch_size = len(num_tokens)
    ps = [0] + list(itertools.accumulate(num_tokens))
    total = ps[-1]
    # first index minimising |left - right| (ties resolve to the smallest index, as min() does)
    mid = min(range(len(ps)), key=lambda i: abs(ps[i] - (total - ps[i])))
    left, right = ps[mid], total - ps[mid]
    if left < min_nano_split_tokens or right < min_nano_split_tokens:
        padded = total
        if use_cudagraph:
            padded, use_cudagraph = pack_tokens(total, capture_sizes)
        return dict(num_nano_batches=1, batch_sizes=[batch_size], batch_indices=[0, batch_size],
                    num_tokens=[total], num_tokens_padded=[padded], split_indices=[0, total],
                    is_dryrun=False, use_cudagraph=use_cudagraph, allow_fallback=True)
    padded = [left, right]
    if use_cudagraph:
        packed = [pack_tokens(n, capture_sizes) for n in padded]
        if all(ok for _, ok in packed):
            padded = [p for p, _ in packed]
        else:
            use_cudagraph = False
    return dict(num_nano_batches=2, batch_sizes=[mid, batch_size - mid], batch_indices=[0, mid, batch_size],
                num_tokens=[left, right], num_tokens_padded=padded, split_indices=[0, left, total],
                is_dryrun=False, use_cudagraph=use_cudagraph, allow_fallback=True)


def equal_split(batch_size: int, num_nano_batches: int, min_nano_split_tokens: int, use_cudagraph: bool) -> dict:
    """n-way equal split of the row axis, remainder to the last nano-batch
    (``examples/ae/scheduler/megatron/nanoflow.py:43-76``)."""
    n = num_nano_batches
    chunk = batch_size // n
    if chunk < min_nano_split_tokens:
        n = max(1, batch_size // min_nano_split_tokens)
        chunk = batch_size // n if n > 1 else batch_size
    if n <= 1:
        return dict(num_nano_batches=1, batch_sizes=[batch_size], batch_indices=[0, batch_size],
                    num_tokens=[batch_size], num_tokens_padded=[batch_size], split_indices=[0, batch_size],
                    is_dryrun=False, use_cudagraph=use_cudagraph, allow_fallback=True)
    sizes = [chunk] * n
    sizes[-1] = batch_size - chunk * (n - 1)
    idx = [chunk * i for i in range(n)] + [batch_size]
    return dict(num_nano_batches=n, batch_sizes=sizes, batch_indices=idx, num_tokens=list(sizes),
                num_tokens_padded=list(sizes), split_indices=list(idx), is_dryrun=False,
                use_cudagraph=use_cudagraph, allow_fallback=True)


def slice_rows(array: np.ndarray, split_indices: list[int], batch_idx: int) -> np.ndarray:
    """Rows a nano-batch receives from a dynamic input (``dynaflow/runtime/engine.py:441-470``)."""
    return array[split_indices[batch_idx]:split_indices[batch_idx + 1]]


def merge_rows(parts: list[np.ndarray]) -> np.ndarray:
    """Concatenation of nano-batch outputs along dim 0 (``dynaflow/manager.py:241-246``)."""
    return np.concatenate(parts, axis=0)


def round_robin_trace(ops_per_batch: list[list[str]]) -> list[tuple[str, int]]:
    """Dispatch order of the NanoFlow policy: rounds in which one operator is popped
    from every live nano-batch and the popped ones are executed in nano-batch order
    (``examples/ae/scheduler/hf/nanoflow.py:123-146``). ``ops_per_batch[b]`` is the
    program-order list of subgraph names of nano-batch ``b``.

    The policy removes finished nano-batches from the list it is iterating over, so
    the entry after a removed one is skipped for that round; this restatement keeps
    that behaviour."""
    cursors = [0] * len(ops_per_batch)
    live = list(range(len(ops_per_batch)))
    trace: list[tuple[str, int]] = []
    while live:
        popped = []
        for b in live:  # iterating while removing, as the policy does
            if cursors[b] >= len(ops_per_batch[b]):
                live.remove(b)
                continue
            popped.append((ops_per_batch[b][cursors[b]], b))
            cursors[b] += 1
        trace.extend(popped)
    return trace


def skewed_trace(ops_per_batch: list[list[str]]) -> list[tuple[str, int]]:
    """Dispatch order of the Megatron NanoFlow policy: nano-batch 0 runs one operator
    ahead, then every live nano-batch pops and executes one operator per round
    (``examples/ae/scheduler/megatron/nanoflow.py:79-102``)."""
    n = len(ops_per_batch)
    cursors = [0] * n
    live = list(range(n))
    trace: list[tuple[str, int]] = []
    if n >= 2:
        if ops_per_batch[0]:
            trace.append((ops_per_batch[0][0], 0))
            cursors[0] = 1
        else:
            live.remove(0)
    while live:
        for b in list(live):
            if cursors[b] >= len(ops_per_batch[b]):
                live.remove(b)
                continue
            trace.append((ops_per_batch[b][cursors[b]], b))
            cursors[b] += 1
    return trace


DBO_WARM_UP = [("attention", 0)]
DBO_SEQUENCE = [("attention", 1), ("dispatch", 0), ("expert", 0), ("dispatch", 1), ("expert", 1), ("combine", 0),
                ("attention", 0), ("combine", 1)]


def dbo_trace(ops_per_batch: list[list[tuple[str, list[str]]]]) -> list[tuple[str, int, str]]:
    """Dispatch order of the dual-batch-overlap policy for MoE layers
    (``examples/ae/scheduler/vllm/dbo.py:154-220``). ``ops_per_batch[b]`` is the program-order
    list of ``(subgraph name, tags)`` of nano-batch ``b``. Returns ``(name, batch, stream)`` with
    stream ``"comm"`` for ``network``-tagged operators and ``"comp"`` otherwise (``"default"``,
    i.e. whatever stream is current, on the one-nano-batch path).

    One nano-batch: program order on the compute stream. Two: after nano-batch 0's first
    attention, the operators tagged attention / dispatch / expert / combine are executed in the
    fixed cyclic order attn1, disp0, exp0, disp1, exp1, comb0, attn0, comb1; an operator that
    arrives before its turn is held back (one per nano-batch) while the other nano-batch
    proceeds; operators without one of those tags run at once. A finished nano-batch advances
    the cycle by one position."""
    n = len(ops_per_batch)
    cursors = [0] * n
    trace: list[tuple[str, int, str]] = []

    def pop(b):
        if cursors[b] >= len(ops_per_batch[b]):
            return None
        op = ops_per_batch[b][cursors[b]]
        cursors[b] += 1
        return op

    def run(op, b):
        name, tags = op
        trace.append((name, b, "comm" if "network" in tags else "comp"))

    if n == 1:
        while (op := pop(0)) is not None:
            trace.append((op[0], 0, "default"))   # the single-batch path keeps the current stream
        return trace
    keys = {k for k, _ in DBO_SEQUENCE}
    live = list(range(n))
    cur, seq, idx = live[0], DBO_WARM_UP, -len(DBO_WARM_UP)
    held: list = [None] * n
    while live:
        assert cur in live
        if held[cur] is None:
            op = pop(cur)
            if op is None:
                live.remove(cur)
                cur ^= 1
                idx += 1
                continue
            if not keys.intersection(op[1]):
                trace.append((op[0], cur, "comp"))
                continue
            if seq[idx][1] != cur:
                held[cur] = op
                cur ^= 1
                continue
        else:
            op, held[cur] = held[cur], None
        assert seq[idx][0] in op[1], (seq[idx], op)
        idx += 1
        if idx > 0:
            idx %= len(DBO_SEQUENCE)
        elif idx == 0:
            seq = DBO_SEQUENCE
        run(op, cur)
    return trace
