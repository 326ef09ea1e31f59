"""Small host-side helpers shared by policies."""
from __future__ import annotations

import bisect


def pack_tokens(num_tokens: int, cudagraph_capture_sizes: list[int]) -> tuple[int, bool]:
    """Rounds a row count up to the nearest CUDA-graph capture size.

    Returns ``(padded, True)`` with the smallest capture size that is at least
    ``num_tokens``, or ``(num_tokens, False)`` when no capture size is large
    enough (the caller then runs without a graph). Same contract as the
    reference's ``dynaflow/utils.py:1-5``; the list need not be sorted.
    """
    ordered = sorted(cudagraph_capture_sizes)
    pos = bisect.bisect_left(ordered, num_tokens)
    if pos == len(ordered):
        return num_tokens, False
    return ordered[pos], True
