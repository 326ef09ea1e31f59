"""The launch form of the split-K cluster GEMM (at most 128 rows), asked from the library's own planner
(``df_small_gemm_plan``: host arithmetic, no GPU): invariants over many shapes, and the forms of the
decode-step projections the time model was fitted on."""
import ctypes

import numpy as np
import pytest

SMEM_CAP = 227 * 1024


def plan(lib, M, N, K, gate_up, sms=148):
    box, splits, stages, tiles = (ctypes.c_int() for _ in range(4))
    smem = ctypes.c_size_t()
    rc = lib.df_small_gemm_plan(M, N, K, int(gate_up), sms, ctypes.byref(box), ctypes.byref(splits), ctypes.byref(stages),
                                ctypes.byref(tiles), ctypes.byref(smem))
    assert rc == 0, lib.df_last_error()
    return box.value, splits.value, stages.value, tiles.value, smem.value


def test_plans_respect_the_hardware_limits(native_lib):
    rng = np.random.default_rng(7)
    for _ in range(400):
        M = int(rng.integers(1, 129))
        N = int(rng.integers(1, 2500)) * 8
        K = int(rng.integers(1, 2000)) * 8
        gate_up = bool(rng.integers(0, 2))
        sms = int(rng.choice([148, 140, 132, 64, 20, 3]))
        box, splits, stages, tiles, smem = plan(native_lib, M, N, K, gate_up, sms)
        num_kb = -(-K // 64)
        assert box in (32, 64, 128) and splits in (1, 2, 4, 8)
        assert splits <= num_kb                                    # every k range has a k-block
        assert tiles == -(-N // (box if gate_up else 2 * box))     # the tiles cover the output columns
        assert smem <= SMEM_CAP
        assert 1 <= stages <= 16 and stages <= -(-num_kb // splits)
        if splits > 1:
            assert tiles * splits <= sms                           # clusters only inside one wave
            a_bytes = -(-M // 8) * 1024
            ring = stages * (a_bytes + 2 * box * 128)
            recv = splits * -(-M // splits) * 2 * box * 4
            assert max(ring, M * 2 * box * 4) + recv + 1536 <= SMEM_CAP   # ring (or the staged tile) + receive area


@pytest.mark.parametrize("name,N,K,gate_up,want", [
    ("qkv", 768, 4096, False, (32, 8)), ("output", 4096, 512, False, (32, 1)), ("down", 4096, 1792, False, (64, 4)),
    ("gate_up", 1792, 4096, True, (64, 4)), ("vocabulary shard", 16032, 4096, False, (64, 1))])
def test_decode_projections_take_the_measured_forms(native_lib, name, N, K, gate_up, want):
    """128 rows, one rank's share of 8, 140 SMs for the GEMMs: the forms that were fastest when every
    (box, cluster) pair was timed on a B200."""
    box, splits, _stages, tiles, _smem = plan(native_lib, 128, N, K, gate_up, 140)
    assert (box, splits) == want, (name, box, splits, tiles)


def test_bad_arguments_are_refused(native_lib):
    assert native_lib.df_small_gemm_plan(129, 256, 256, 0, 148, None, None, None, None, None) != 0
    assert native_lib.df_small_gemm_plan(16, 256, 256, 0, 0, None, None, None, None, None) != 0
    assert native_lib.df_small_gemm_plan(16, 256, 256, 0, 148, None, None, None, None, None) == 0
