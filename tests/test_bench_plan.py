"""bench.py's choice of reduction kernel and SM split at N > 1 (pure host logic, no GPU)."""
import argparse
import os
import sys

from conftest import ROOT

sys.path.insert(0, ROOT)
import bench  # noqa: E402


def _args(**kw):
    base = dict(comm="auto", comm_ctas=0, gemm_ctas=-1, shared_sms=False)
    base.update(kw)
    return argparse.Namespace(**base)


def test_single_gpu_has_no_reduction():
    assert bench.comm_plan(_args(), 1) == {"comm": None, "comm_ctas": 0, "gemm_ctas": 0, "exclusive_sms": False}


def test_default_plan_gives_the_reduction_its_own_sms():
    # in-switch reduction: 16 CTAs, two per SM, on the 8 SMs the GEMMs leave free
    assert bench.comm_plan(_args(), 8, sms=148, multicast=True) == \
        {"comm": "multicast", "comm_ctas": 16, "gemm_ctas": 140, "exclusive_sms": True}
    # devices without multicast mappings: the peer-memory kernel on 32 CTAs = 16 SMs
    assert bench.comm_plan(_args(), 8, sms=148, multicast=False) == \
        {"comm": "peer", "comm_ctas": 32, "gemm_ctas": 132, "exclusive_sms": True}


def test_flags_override_the_plan():
    plan = bench.comm_plan(_args(comm="peer", comm_ctas=64, gemm_ctas=0, shared_sms=True), 2, sms=148)
    assert plan == {"comm": "peer", "comm_ctas": 64, "gemm_ctas": 0, "exclusive_sms": False}
    assert bench.comm_plan(_args(shared_sms=True), 4, sms=148, multicast=True)["gemm_ctas"] == 0
    assert bench.comm_plan(_args(comm_ctas=9), 4, sms=148, multicast=True)["gemm_ctas"] == 143   # 9 CTAs fill 5 SMs


def test_reference_arm_exits_quietly_on_other_ranks(monkeypatch, capsys):
    monkeypatch.setenv("RANK", "3")
    bench.run_reference_arm(argparse.Namespace(steps=1, warmup=0, gpus=4))
    assert capsys.readouterr().out == ""
