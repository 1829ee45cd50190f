"""The transport selector reproduces the decision table of the measured probes."""
import json

import pytest

from tileccl_b200.utils import selector as S


def test_large_independent_copy_goes_to_the_copy_engine():
    p = S.Platform()
    r = S.choose(p, 128 << 20, compute_us=400.0, bound="tensor")
    assert r["best"] == "ce"                      # no SMs taken from an SM-bound kernel
    assert r["table"]["reg"]["compute_us"] > r["table"]["ce"]["compute_us"]


def test_many_small_messages_go_to_an_sm_mover():
    p = S.Platform()
    r = S.choose(p, 64 << 20, n_msgs=(64 << 20) // 4096)     # 4 KB messages: the per-copy cost kills the copy engine
    assert r["best"] in ("reg", "bulk")
    assert r["table"]["ce"]["comm_us"] > 10 * r["table"]["reg"]["comm_us"]


def test_no_spare_sms_leaves_only_the_copy_engine_or_fusion():
    p = S.Platform()
    assert set(S.choose(p, 1 << 20, sms_spare=0)["table"]) == {"ce"}
    assert set(S.choose(p, 1 << 20, sms_spare=0, fused_possible=True)["table"]) == {"ce", "fused_st", "fused_pull"}


def test_fused_wins_when_the_producer_can_carry_it():
    p = S.Platform()
    # one rank's GEMM+RS at 8 GPUs: 470 MB leave the GPU while a 370 us GEMM runs
    r = S.choose(p, 470 << 20, compute_us=370.0, bound="tensor", fused_possible=True)
    assert r["best"].startswith("fused") or r["best"] == "ce"
    assert r["table"]["fused_st"]["compute_us"] == pytest.approx(370.0)


def test_l2_bound_kernels_avoid_the_bulk_mover():
    p = S.Platform()
    r = S.choose(p, 64 << 20, compute_us=1000.0, bound="l2")
    assert r["best"] != "bulk" and r["table"]["bulk"]["compute_us"] > 1900


def test_transfer_model_pieces():
    p = S.Platform()
    assert S.transfer_us(p, "reg", 0) == 0.0
    assert S.transfer_us(p, "reg", 1 << 20, sms=4) > S.transfer_us(p, "reg", 1 << 20, sms=16)
    assert S.transfer_us(p, "reg", 1 << 20, n_msgs=8192) > S.transfer_us(p, "reg", 1 << 20)      # 128-byte messages
    assert S.pipeline_us(3.0, 5.0, 4.0) == 5.0
    with pytest.raises(ValueError):
        S.transfer_us(p, "carrier_pigeon", 1)
    with pytest.raises(ValueError):
        S.compute_slowdown(p, "ce", "tea")


def test_platform_file_round_trip(tmp_path):
    f = tmp_path / "p.json"
    S.Platform(name="x", ce_gbps=100.0).to_json(str(f))
    q = S.Platform.from_json(str(f))
    assert q.name == "x" and q.ce_gbps == 100.0 and q.s_c["bulk"]["l2"] == 1.97
    f.write_text(json.dumps({"warp_drive": 1}))
    with pytest.raises(ValueError):
        S.Platform.from_json(str(f))


def test_shipped_platform_files_reproduce_the_reference_table():
    """The parameter files load, and the selector gives the rows of the reference's decision table for its two
    machines (tests/ANALYSIS.md:118-128): L2-sensitive compute on H20 -> copy engine; an HBM-heavy phase on the
    PCIe pair where the transfer's latency matters -> an SM mover (S_m 1.01 against 1.41 for the copy engine)."""
    b200 = S.load_platform("b200_nvswitch")
    assert b200.ce_gbps == S.Platform().ce_gbps and "measured" in b200.notes
    h20 = S.load_platform("h20_nvlink_reference")
    r = S.choose(h20, 64 << 20, compute_us=2000.0, bound="l2")
    assert r["best"] == "ce" and r["table"]["reg"]["compute_us"] > 1.8 * 2000
    pcie = S.load_platform("rtx_pcie5_reference")
    r = S.choose(pcie, 64 << 20, compute_us=100.0, bound="hbm")          # transfer-bound: its own slow-down decides
    assert r["best"] in ("reg", "bulk") and r["table"]["ce"]["comm_us"] > 1.2 * r["table"]["reg"]["comm_us"]
