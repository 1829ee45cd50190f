"""Host-side helpers: size/shape parsing, statistics, CSV layout, roofline arithmetic, clocks."""

import pytest

from tileccl_b200.bench import _common as C
from tileccl_b200.utils import clocks, csvio, roofline, stats


def test_parse_size_and_shape():
    assert C.parse_size("4096") == 4096 and C.parse_size("4K") == 4096 and C.parse_size("1.5M") == 1572864 and C.parse_size("1G") == 1 << 30
    assert C.parse_shape("8192") == (8192, 8192, 8192)
    assert C.parse_shape("32768x8192x1024") == (32768, 8192, 1024)
    with pytest.raises(Exception):
        C.parse_shape("1x2")
    assert C.split_csv("a, b,,c") == ["a", "b", "c"]


def test_stats_order_statistics():
    s = stats.make_stats([5, 1, 4, 2, 3])
    assert (s.n, s.min, s.max, s.p50, s.mean) == (5, 1, 5, 3, 3)
    v = list(range(100))
    s = stats.make_stats(v)
    assert s.p95 == 95 and s.p99 == 99
    assert stats.iters_for_ms(100.0, 10.0) == 100 and stats.iters_for_ms(0, 10) == 5


def test_csv_headers_match_reference_layout():
    assert csvio.EXP3_FUSED_COLUMNS[:27] == ("m,n,k,world,rank,base_us,base_p95,ctrl_us,ctrl_p95,fused_us,fused_p95,struct_sd,comm_sd,total_sd,"
                                             "pull_gbps,max_rel_diff,base_p50,ctrl_p50,fused_p50,base_min,ctrl_min,fused_min,comm_sd_p50,"
                                             "comm_sd_skew,comm_abs_us,order,iters").split(",")
    assert csvio.EXP3_FUSED_COLUMNS[27:] == csvio.EXTRA_COLUMNS + ["knobs"]   # appended only, after the reference's 27
    assert csvio.SIGNAL_FANIN_COLUMNS == "mode,fanin,bytes,min_us,p50_us,p95_us,p99_us,verify".split(",")
    assert csvio.EXP2_COLUMNS[:4] == ["m", "n", "k", "world"] and "seg_eff" in csvio.EXP2_COLUMNS


def test_csv_append_and_multi_header_read(tmp_path):
    p = str(tmp_path / "x.csv")
    for run in range(2):
        w = csvio.CsvAppender(p, ["m", "n", "order", "v"])
        w.row(m=1 + run, n=2, order="a,b", v=3.14159)
        w.close()
    rows = csvio.read_rows(p)
    assert len(rows) == 2 and rows[1]["m"] == "2" and rows[0]["order"] == "a|b" and rows[0]["v"] == "3.1416"
    assert open(p).read().count("m,n,order,v") == 2


def test_roofline_headline_shapes():
    r = roofline.gemm_rs_roofline_us(32768, 8192, 1024, 8)
    assert r["link_us"] == pytest.approx(7 / 8 * 32768 * 8192 * 2 / 770e9 * 1e6)
    assert r["roofline_us"] == max(r["link_us"], r["compute_us"])
    a = roofline.ag_gemm_roofline_us(32768, 3584, 8192, 8)
    assert a["roofline_us"] == a["compute_us"] > a["link_us"]
    assert roofline.gemm_rs_roofline_us(1024, 1024, 1024, 1)["link_us"] == 0


def test_roofline_fraction_follows_the_clock_the_run_held():
    r = roofline.ag_gemm_roofline_us(32768, 14336, 8192, 2)
    assert r["roofline_burst_us"] <= r["roofline_us"] and r["link_file"].endswith(".json")
    fast = {"sm_mhz": 1965.0, "sm_max_mhz": 1965.0}
    slow = {"sm_mhz": 1350.0, "sm_max_mhz": 1965.0}
    assert roofline.pick_peak(fast) == "burst" and roofline.pick_peak(slow) == "sustained" and roofline.pick_peak(None) == "sustained"
    t = r["roofline_us"] * 0.99               # faster than the sustained roofline: a run that held a high clock
    f = roofline.fractions(r, t, slow)
    assert f["of"] == "burst" and f["pct"] <= 100.0 and f["pct_sustained"] > 100.0
    f2 = roofline.fractions(r, r["roofline_us"] * 1.25, slow)
    assert f2["of"] == "sustained" and f2["pct"] == pytest.approx(80.0)
    assert roofline.fractions(r, r["roofline_us"] * 1.25, fast)["of"] == "burst"
    assert roofline.fractions(r, 0.0)["pct"] is None


def test_clock_summary_flags_throttling():
    text = "\n".join([
        "0, 1965, 1965, 250.0, 0x0, Not Active, Not Active, Not Active, Not Active",
        "0, 1400, 1965, 990.0, 0x4, Not Active, Not Active, Not Active, Active",
        "0, 1380, 1965, 1001.0, 0x4, Not Active, Not Active, Not Active, Active",
        "0, 1200, 1965, 980.0, 0x8, Not Active, Active, Not Active, Not Active",
    ])
    s = clocks.summarize(clocks.parse_samples(text))
    assert s["samples"] == 4 and s["sm_max_mhz"] == 1965 and s["sm_mhz"] in (1380.0, 1400.0)
    assert "sw_power_cap" in s["reasons"] and "hw_thermal_slowdown" in s["reasons"]
    assert clocks.summarize([])["sm_mhz"] is None


def test_wave_efficiency_of_the_persistent_grid():
    w = roofline.wave_efficiency(32768, 8192, cta_group=2, sms=148)        # GEMM+RS headline shape
    assert (w["tiles"], w["groups"], w["waves"]) == (4096, 74, 56) and abs(w["efficiency"] - 4096 / (56 * 74)) < 1e-12
    assert roofline.wave_efficiency(256 * 74, 256)["efficiency"] == 1.0     # exactly one full wave
    assert roofline.wave_efficiency(128, 256, cta_group=1)["efficiency"] == 1 / 148


def test_turn_order_changes_every_variants_predecessor():
    from collections import Counter
    from tileccl_b200.bench._common import turn_order
    names = [f"v{i}" for i in range(12)]
    pred = Counter()
    for i in range(24):
        order = turn_order(names, i)
        assert sorted(order) == sorted(names)
        for a, b in zip(order, order[1:]):
            pred[(a, b)] += 1
    # no variant follows the same neighbour in more than a third of the iterations
    assert max(pred.values()) <= 8
    assert turn_order(["a", "b"], 1) == ["b", "a"] and turn_order([], 3) == []


def test_gather_tiles_of_the_ag_gemm_sweep():
    from tileccl_b200.bench.exp2_ag_gemm_granularity import gather_tiles
    assert gather_tiles(["128", "512", "2048", "4096"], 4096) == ([128, 512, 2048, 4096], [])      # 8 ranks
    assert gather_tiles(["128", "512", "2048", "4096"], 16384) == ([128, 512, 2048, 4096], [])     # 2 ranks
    assert gather_tiles(["64", "384", "8192"], 4096) == ([4096], [64, 384])                         # 8192 becomes the segment
    assert gather_tiles(["192"], 192) == ([192], [])                                                # the whole segment always runs
