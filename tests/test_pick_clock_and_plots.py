"""Clock picker against a fake NVML (nothing here touches a GPU), and the SVG figure writer."""
import os

from tileccl_b200.bench import pick_clock, plots
from tileccl_b200.utils import csvio


class FakeNvml(pick_clock.NvmlBackend):
    """A GPU that holds any clock up to 1400 MHz and sags to 1380 above it."""

    def __init__(self):
        self.locked = None
        self.calls = []

    def sm_clock(self, index):
        want = self.locked or 1965
        return want if want <= 1400 else 1380

    def max_sm_clock(self, index):
        return 1965

    def lock_clocks(self, index, mhz):
        self.calls.append(("lock", mhz))
        self.locked = mhz

    def reset_clocks(self, index):
        self.calls.append(("reset",))
        self.locked = None


def test_observe_mode_changes_nothing():
    nv = FakeNvml()
    res = pick_clock.run(nv, 0, [1965, 1400, 1305], seconds=0.25, load=lambda: None, apply=False)
    assert nv.calls == []                                     # read-only
    assert pick_clock.pick(res) == 1400                       # 1380 is within 2 % of 1400


def test_apply_mode_locks_and_always_resets():
    nv = FakeNvml()
    res = pick_clock.run(nv, 0, [1965, 1305], seconds=0.25, load=lambda: None, apply=True)
    assert nv.calls == [("lock", 1965), ("reset",), ("lock", 1305), ("reset",)]
    assert nv.locked is None
    assert pick_clock.pick(res) == 1305

    def boom():
        raise RuntimeError("load failed")
    nv2 = FakeNvml()
    try:
        pick_clock.run(nv2, 0, [1500], seconds=0.2, load=boom, apply=True)
    except RuntimeError:
        pass
    assert nv2.calls[-1] == ("reset",) and nv2.locked is None   # the lock never outlives a failure


def test_soak_stats():
    s = pick_clock.soak_stats([1300, 1305, 1310, 1000], 1305)
    assert s["hold_pct"] == 75.0 and s["min"] == 1000
    assert pick_clock.pick([s]) is None


def test_figures_from_csv(tmp_path):
    w = csvio.CsvAppender(str(tmp_path / "pk_bw.csv"), csvio.PK_BW_COLUMNS)
    for mover, scale in (("ce", 1.0), ("reg", 0.9)):
        for i, msg in enumerate((128, 4096, 1 << 20, 1 << 30)):
            w.row(figure="size", mover=mover, msg_bytes=msg, sms=148, total_bytes=1 << 30, us=10.0, gbps=scale * 100 * (i + 1), verify="ok")
        for sms in (1, 16, 148):
            w.row(figure="sms", mover=mover, msg_bytes=16384, sms=sms, total_bytes=1 << 30, us=10.0, gbps=scale * 5 * sms, verify="ok")
    w.close()
    w = csvio.CsvAppender(str(tmp_path / "interference.csv"), csvio.INTERFERENCE_COLUMNS)
    for probe in ("ffma", "hbm"):
        for comm in ("ce", "reg"):
            w.row(mode="matrix", probe=probe, comm=comm, probe_dev="src", S_m=1.1, S_c=1.02)
    w.close()
    w = csvio.CsvAppender(str(tmp_path / "nvls_bw.csv"), "mover,bytes,world,us,gbps,verify".split(","))
    for mover in ("p2p_st", "mc_bcast"):
        for b in (65536, 1 << 24):
            w.row(mover=mover, bytes=b, world=8, us=10.0, gbps=b / 1e5, verify="-")
    w.row(mover="barrier_mc", bytes=0, world=8, us=14.0, gbps=0.0, verify="-")      # latency rows stay out of the figure
    w.close()
    w = csvio.CsvAppender(str(tmp_path / "exp3_tuning.csv"), csvio.EXP3_FUSED_COLUMNS)
    for knobs, us in (("cta_group=2|transport=p2p|rs_chunks=0|group_m=0|num_ctas=0|st256=0|ablate=0", 800.0),
                      ("cta_group=2|transport=p2p|rs_chunks=0|group_m=0|num_ctas=0|st256=1|ablate=0", 700.0)):
        w.row(m=32768, n=8192, k=1024, world=8, rank=0, max_over_ranks_us=us, nccl_cublas_us=1200.0, roofline_us=610.0, knobs=knobs)
    w.close()
    made = plots.make_all(str(tmp_path))
    names = {os.path.basename(p) for p in made}
    assert {"pk_bw_vs_size.svg", "pk_bw_vs_sms.svg", "interference_S_c.svg", "interference_S_m.svg", "nvls_bw.svg", "gemm_rs_tuning.svg"} <= names
    tune = open(os.path.join(str(tmp_path), "figs", "gemm_rs_tuning.svg")).read()
    assert "st256=1" in tune and "default" in tune and "barrier_mc" not in open(os.path.join(str(tmp_path), "figs", "nvls_bw.svg")).read()
    svg = open(made[0]).read()
    assert svg.startswith("<svg") and "polyline" in svg and "reg" in svg
