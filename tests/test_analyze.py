"""Verdict reducers of the analysis script, on synthetic bundles."""

from tileccl_b200.bench import analyze, run_all
from tileccl_b200.utils import csvio


def _fused_row(w, **kv):
    base = dict(m=8192, n=8192, k=1024, world=2, rank=0, base_us=100, base_p95=101, ctrl_us=102, ctrl_p95=103, fused_us=110, fused_p95=112,
                base_p50=100, ctrl_p50=102, fused_p50=110, order="base|ctrl|fused", iters=10, nccl_cublas_us=150, roofline_us=90)
    base.update(kv)
    w.row(**base)


def test_msweep_plateau_and_shift(tmp_path):
    w = csvio.CsvAppender(str(tmp_path / "exp3_fused_msweep.csv"), csvio.EXP3_FUSED_COLUMNS)
    for m in (4096, 8192, 16384, 32768):
        tiles = (m // 128) * 32
        for rank in (0, 1):
            _fused_row(w, m=m, rank=rank, base_us=m / 10, ctrl_us=m / 10 * 1.02, fused_us=m / 10 * 1.02 + tiles * 0.08,
                       base_p50=m / 10, ctrl_p50=m / 10 * 1.02, fused_p50=m / 10 * 1.02 + tiles * 0.08)
    w.close()
    txt = analyze.report(str(tmp_path))
    assert "PLATEAU" in txt and "NO PLATEAU" not in txt
    assert "SHIFT" in txt and "80.0" in txt          # 0.08 us per tile = 80 ns


def test_tail_verdict_and_tail_shape(tmp_path):
    w = csvio.CsvAppender(str(tmp_path / "exp3_fused_msweep.csv"), csvio.EXP3_FUSED_COLUMNS)
    _fused_row(w, fused_us=130, fused_p50=104)        # the mean is lifted by outliers
    _fused_row(w, rank=1, fused_us=130, fused_p50=104)
    w.close()
    d = csvio.CsvAppender(str(tmp_path / "iters_m8192.rank0.csv"), csvio.EXP3_ITER_COLUMNS)
    for i in range(40):
        d.row(m=8192, n=8192, k=1024, world=2, rank=0, variant="fused", iter=i, us=300.0 if i in (7, 23) else 100.0)
    d.close()
    txt = analyze.report(str(tmp_path))
    assert "TAIL" in txt and "ISOLATED outliers" in txt


def test_tiles_or_duration_and_order(tmp_path):
    w = csvio.CsvAppender(str(tmp_path / "exp3_fused_ksweep.csv"), csvio.EXP3_FUSED_COLUMNS)
    for k, ctrl in ((512, 50), (2048, 200), (8192, 800)):
        _fused_row(w, k=k, ctrl_us=ctrl, fused_us=ctrl + 40, world=1)
    w.close()
    w = csvio.CsvAppender(str(tmp_path / "exp3_order.csv"), csvio.EXP3_FUSED_COLUMNS)
    _fused_row(w, order="base|ctrl|fused", world=1)
    _fused_row(w, order="fused|ctrl|base", world=1, ctrl_us=102.5)
    w.close()
    txt = analyze.report(str(tmp_path))
    assert "TILES" in txt and "NO BIAS" in txt


def test_l2_verdicts(tmp_path):
    def write(tag, local, peer):
        w = csvio.CsvAppender(str(tmp_path / f"{tag}_bw.csv"), csvio.PEER_L2_BW_COLUMNS)
        for frac, g in local:
            w.row(build="cg", target="local", bytes=int(frac * 1e8), frac_l2=frac, gbps=g)
        for frac, g in peer:
            w.row(build="cg", target="peer", bytes=int(frac * 1e8), frac_l2=frac, gbps=g)
        w.close()
    fr = (0.0625, 0.125, 0.25, 1.0, 2.0, 4.0)
    write("probe_cg", [(f, 15000 if f < 1 else 6500) for f in fr], [(f, 760) for f in fr])
    txt = analyze.report(str(tmp_path))
    assert "NOT CACHED" in txt
    write("probe_ca", [(f, 6500) for f in fr], [(f, 760) for f in fr])
    assert "INCONCLUSIVE" in analyze.report(str(tmp_path))


def test_manifest_resume_and_plan(tmp_path):
    (tmp_path / "manifest.txt").write_text("a rc=0 seconds=1.0\nb rc=124 seconds=9.0\nc rc=0 seconds=2\nc rc=1 seconds=2\n")
    assert run_all.done_steps(tmp_path) == {"a"}
    names = [s[0] for s in run_all.plan(8, True, tmp_path)]
    for want in ("exp3_fused_m32768", "exp2_ag_gemm", "exp1_ce_interference", "pk_bw_sweep", "signal_fanin", "sync_cost", "l2_probe_cg",
                 "pipeline_e2e", "interference_matrix", "intra_sm_matrix", "ce_gemm_overlap", "mlp_e2e", "exp3_epilogue"):
        assert want in names
    assert len(set(names)) == len(names)
    assert "2 not ok" in analyze.report(str(tmp_path))


def test_tuning_summary_sorts_knob_settings(tmp_path):
    w = csvio.CsvAppender(str(tmp_path / "exp3_tuning.csv"), csvio.EXP3_FUSED_COLUMNS)
    dflt = "cta_group=2|transport=p2p|rs_chunks=0|group_m=0|num_ctas=0|st256=0|ablate=0"
    fast = "cta_group=2|transport=p2p|rs_chunks=0|group_m=0|num_ctas=0|st256=1|ablate=0"
    for rank in (0, 1):
        _fused_row(w, rank=rank, max_over_ranks_us=800.0, nccl_cublas_us=1200.0, knobs=dflt)
        _fused_row(w, rank=rank, max_over_ranks_us=700.0, nccl_cublas_us=1190.0, knobs=fast)
    w.close()
    txt = analyze.report(str(tmp_path))
    lines = [line for line in txt.splitlines() if "st256=" in line]
    assert len(lines) == 2 and "st256=1" in lines[0] and "700.0" in lines[0] and "1.143x of default" in lines[0]
    assert "1.000x of default" in lines[1] and "1.500x of NCCL+cuBLAS" in lines[1]


def test_sweep_settings_match_the_op_and_the_analyser():
    """Every setting of the sweep driver is a keyword of the op it tunes, and the analyser finds each sweep's
    default row."""
    import inspect

    from tileccl_b200.bench import tune_fused
    from tileccl_b200.ops.ag_gemm import AgGemm
    from tileccl_b200.ops.gemm_rs import GemmRs
    for settings, op in ((tune_fused.RS_SETTINGS, GemmRs), (tune_fused.AG_SETTINGS, AgGemm)):
        params = set(inspect.signature(op.__init__).parameters)
        for name, kw in settings.items():
            assert set(kw) <= params, name
    base = {"cta_group": 2, "transport": "p2p", "rs_chunks": 0, "group_m": 0, "num_ctas": 0, "st256": 0, "ablate": 0}
    assert tune_fused.knobs_string({}, base) == "cta_group=2|transport=p2p|rs_chunks=0|group_m=0|num_ctas=0|st256=0|ablate=0"
    rows = [{"max_over_ranks_us": "800", "nccl_cublas_us": "1200", "knobs": "op=gemm_rs|setting=default|" + tune_fused.knobs_string({}, base)},
            {"max_over_ranks_us": "760", "nccl_cublas_us": "1200", "knobs": "op=gemm_rs|setting=st256|" + tune_fused.knobs_string({"st256": True}, base)},
            {"max_over_ranks_us": "1400", "nccl_cublas_us": "2100", "knobs": "op=ag_gemm|setting=default|gather_rows=512"},
            {"max_over_ranks_us": "1250", "nccl_cublas_us": "2100", "knobs": "op=ag_gemm|setting=nowait|ablate=4"}]
    txt = analyze.tuning_summary(rows)
    assert "1.053x of default" in txt and txt.index("st256=1") < txt.index("st256=0")
    assert "fused ag_gemm" in txt and "1.120x of default" in txt
