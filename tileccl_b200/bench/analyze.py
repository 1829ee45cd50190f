"""Analysis of a results bundle: tables and verdicts from the CSV files, safe on partial bundles.

    python -m tileccl_b200.bench.analyze reports/results_<stamp>

Sections (each is skipped when its files are missing):
  * fused GEMM+RS M-sweep: struct / comm / total per M, speed-up over NCCL+cuBLAS, % of roofline,
    and the communication residual per tile (comm_abs_us * 1000 / tiles): a flat residual means the
    tax is per-tile work, a falling one means a fixed cost being amortised
  * four diagnostic verdicts for the fused kernel
      1. shift or tail      does comm_sd rise on the p50s, or only on the means?
      2. tiles or duration  does the absolute comm cost follow the tile count or the kernel time (K-sweep)?
      3. run-order bias     does the struct ratio depend on which variant ran first?
      4. tail shape         isolated outliers or a drift over the run (per-iteration dumps)?
  * AG+GEMM granularity: best gather tile per mode, overlap efficiency
  * peer-L2 probe verdict: CONTROL (the local curve must show the L2 knee), then TEST (does the peer
    curve show it too?) -> CACHED / NOT CACHED / INCONCLUSIVE, with the wire ratio when counters exist
  * sanity rows of the interference matrices (controls that must read 1.00)

Reference parity: comm_comp/analyze_rerun.py (read_rows :37-59, msweep :124-175, step1..4 :177-440) and
the awk reduction of l2_peer_cache/run_all.sh:386-516.
"""
from __future__ import annotations

import glob
import os
import statistics
import sys

from ..utils import csvio

TILE_M, TILE_N = 128, 256


def _f(row: dict, key: str, default: float = 0.0) -> float:
    try:
        return float(row.get(key, default))
    except (TypeError, ValueError):
        return default


def read(path: str) -> list[dict]:
    return csvio.read_rows(path) if os.path.exists(path) else []


def by_shape(rows: list[dict]) -> dict:
    """Per (m, n, k): worst rank of every column that matters (a fused kernel ends with its slowest peer)."""
    out: dict = {}
    for r in rows:
        key = (int(_f(r, "m")), int(_f(r, "n")), int(_f(r, "k")))
        out.setdefault(key, []).append(r)
    agg = {}
    for key, rs in out.items():
        last_world = int(_f(rs[-1], "world", 1))
        rs = rs[-last_world:] if last_world > 0 else rs   # the most recent invocation of this shape
        agg[key] = {
            "world": last_world,
            "base": max(_f(r, "base_us") for r in rs), "ctrl": max(_f(r, "ctrl_us") for r in rs),
            "fused": max(_f(r, "fused_us") for r in rs), "base_p50": max(_f(r, "base_p50") for r in rs),
            "ctrl_p50": max(_f(r, "ctrl_p50") for r in rs), "fused_p50": max(_f(r, "fused_p50") for r in rs),
            "nccl": max(_f(r, "nccl_cublas_us") for r in rs), "roof": max(_f(r, "roofline_us") for r in rs),
            "order": rs[-1].get("order", ""),
        }
    return agg


def msweep(rows: list[dict]) -> str:
    agg = by_shape(rows)
    if not agg:
        return ""
    lines = ["## fused GEMM+RS sweep (worst rank)",
             f"{'M':>7} {'N':>6} {'K/rank':>7} {'tiles':>6} | {'base':>8} {'ctrl':>8} {'fused':>8} | {'struct':>6} {'comm':>6} {'total':>6} | "
             f"{'nccl+cublas':>11} {'speedup':>7} {'%roof':>6} | {'ns/tile':>8}"]
    resid = []
    for (m, n, k), a in sorted(agg.items()):
        tiles = (m // TILE_M) * (n // TILE_N)
        comm_abs = a["fused"] - a["ctrl"]
        ns_tile = comm_abs * 1000.0 / tiles if tiles else 0.0
        resid.append((m, ns_tile))
        st = a["ctrl"] / a["base"] if a["base"] else 0
        cm = a["fused"] / a["ctrl"] if a["ctrl"] else 0
        tt = a["fused"] / a["base"] if a["base"] else 0
        sp = a["nccl"] / a["fused"] if a["fused"] and a["nccl"] else 0
        pr = 100 * a["roof"] / a["fused"] if a["fused"] else 0
        lines.append(f"{m:7d} {n:6d} {k:7d} {tiles:6d} | {a['base']:8.1f} {a['ctrl']:8.1f} {a['fused']:8.1f} | {st:6.3f} {cm:6.3f} {tt:6.3f} | "
                     f"{a['nccl']:11.1f} {sp:7.3f} {pr:6.1f} | {ns_tile:8.1f}")
    big = [r for m, r in resid if m >= 4096]
    if len(big) >= 3:
        spread = (max(big) - min(big)) / (statistics.mean(big) or 1)
        lines.append(f"per-tile residual for M >= 4096: mean {statistics.mean(big):.1f} ns, spread {100 * spread:.0f} % -> "
                     + ("PLATEAU: the communication tax is per-tile work" if spread < 0.35 else "NO PLATEAU: a fixed cost is still being amortised"))
    return "\n".join(lines) + "\n"


def verdict_shift_or_tail(rows: list[dict]) -> str:
    agg = by_shape(rows)
    out = ["## verdict 1: shift or tail (comm ratio on means vs on p50s)"]
    for key, a in sorted(agg.items()):
        if not a["ctrl"] or not a["ctrl_p50"]:
            continue
        mean_r, p50_r = a["fused"] / a["ctrl"], a["fused_p50"] / a["ctrl_p50"]
        kind = "SHIFT (the whole distribution moved)" if abs(mean_r - p50_r) < 0.03 else "TAIL (outlier iterations lift the mean)"
        out.append(f"  M={key[0]}: comm {mean_r:.3f} on means, {p50_r:.3f} on p50s -> {kind}")
    return "\n".join(out) + "\n" if len(out) > 1 else ""


def verdict_tiles_or_duration(rows: list[dict]) -> str:
    agg = by_shape(rows)
    pts = [(k, a["ctrl"], a["fused"] - a["ctrl"]) for (m, n, k), a in sorted(agg.items()) if a["ctrl"]]
    if len(pts) < 2:
        return ""
    out = ["## verdict 2: does the absolute communication cost follow tiles or duration? (same M, N; K varies)"]
    for k, ctrl, cabs in pts:
        out.append(f"  K/rank={k}: ctrl {ctrl:.1f} us, comm_abs {cabs:.1f} us")
    cabs = [p[2] for p in pts]
    ctrl = [p[1] for p in pts]
    rel_spread = (max(cabs) - min(cabs)) / (max(abs(statistics.mean(cabs)), 1e-9))
    dur_ratio = max(ctrl) / max(min(ctrl), 1e-9)
    out.append("  -> " + ("TILES: the cost stays put while the kernel time changes %.1fx (it is paid per tile / per byte moved)" % dur_ratio
                          if rel_spread < 0.5 else "DURATION: the cost moves with the kernel time (exposure, not per-tile work)"))
    return "\n".join(out) + "\n"


def verdict_order(rows: list[dict]) -> str:
    runs: dict = {}
    for r in rows:
        runs.setdefault(r.get("order", ""), []).append(r)
    if len(runs) < 2:
        return ""
    out = ["## verdict 3: run-order bias (struct = ctrl/base under different variant orders)"]
    vals = []
    for order, rs in runs.items():
        b = max(_f(r, "base_us") for r in rs)
        c = max(_f(r, "ctrl_us") for r in rs)
        if b:
            vals.append(c / b)
            out.append(f"  order {order}: struct {c / b:.3f}")
    if vals:
        out.append("  -> " + ("NO BIAS: interleaved timing gives the same ratio in every order" if max(vals) - min(vals) < 0.02
                              else "BIAS: the ratio depends on the order; trust the interleaved p50s only"))
    return "\n".join(out) + "\n"


def verdict_tail_shape(bundle: str) -> str:
    files = sorted(glob.glob(os.path.join(bundle, "iters_*.rank0.csv")))
    if not files:
        return ""
    out = ["## verdict 4: tail shape of the fused variant (rank 0 per-iteration dumps)"]
    for f in files:
        us = [_f(r, "us") for r in read(f) if r.get("variant") == "fused"]
        if len(us) < 10:
            continue
        med = statistics.median(us)
        outliers = sum(1 for x in us if x > 1.15 * med)
        half = len(us) // 2
        drift = statistics.median(us[half:]) / statistics.median(us[:half])
        shape = "DRIFT over the run" if abs(drift - 1) > 0.03 else ("ISOLATED outliers" if outliers else "FLAT")
        out.append(f"  {os.path.basename(f)}: median {med:.1f} us, {outliers}/{len(us)} iterations > 1.15 x median, second half / first half {drift:.3f} -> {shape}")
    return "\n".join(out) + "\n" if len(out) > 1 else ""


def exp2_summary(rows: list[dict]) -> str:
    if not rows:
        return ""
    out = ["## AG+GEMM granularity"]
    best: dict = {}
    for r in rows:
        mode = r.get("mode", "")
        t = _f(r, "t_ovl_us")
        if t and (mode not in best or t < _f(best[mode], "t_ovl_us")):
            best[mode] = r
    for mode, r in best.items():
        out.append(f"  {mode}: best gather tile {r.get('chunk_rows')} rows (S={r.get('S')}), t_ovl {_f(r, 't_ovl_us'):.1f} us, overlap_eff {_f(r, 'overlap_eff'):.3f}, "
                   f"seg_eff {_f(r, 'seg_eff'):.3f}, speed-up {_f(r, 'speedup'):.3f}x, {_f(r, 'pct_roofline'):.1f} % of roofline, verify {r.get('verify')}")
    return "\n".join(out) + "\n"


def l2_verdict(bundle: str) -> str:
    out = []
    for tag in ("probe_cg", "probe_ca", "probe_st", "probe_tma", "probe_tmast"):
        rows = read(os.path.join(bundle, f"{tag}_bw.csv"))
        if not rows:
            continue
        curves: dict = {}
        for r in rows:
            curves.setdefault(r.get("target", ""), []).append((_f(r, "frac_l2"), _f(r, "gbps")))

        def knee(pts):
            # 1/64 of L2 and below can be served by L1: the L2 plateau is measured between L2/32 and L2/4
            ins = [g for fr, g in pts if 1 / 32 <= fr <= 0.25]
            outs = [g for fr, g in pts if fr >= 2.0]
            return (max(ins) / min(outs)) if ins and outs and min(outs) > 0 else 0.0

        kl, kp = knee(curves.get("local", [])), knee(curves.get("peer", []))
        if kl < 1.3:
            verdict = "INCONCLUSIVE (the local control shows no L2 knee: the instrument cannot see L2 here)"
        elif not curves.get("peer"):
            verdict = "CONTROL only (no peer GPU)"
        elif kp > 1.3:
            verdict = "CACHED: the peer curve has the knee too"
        else:
            verdict = "NOT CACHED in the requester's L2: the peer curve is flat across the L2 size"
        out.append(f"  {tag}: local knee {kl:.2f}x, peer knee {kp:.2f}x -> {verdict}")
        wire = read(os.path.join(bundle, f"{tag}_wire.csv"))
        ok = [r for r in wire if r.get("counters_ok") == "1"]
        if ok:
            out.append("    wire rx/asked: " + ", ".join(f"{int(_f(r, 'bytes')) >> 20} MiB {_f(r, 'rx_over_asked'):.3f}" for r in ok))
        elif wire:
            out.append("    wire: NVLink counters unavailable on this box")
    return ("## peer-L2 probe verdict\n" + "\n".join(out) + "\n") if out else ""


def interference_sanity(bundle: str) -> str:
    rows = read(os.path.join(bundle, "interference.csv"))
    if not rows:
        return ""
    out = ["## interference matrix"]
    worst_c = max((r for r in rows if r.get("mode") == "matrix"), key=lambda r: _f(r, "S_c"), default=None)
    worst_m = max((r for r in rows if r.get("mode") == "matrix"), key=lambda r: _f(r, "S_m"), default=None)
    ctrl = [r for r in rows if r.get("mode") == "matrix" and r.get("comm") == "ce" and r.get("probe") in ("tcgen05", "mma", "ffma", "smem")]
    if ctrl:
        bad = [r for r in ctrl if abs(_f(r, "S_c") - 1) > 0.05]
        out.append(f"  sanity (copy engine vs register-only probes must read 1.00): {'ok' if not bad else 'VIOLATED by ' + ', '.join(r['probe'] for r in bad)}")
    if worst_c:
        out.append(f"  largest compute slow-down: S_c {_f(worst_c, 'S_c'):.2f} ({worst_c['probe']} x {worst_c['comm']})")
    if worst_m:
        out.append(f"  largest transfer slow-down: S_m {_f(worst_m, 'S_m'):.2f} ({worst_m['probe']} x {worst_m['comm']})")
    return "\n".join(out) + "\n"


def tuning_summary(rows: list[dict]) -> str:
    """Knob sweeps of the fused ops (``run_all --tuning``): per op, one line per knob setting, fastest first,
    against NCCL + cuBLAS and against the default setting of the same sweep."""
    if not rows:
        return ""
    by_op: dict[str, dict[str, tuple[float, float]]] = {}
    for r in rows:
        t, n = _f(r, "max_over_ranks_us"), _f(r, "nccl_cublas_us")
        k = r.get("knobs", "?")
        op = next((p[3:] for p in k.split("|") if p.startswith("op=")), "gemm_rs")
        if t > 0:
            by_op.setdefault(op, {})[k] = (t, n)       # every rank's row carries the same max over ranks
    out = []
    for op, best in by_op.items():
        out.append(f"## knob sweep of the fused {op} (max over ranks)")
        ref = next((v for k, v in best.items() if "setting=default" in k), None)
        if ref is None:   # rows without a setting name: the default is the row with every knob at its default
            ref = next((v for k, v in best.items() if "rs_chunks=0|group_m=0|num_ctas=0|st256=0|ablate=0" in k and "cta_group=2" in k and "transport=p2p" in k), None)
        for k, (t, n) in sorted(best.items(), key=lambda kv: kv[1][0]):
            rel = f"  {ref[0] / t:5.3f}x of default" if ref else ""
            out.append(f"  {t:9.1f} us  {n / t if t else 0:5.3f}x of NCCL+cuBLAS{rel}  {k}")
    return "\n".join(out) + "\n" if out else ""


def report(bundle: str) -> str:
    parts = [f"# analysis of {os.path.basename(os.path.normpath(bundle))}\n"]
    ms = read(os.path.join(bundle, "exp3_fused_msweep.csv"))
    ks = read(os.path.join(bundle, "exp3_fused_ksweep.csv"))
    parts += [msweep(ms), verdict_shift_or_tail(ms), verdict_tiles_or_duration(ks), verdict_order(read(os.path.join(bundle, "exp3_order.csv"))),
              verdict_tail_shape(bundle), tuning_summary(read(os.path.join(bundle, "exp3_tuning.csv"))), exp2_summary(read(os.path.join(bundle, "exp2.csv"))), l2_verdict(bundle), interference_sanity(bundle)]
    mf = os.path.join(bundle, "manifest.txt")
    if os.path.exists(mf):
        lines = open(mf).read().splitlines()
        bad = [line for line in lines if " rc=0 " not in line + " " and "rc=skipped" not in line]
        parts.append(f"## manifest: {len(lines)} steps, {len(bad)} not ok" + ("".join("\n  " + b for b in bad)) + "\n")
    return "\n".join(p for p in parts if p)


def main(argv=None) -> int:
    argv = sys.argv[1:] if argv is None else argv
    if len(argv) != 1:
        print(__doc__)
        return 1
    print(report(argv[0]))
    return 0


if __name__ == "__main__":
    sys.exit(main())
