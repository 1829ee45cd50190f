"""Figures from the CSV files of a bundle, written as SVG files with no plotting dependency.

    python -m tileccl_b200.bench.plots reports/results_<stamp>

The reference draws its figures with matplotlib's headless Agg back end
(tests/plot_pk_bw.py, tests/plot_interference.py, l2_peer_cache/plot_peer_l2.py and the per-bundle
plot scripts) and keeps the measured numbers as literals inside those scripts.  Here the numbers
stay in the CSV files and a small built-in SVG writer draws them: line charts on log/linear axes
and grouped bars.
"""
from __future__ import annotations

import math
import os
import sys

from ..utils import csvio

PALETTE = ["#1f77b4", "#d62728", "#2ca02c", "#ff7f0e", "#9467bd", "#8c564b", "#17becf", "#7f7f7f"]


def _ticks(lo: float, hi: float, log: bool) -> list[float]:
    if log:
        a, b = math.floor(math.log10(max(lo, 1e-12))), math.ceil(math.log10(max(hi, 1e-12)))
        return [10.0 ** e for e in range(a, b + 1)]
    if hi <= lo:
        hi = lo + 1
    step = 10 ** math.floor(math.log10((hi - lo) / 4))
    for m in (1, 2, 5, 10):
        if (hi - lo) / (step * m) <= 6:
            step *= m
            break
    t0 = math.floor(lo / step) * step
    return [t0 + i * step for i in range(int((hi - t0) / step) + 2)]


def _fmt(v: float) -> str:
    if v == 0:
        return "0"
    if abs(v) >= 1 << 30 and v % (1 << 20) == 0:
        return f"{v / (1 << 30):g}G"
    if abs(v) >= 1 << 20 and v % (1 << 10) == 0:
        return f"{v / (1 << 20):g}M"
    if abs(v) >= 1 << 10 and v % (1 << 10) == 0:
        return f"{v / (1 << 10):g}K"
    return f"{v:g}"


def line_chart(path: str, series: dict[str, list[tuple[float, float]]], title: str, xlabel: str, ylabel: str,
               logx: bool = False, logy: bool = False, w: int = 720, h: int = 420) -> None:
    """series: name -> [(x, y)]."""
    pts = [p for s in series.values() for p in s if p[1] > 0 or not logy]
    if not pts:
        return
    xs, ys = [p[0] for p in pts], [p[1] for p in pts]
    x0, x1, y0, y1 = min(xs), max(xs), (min(ys) if logy else 0.0), max(ys) * 1.05
    L, R, T, B = 70, 160, 40, 50
    tx = (lambda v: math.log10(v)) if logx else (lambda v: v)
    ty = (lambda v: math.log10(v)) if logy else (lambda v: v)
    X = lambda v: L + (tx(v) - tx(x0)) / max(tx(x1) - tx(x0), 1e-12) * (w - L - R)  # noqa: E731
    Y = lambda v: h - B - (ty(v) - ty(y0)) / max(ty(y1) - ty(y0), 1e-12) * (h - T - B)  # noqa: E731
    o = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{w}" height="{h}" font-family="sans-serif" font-size="11">',
         f'<rect width="{w}" height="{h}" fill="white"/><text x="{w / 2}" y="20" text-anchor="middle" font-size="14">{title}</text>']
    for t in _ticks(x0, x1, logx):
        if x0 <= t <= x1:
            o.append(f'<line x1="{X(t):.1f}" y1="{T}" x2="{X(t):.1f}" y2="{h - B}" stroke="#ddd"/><text x="{X(t):.1f}" y="{h - B + 14}" text-anchor="middle">{_fmt(t)}</text>')
    for t in _ticks(y0, y1, logy):
        if y0 <= t <= y1:
            o.append(f'<line x1="{L}" y1="{Y(t):.1f}" x2="{w - R}" y2="{Y(t):.1f}" stroke="#ddd"/><text x="{L - 6}" y="{Y(t) + 4:.1f}" text-anchor="end">{_fmt(t)}</text>')
    o.append(f'<rect x="{L}" y="{T}" width="{w - L - R}" height="{h - T - B}" fill="none" stroke="black"/>')
    o.append(f'<text x="{(L + w - R) / 2}" y="{h - 10}" text-anchor="middle">{xlabel}</text>')
    o.append(f'<text x="14" y="{(T + h - B) / 2}" text-anchor="middle" transform="rotate(-90 14 {(T + h - B) / 2})">{ylabel}</text>')
    for i, (name, s) in enumerate(series.items()):
        c = PALETTE[i % len(PALETTE)]
        s = sorted(p for p in s if (p[1] > 0 or not logy))
        if not s:
            continue
        o.append(f'<polyline fill="none" stroke="{c}" stroke-width="1.8" points="' + " ".join(f"{X(x):.1f},{Y(y):.1f}" for x, y in s) + '"/>')
        o += [f'<circle cx="{X(x):.1f}" cy="{Y(y):.1f}" r="2.5" fill="{c}"/>' for x, y in s]
        o.append(f'<rect x="{w - R + 10}" y="{T + 16 * i}" width="12" height="3" fill="{c}"/><text x="{w - R + 28}" y="{T + 16 * i + 5}">{name}</text>')
    o.append("</svg>")
    with open(path, "w") as f:
        f.write("\n".join(o))


def bar_chart(path: str, groups: list[str], series: dict[str, list[float]], title: str, ylabel: str, ref_line: float | None = None,
              w: int = 760, h: int = 420) -> None:
    vals = [v for s in series.values() for v in s]
    if not vals:
        return
    y1 = max(vals + ([ref_line] if ref_line else [])) * 1.1
    L, R, T, B = 60, 150, 40, 70
    gw = (w - L - R) / max(1, len(groups))
    bw = gw * 0.8 / max(1, len(series))
    Y = lambda v: h - B - v / y1 * (h - T - B)  # noqa: E731
    o = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{w}" height="{h}" font-family="sans-serif" font-size="11">',
         f'<rect width="{w}" height="{h}" fill="white"/><text x="{w / 2}" y="20" text-anchor="middle" font-size="14">{title}</text>']
    for t in _ticks(0, y1, False):
        if t <= y1:
            o.append(f'<line x1="{L}" y1="{Y(t):.1f}" x2="{w - R}" y2="{Y(t):.1f}" stroke="#ddd"/><text x="{L - 6}" y="{Y(t) + 4:.1f}" text-anchor="end">{_fmt(t)}</text>')
    for gi, g in enumerate(groups):
        for si, (name, s) in enumerate(series.items()):
            if gi < len(s):
                x = L + gi * gw + gw * 0.1 + si * bw
                o.append(f'<rect x="{x:.1f}" y="{Y(s[gi]):.1f}" width="{bw:.1f}" height="{h - B - Y(s[gi]):.1f}" fill="{PALETTE[si % len(PALETTE)]}"/>')
        o.append(f'<text x="{L + gi * gw + gw / 2:.1f}" y="{h - B + 14}" text-anchor="middle">{g}</text>')
    if ref_line:
        o.append(f'<line x1="{L}" y1="{Y(ref_line):.1f}" x2="{w - R}" y2="{Y(ref_line):.1f}" stroke="black" stroke-dasharray="4 3"/>')
    for si, name in enumerate(series):
        o.append(f'<rect x="{w - R + 10}" y="{T + 16 * si}" width="12" height="8" fill="{PALETTE[si % len(PALETTE)]}"/><text x="{w - R + 28}" y="{T + 16 * si + 8}">{name}</text>')
    o.append(f'<rect x="{L}" y="{T}" width="{w - L - R}" height="{h - T - B}" fill="none" stroke="black"/>')
    o.append(f'<text x="14" y="{(T + h - B) / 2}" text-anchor="middle" transform="rotate(-90 14 {(T + h - B) / 2})">{ylabel}</text></svg>')
    with open(path, "w") as f:
        f.write("\n".join(o))


def _rows(bundle: str, name: str) -> list[dict]:
    p = os.path.join(bundle, name)
    return csvio.read_rows(p) if os.path.exists(p) else []


def _num(r: dict, k: str) -> float:
    try:
        return float(r.get(k, 0))
    except ValueError:
        return 0.0


def make_all(bundle: str) -> list[str]:
    made = []
    figs = os.path.join(bundle, "figs")
    os.makedirs(figs, exist_ok=True)

    def done(p):
        if os.path.exists(p):
            made.append(p)

    r = _rows(bundle, "pk_bw.csv")
    if r:
        for fig, key, lx, xl in (("size", "msg_bytes", True, "message size (bytes)"), ("sms", "sms", False, "SMs")):
            s: dict = {}
            for row in r:
                if row.get("figure") == fig:
                    s.setdefault(row["mover"], []).append((_num(row, key), _num(row, "gbps")))
            p = os.path.join(figs, f"pk_bw_vs_{fig}.svg")
            line_chart(p, s, f"P2P push bandwidth vs {fig}", xl, "GB/s", logx=lx)
            done(p)
    for tag in ("probe_cg", "probe_ca"):
        r = _rows(bundle, f"{tag}_bw.csv")
        if r:
            s = {}
            for row in r:
                s.setdefault(row["target"], []).append((_num(row, "bytes"), _num(row, "gbps")))
            p = os.path.join(figs, f"peer_l2_{tag}.svg")
            line_chart(p, s, f"streaming bandwidth vs working set ({tag})", "working set (bytes)", "GB/s", logx=True, logy=True)
            done(p)
    r = _rows(bundle, "signal_fanin.csv")
    if r:
        s = {}
        for row in r:
            if row["mode"] in ("signal", "post") or row.get("bytes") == "4096":
                s.setdefault(row["mode"], []).append((_num(row, "fanin"), _num(row, "p50_us")))
        p = os.path.join(figs, "signal_fanin.svg")
        line_chart(p, s, "completion latency vs fan-in (p50, 4 KiB payload)", "logical producers", "us", logx=True)
        done(p)
    r = _rows(bundle, "exp3_fused_msweep.csv")
    if r:
        agg: dict = {}
        for row in r:
            a = agg.setdefault(int(_num(row, "m")), {"f": 0.0, "n": 0.0, "roof": 0.0})
            a["f"] = max(a["f"], _num(row, "fused_us"))
            a["n"] = max(a["n"], _num(row, "nccl_cublas_us"))
            a["roof"] = max(a["roof"], _num(row, "roofline_us"))
        ms = sorted(agg)
        p = os.path.join(figs, "gemm_rs_msweep.svg")
        bar_chart(p, [str(m) for m in ms], {"fused": [agg[m]["f"] for m in ms], "NCCL+cuBLAS": [agg[m]["n"] for m in ms],
                                            "roofline": [agg[m]["roof"] for m in ms]}, "GEMM+RS time vs M (max over ranks)", "us")
        done(p)
    r = _rows(bundle, "exp2.csv")
    if r:
        s = {}
        for row in r:
            s.setdefault(row["mode"], []).append((_num(row, "chunk_rows"), _num(row, "e2e_tflops")))
        p = os.path.join(figs, "ag_gemm_granularity.svg")
        line_chart(p, s, "AG+GEMM end-to-end TFLOP/s vs gather tile", "rows per gather tile", "TFLOP/s", logx=True)
        done(p)
    r = [x for x in _rows(bundle, "interference.csv") if x.get("mode") == "matrix"]
    if r:
        probes = sorted({x["probe"] for x in r})
        for metric in ("S_c", "S_m"):
            ser = {c: [next((_num(x, metric) for x in r if x["probe"] == pr and x["comm"] == c), 0.0) for pr in probes] for c in sorted({x["comm"] for x in r})}
            p = os.path.join(figs, f"interference_{metric}.svg")
            bar_chart(p, probes, ser, f"interference matrix: {metric}", metric, ref_line=1.0)
            done(p)
    r = [x for x in _rows(bundle, "nvls_bw.csv") if _num(x, "bytes") > 0]
    if r:
        s = {}
        for row in r:
            s.setdefault(row["mover"], []).append((_num(row, "bytes"), _num(row, "gbps")))
        p = os.path.join(figs, "nvls_bw.svg")
        line_chart(p, s, "NVSwitch paths: bandwidth per rank vs payload (all ranks active)", "payload (bytes)", "GB/s", logx=True, logy=True)
        done(p)
    r = _rows(bundle, "exp3_tuning.csv")
    if r:
        best: dict = {}
        for row in r:
            if _num(row, "max_over_ranks_us") > 0:
                best[row.get("knobs", "?")] = (_num(row, "max_over_ranks_us"), _num(row, "nccl_cublas_us"), _num(row, "roofline_us"))
        if best:
            ks = sorted(best, key=lambda k: best[k][0])
            short = ["|".join(kv for kv in k.split("|") if not kv.endswith("=0") and kv not in ("transport=p2p", "cta_group=2")) or "default" for k in ks]
            p = os.path.join(figs, "gemm_rs_tuning.svg")
            bar_chart(p, short, {"fused": [best[k][0] for k in ks], "NCCL+cuBLAS": [best[k][1] for k in ks], "roofline": [best[k][2] for k in ks]},
                      "GEMM+RS knob sweep (max over ranks)", "us")
            done(p)
    r = _rows(bundle, "pipeline_e2e.csv")
    if r:
        s = {}
        for row in r:
            s.setdefault(row["method"], []).append((max(_num(row, "intensity"), 1), _num(row, "To_ms")))
        p = os.path.join(figs, "pipeline_e2e.svg")
        line_chart(p, s, "producer -> transfer -> consumer: overlapped time", "FMAs per element", "ms", logx=True, logy=True)
        done(p)
    return made


def main(argv=None) -> int:
    argv = sys.argv[1:] if argv is None else argv
    if len(argv) != 1:
        print(__doc__)
        return 1
    for p in make_all(argv[0]):
        print(p)
    return 0


if __name__ == "__main__":
    sys.exit(main())
