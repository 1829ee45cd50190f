"""Same-box comparison with the reference's own plain-CUDA movers.

Two of the reference's programs build for sm_100a without any third-party code and contain no wait on
another GPU (their only spins are on the local mbarrier of a bulk copy the same thread issued):
``tests/pk_bw_sweep.cu`` (bandwidth against message size and SM count for the copy engine, the bulk-copy
pipeline and register copies) and ``tests/p2p_ce_vs_tma.cu`` (token-granular transfers, eight methods).
This driver builds them unmodified, runs them and this package's counterparts with the same arguments on
the same pair of GPUs, and writes the figures side by side.

    python -m tileccl_b200.bench.ref_movers --build --reference-dir <checkout of the reference>
    python -m tileccl_b200.bench.ref_movers --run --out <dir>          # needs 2 GPUs

The reference's binaries land in ``baseline/_ref/bin`` (not tracked).  The reference prints tables only
(tests/pk_bw_sweep.cu:756-774, tests/p2p_ce_vs_tma.cu:774-789); they are parsed here.  The other reference
probes spin on flags that a second GPU writes, without a limit, and are not run.
"""
from __future__ import annotations

import argparse
import re
import shutil
import subprocess
import sys
from pathlib import Path

from ..utils import csvio

ROOT = Path(__file__).resolve().parents[2]
REF_BIN = ROOT / "baseline" / "_ref" / "bin"
OWN_BIN = Path(__file__).resolve().parents[1] / "bin"
PROGRAMS = ("pk_bw_sweep", "p2p_ce_vs_tma")
COLUMNS = "program,row,method,size,ref_gbps,own_gbps,own_over_ref,ref_us,own_us".split(",")

_UNITS = {"B": 1, "KiB": 1 << 10, "MiB": 1 << 20, "GiB": 1 << 30}


def build(reference_dir: str, verbose: bool = True) -> list[Path]:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    REF_BIN.mkdir(parents=True, exist_ok=True)
    outs = []
    for name in PROGRAMS:
        src = Path(reference_dir) / "tests" / f"{name}.cu"
        out = REF_BIN / name
        cmd = [nvcc, "-O3", "-std=c++17", "-lineinfo", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(out), str(src)]
        if verbose:
            print(" ".join(cmd))
        subprocess.run(cmd, check=True)
        outs.append(out)
    return outs


def parse_size(text: str) -> int:
    m = re.fullmatch(r"(\d+)\s*(B|KiB|MiB|GiB)", text.strip())
    if not m:
        raise ValueError(f"bad size {text!r}")
    return int(m.group(1)) * _UNITS[m.group(2)]


def parse_pk_fig2(text: str) -> dict[tuple[str, int], float]:
    """{(method, msg_bytes): GB/s} from the reference's 'bandwidth vs message size' table."""
    out: dict[tuple[str, int], float] = {}
    lines = text.splitlines()
    for i, line in enumerate(lines):
        if line.startswith("msg_size"):
            methods = line.split()[1:]
            for row in lines[i + 1:]:
                m = re.match(r"^(\d+ (?:B|KiB|MiB|GiB))\s+(.*)$", row)
                if not m:
                    break
                size = parse_size(m.group(1))
                cells = re.findall(r"(-|[0-9.]+)[*^! ]?", m.group(2))
                cells = [c for c in cells if c != ""]
                for meth, c in zip(methods, cells):
                    if c != "-":
                        out[(meth, size)] = float(c)
            break
    return out


def parse_pk_fig3(text: str) -> dict[tuple[str, int], float]:
    """{(method, sms): GB/s} from the 'bandwidth vs SM count' table."""
    out: dict[tuple[str, int], float] = {}
    lines = text.splitlines()
    for i, line in enumerate(lines):
        if re.match(r"^sms\s", line):
            methods = line.split()[1:]
            for row in lines[i + 1:]:
                p = row.split()
                if not p or not p[0].isdigit():
                    break
                for meth, c in zip(methods, p[1:]):
                    c = c.rstrip("*^!")
                    if c not in ("-", ""):
                        out[(meth, int(p[0]))] = float(c)
            break
    return out


def parse_p2p(text: str) -> dict[tuple[str, int], tuple[float, float]]:
    """{(method, tokens): (avg_us, GB/s)} from the reference's per-token-count blocks."""
    out: dict[tuple[str, int], tuple[float, float]] = {}
    tokens = None
    for line in text.splitlines():
        m = re.match(r"^--- tokens=(\d+)", line)
        if m:
            tokens = int(m.group(1))
            continue
        p = line.split()
        if tokens is not None and len(p) >= 5 and re.fullmatch(r"[a-z_]+", p[0]) and p[0] != "method":
            try:
                out[(p[0], tokens)] = (float(p[1]), float(p[4]))
            except ValueError:
                continue
    return out


def run(out_dir: Path, total: str, tokens: str, iters: int) -> int:
    out_dir.mkdir(parents=True, exist_ok=True)

    def call(cmd: list[str], log: str) -> str:
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
        (out_dir / log).write_text("$ " + " ".join(Path(c).name if c.startswith("/") else c for c in cmd) + "\n" + r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError(f"{cmd[0]} exited with {r.returncode}; see {log}")
        return r.stdout

    for name in PROGRAMS:
        if not (REF_BIN / name).exists():
            print(f"{REF_BIN / name} is missing: run with --build --reference-dir first", file=sys.stderr)
            return 2
    csv = csvio.CsvAppender(str(out_dir / "ref_movers.csv"), COLUMNS)
    # ---- pk_bw_sweep: the same payload, iteration count and sweeps on both ----
    ref = call([str(REF_BIN / "pk_bw_sweep"), "--total", total, "--iters", str(iters)], "ref_pk_bw_sweep.log")
    call([str(OWN_BIN / "pk_bw_sweep"), "--total", total, "--iters", str(iters), "--csv", str(out_dir / "own_pk_bw.csv")], "own_pk_bw_sweep.log")
    own = csvio.read_rows(str(out_dir / "own_pk_bw.csv"))
    f2, f3 = parse_pk_fig2(ref), parse_pk_fig3(ref)
    own2 = {(r["mover"], int(r["msg_bytes"])): float(r["gbps"]) for r in own if r["figure"] == "size"}
    own3 = {(r["mover"], int(r["sms"])): float(r["gbps"]) for r in own if r["figure"] == "sms"}
    print(f"{'program':14s} {'row':6s} {'method':10s} {'size':>11s} | {'ref GB/s':>9s} {'own GB/s':>9s} {'own/ref':>8s}")
    for (meth, size), g in sorted(f2.items(), key=lambda kv: (kv[0][0], kv[0][1])):
        o = own2.get((meth, size))
        if o is None:
            continue
        print(f"{'pk_bw_sweep':14s} {'size':6s} {meth:10s} {size:11d} | {g:9.2f} {o:9.2f} {o / g if g else 0:8.3f}")
        csv.row(program="pk_bw_sweep", row="size", method=meth, size=size, ref_gbps=g, own_gbps=o, own_over_ref=o / g if g else 0, ref_us="", own_us="")
    for (meth, sms), g in sorted(f3.items(), key=lambda kv: (kv[0][0], kv[0][1])):
        o = own3.get((meth, sms))
        if o is None:
            continue
        print(f"{'pk_bw_sweep':14s} {'sms':6s} {meth:10s} {sms:11d} | {g:9.2f} {o:9.2f} {o / g if g else 0:8.3f}")
        csv.row(program="pk_bw_sweep", row="sms", method=meth, size=sms, ref_gbps=g, own_gbps=o, own_over_ref=o / g if g else 0, ref_us="", own_us="")
    # ---- p2p_ce_vs_tma ----
    ref = call([str(REF_BIN / "p2p_ce_vs_tma"), "--tokens", tokens, "--iters", str(max(iters, 20))], "ref_p2p_ce_vs_tma.log")
    call([str(OWN_BIN / "p2p_ce_vs_tma"), "--tokens", tokens, "--iters", str(max(iters, 20)), "--csv", str(out_dir / "own_p2p_ce_vs_tma.csv")], "own_p2p_ce_vs_tma.log")
    refp = parse_p2p(ref)
    ownp = {(r["method"], int(r["tokens"])): (float(r["avg_us"]), float(r["gbps"])) for r in csvio.read_rows(str(out_dir / "own_p2p_ce_vs_tma.csv"))}
    for (meth, tok), (us, g) in sorted(refp.items(), key=lambda kv: (kv[0][0], kv[0][1])):
        if (meth, tok) not in ownp:
            continue
        ous, og = ownp[(meth, tok)]
        print(f"{'p2p_ce_vs_tma':14s} {'tokens':6s} {meth:10s} {tok:11d} | {g:9.2f} {og:9.2f} {og / g if g else 0:8.3f}   ({us:.2f} us vs {ous:.2f} us)")
        csv.row(program="p2p_ce_vs_tma", row="tokens", method=meth, size=tok, ref_gbps=g, own_gbps=og, own_over_ref=og / g if g else 0, ref_us=us, own_us=ous)
    csv.close()
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--build", action="store_true")
    ap.add_argument("--reference-dir", default=None, help="checkout of the reference (for --build)")
    ap.add_argument("--run", action="store_true")
    ap.add_argument("--out", default="reports/ref_movers")
    ap.add_argument("--total", default="256M", help="payload per measurement of pk_bw_sweep")
    ap.add_argument("--tokens", default="1,64,1024,4096")
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args(argv)
    if args.build:
        if not args.reference_dir:
            ap.error("--build needs --reference-dir")
        build(args.reference_dir)
    if args.run:
        return run(Path(args.out), args.total, args.tokens, args.iters)
    return 0


if __name__ == "__main__":
    sys.exit(main())
