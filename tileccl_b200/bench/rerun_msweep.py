"""Diagnostic rerun of the fused GEMM+RS: the questions a surprising M-sweep raises, as three short
steps (or the full M-sweep with ``--full``), followed by the analysis.

    python -m tileccl_b200.bench.rerun_msweep [--full] [--quick] [--out DIR]

  step 1  statistics at the large shape with per-iteration dumps     -> shift or tail? tail shape?
  step 2  K-sweep at fixed M, N                                       -> tiles or duration?
  step 3  the same shape under different variant orders               -> run-order bias?

It drives the same steps as ``run_all`` (which see) restricted to the fused GEMM+RS experiments.
Reference parity: comm_comp/rerun_m32768.sh (run_point :148-163, steps :191-212) + analyze_rerun.py.
"""
from __future__ import annotations

import sys
import time

from . import run_all


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if "-h" in argv or "--help" in argv:
        print(__doc__)
        print("Other flags are those of run_all:\n")
    full = "--full" in argv
    argv = [a for a in argv if a != "--full"]
    if "--out" not in argv and "--resume" not in argv:
        argv += ["--out", f"reports/rerun_{time.strftime('%Y%m%d_%H%M%S')}"]
    only = "exp3_fused_m" if full else "exp3_fused_m32768,exp3_fused_k,exp3_order"
    return run_all.main(argv + ["--only", only, "--keep"])


if __name__ == "__main__":
    sys.exit(main())
