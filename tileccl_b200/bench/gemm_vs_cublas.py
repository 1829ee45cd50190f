"""Plain GEMM: the tcgen05 kernel (CTA pairs and single CTAs, several raster group heights) against
cuBLAS on one GPU, one iteration of every variant in turn (same clocks and temperature for all),
L2 flushed between iterations.

    python -m tileccl_b200.bench.gemm_vs_cublas [--shapes 32768x8192x8192,32768x3584x8192] [--iters 12]

The reference's counterpart is the `local` row of comm_comp/exp3_epilogue_remote.cu (its own GEMM
alone); cuBLAS is the library baseline here.
"""
from __future__ import annotations

import argparse
import sys

import torch

from ..ops import elementwise as ew
from ..ops.gemm import GemmPlan
from ..utils.timing import L2Flusher
from . import _common as C


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--shapes", default="32768x8192x8192,32768x3584x8192,16384x14336x8192,8192")
    ap.add_argument("--group-m", default="4,8,16")
    ap.add_argument("--iters", type=int, default=12)
    args = ap.parse_args(argv)
    flush = L2Flusher()
    print(f"# gemm_vs_cublas [{C.device_line()}]  p50 us / TFLOP/s, variants interleaved")
    for shape in C.split_csv(args.shapes):
        M, N, K = C.parse_shape(shape)
        A = torch.empty(M, K, device="cuda", dtype=torch.bfloat16)
        Bt = torch.empty(N, K, device="cuda", dtype=torch.bfloat16)
        ew.fill_normal_(A, 1)
        ew.fill_normal_(Bt, 2, std=0.02)
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        fns = {f"pair_gm{g}": GemmPlan(A, Bt, out=out, cta_group=2, group_m=int(g)) for g in C.split_csv(args.group_m)}
        fns["single_cta"] = GemmPlan(A, Bt, out=out, cta_group=1)
        fns["cublas"] = lambda: torch.matmul(A, Bt.t(), out=out)
        ser = C.timed_interleaved(fns, args.iters, 3, flush=flush)
        fl = 2.0 * M * N * K / 1e6
        base = C.stats_of(ser["cublas"]).p50
        cells = "  ".join(f"{k} {C.stats_of(v).p50:.0f}/{fl / C.stats_of(v).p50:.0f} ({base / C.stats_of(v).p50:.3f}x)" for k, v in ser.items())
        print(f"{M}x{N}x{K}: {cells}")
        for p in fns.values():
            if hasattr(p, "check"):
                p.check()
    return 0


if __name__ == "__main__":
    sys.exit(main())
