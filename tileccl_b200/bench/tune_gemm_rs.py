"""Knob sweep of the fused GEMM + reduce-scatter in ONE process per rank.

Builds one plan per knob setting on the same operands and times all of them (and NCCL + cuBLAS)
one iteration each in turn, so that every setting sees the same clocks; prints the settings
fastest first and appends one row per setting to the CSV (the columns of the fused experiment,
`knobs` telling the setting; `max_over_ranks_us` is the figure to compare).

    python -m tileccl_b200.launch -n 8 tune_gemm_rs --m 32768 --n 8192 --k-global 8192 --csv exp3_tuning.csv

Settings: default; 32-byte epilogue stores; raster group heights; chunks per segment; fewer CTAs;
single-CTA tiles; and three timing-only ablations (no reduce warps, no tile signals, neither: their
results are not valid outputs, they show where the time goes).  ``--only`` narrows the list.

The reference tunes by hand-edited reruns (comm_comp/rerun_m32768.sh:148-212); it has no sweep driver.
"""
from __future__ import annotations

import argparse
import sys

import torch

from ..ops import baseline as base_ops
from ..ops import elementwise as ew
from ..ops.gemm_rs import GemmRs
from ..parallel import group as G
from ..parallel.heap import SymmetricHeap
from ..utils import csvio, roofline
from ..utils.timing import L2Flusher
from . import _common as C

SETTINGS: dict[str, dict] = {
    "default": {},
    "st256": {"st256": True},
    "gm4": {"group_m": 4}, "gm16": {"group_m": 16}, "gm32": {"group_m": 32},
    "chunks1": {"rs_chunks": 1}, "chunks4": {"rs_chunks": 4},
    "ctas128": {"num_ctas": 128}, "ctas96": {"num_ctas": 96},
    "cg1": {"cta_group": 1},
    "noreduce": {"ablate": 1}, "nosignal": {"ablate": 2}, "nocomm_warps": {"ablate": 3},
}


def knobs_string(kw: dict, transport: str = "p2p") -> str:
    full = {"cta_group": 2, "transport": transport, "rs_chunks": 0, "group_m": 0, "num_ctas": 0, "st256": 0, "ablate": 0}
    full.update({k: int(v) if isinstance(v, bool) else v for k, v in kw.items()})
    return "|".join(f"{k}={v}" for k, v in full.items())


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--m", type=C.parse_size, default=32768)
    ap.add_argument("--n", type=C.parse_size, default=8192)
    ap.add_argument("--k", type=C.parse_size, default=0, help="K per rank")
    ap.add_argument("--k-global", type=C.parse_size, default=8192)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--only", default=None, help="comma list of setting names (default: all that fit the shape)")
    ap.add_argument("--csv", default=None)
    args = ap.parse_args(argv)
    rank, world, _ = G.init()
    M, N = args.m, args.n
    K = args.k if args.k > 0 else args.k_global // world
    dev = torch.device("cuda", torch.cuda.current_device())
    names = C.split_csv(args.only) if args.only else list(SETTINGS)
    for n in names:
        if n not in SETTINGS:
            ap.error(f"unknown setting {n!r}; known: {', '.join(SETTINGS)}")
    per_plan = M * N * 2 + (M // world) * N * 2 + (1 << 20)
    heap = SymmetricHeap(len(names) * per_plan + (64 << 20))
    A = torch.empty(M, K, dtype=torch.bfloat16, device=dev)
    Bt = torch.empty(N, K, dtype=torch.bfloat16, device=dev)
    ew.fill_normal_(A, seed=1000 + rank)
    ew.fill_normal_(Bt, seed=2000 + rank)
    plans: dict[str, GemmRs] = {}
    skipped = []
    for n in names:
        try:
            plans[n] = GemmRs(heap, A, Bt, **SETTINGS[n])
        except ValueError as e:          # a setting that does not tile this shape (e.g. rs_chunks that does not divide)
            skipped.append(f"{n}: {e}")
    # every rank must time the same set
    ok = G.all_gather_object(sorted(plans))
    common = [n for n in names if all(n in o for o in ok)]
    D = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
    out_nccl = torch.empty(M // world, N, dtype=torch.bfloat16, device=dev) if world > 1 else None
    runners = {n: plans[n] for n in common}
    runners["nccl"] = lambda: base_ops.gemm_rs_baseline(A, Bt, out=out_nccl, full=D)
    bar = ew.DeviceBarrier(heap)
    flush = L2Flusher()
    series = C.timed_interleaved(runners, args.iters, args.warmup, before=bar, flush=flush)
    torch.cuda.synchronize()
    bar.check()
    for n in common:
        plans[n].check()
    mine = {n: C.stats_of(v).mean for n, v in series.items()}
    allr = G.all_gather_object(mine)
    if rank == 0:
        roof = roofline.gemm_rs_roofline_us(M, N, K, world)
        worst = {n: max(r[n] for r in allr) for n in mine}
        nccl = worst.pop("nccl")
        print(f"# tune_gemm_rs M={M} N={N} K/rank={K} world={world} iters={args.iters} [{C.device_line()}]")
        for s in skipped:
            print(f"# skipped {s}")
        print(f"{'setting':14s} | {'us (max over ranks)':>20s} | vs NCCL+cuBLAS | vs default | % roofline")
        csv = csvio.CsvAppender(args.csv, csvio.EXP3_FUSED_COLUMNS)
        dflt = worst.get("default", 0.0)
        for n in sorted(worst, key=worst.get):
            t = worst[n]
            print(f"{n:14s} | {t:20.1f} | {nccl / t:14.3f} | {dflt / t if dflt else 0:10.3f} | {100 * roof['roofline_burst_us'] / t:9.1f}"
                  + ("   (timing only)" if SETTINGS[n].get("ablate") else ""))
            csv.row(m=M, n=N, k=K, world=world, rank=0, fused_us=mine[n], order="|".join(runners), iters=args.iters, max_over_ranks_us=t,
                    nccl_cublas_us=nccl, speedup=nccl / t, roofline_us=roof["roofline_burst_us"], pct_roofline=100 * roof["roofline_burst_us"] / t, dtype="bf16",
                    knobs=knobs_string(SETTINGS[n]))
        csv.close()
        print(f"nccl+cublas    | {nccl:20.1f}")
    torch.cuda.synchronize()
    G.host_barrier()
    heap.close()
    G.shutdown()
    return 0


if __name__ == "__main__":
    sys.exit(main())
