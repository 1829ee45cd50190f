"""Knob sweep of the two fused ops in ONE process per rank.

Builds one plan per knob setting on the same operands and times all of them (and NCCL + cuBLAS) one
iteration each in turn, so that every setting sees the same clocks; prints the settings fastest first and
appends one row per setting to the CSV (`knobs` tells the setting, `max_over_ranks_us` is the figure to
compare).  A device barrier and an L2 flush run, untimed, ahead of every timed call.

    python -m tileccl_b200.launch -n 8 tune_fused --ops rs,ag --csv tuning.csv

GEMM + reduce-scatter settings: default; 32-byte epilogue stores; raster group heights; chunks per segment;
fewer CTAs; single-CTA tiles; the in-switch reduction (`nvls`, when the GPUs support multicast); and two
timing-only ablations (no reduce warps; no tile signals and no reduce warps).  All-gather + GEMM settings: gather
granularities, 8-row work items, the push form, single-CTA tiles, and two floors of the same kernel: `nowait`
(the TMA producer does not wait for gathered rows: what the gather costs in exposed time is
default - nowait) and `nocomm` (no gather at all).  Results of the ablations and floors are not valid
outputs; they show where the time goes.  ``--only`` narrows the list.

The reference tunes by hand-edited reruns (comm_comp/rerun_m32768.sh:148-212); it has no sweep driver.
"""
from __future__ import annotations

import argparse
import sys

import torch

from .. import _native
from ..ops import baseline as base_ops
from ..ops import elementwise as ew
from ..ops.ag_gemm import AgGemm
from ..ops.gemm_rs import GemmRs
from ..parallel import group as G
from ..parallel.heap import SymmetricHeap
from ..utils import csvio, roofline
from ..utils.timing import L2Flusher
from . import _common as C

RS_SETTINGS: dict[str, dict] = {
    "default": {},
    "st256": {"st256": True},
    "gm4": {"group_m": 4}, "gm16": {"group_m": 16}, "gm32": {"group_m": 32},
    "chunks1": {"rs_chunks": 1}, "chunks4": {"rs_chunks": 4}, "chunks8": {"rs_chunks": 8},
    "ctas128": {"num_ctas": 128}, "ctas96": {"num_ctas": 96}, "ctas64": {"num_ctas": 64},
    "sb1": {"signal_batch": 1}, "sb2": {"signal_batch": 2}, "sb8": {"signal_batch": 8}, "sb16": {"signal_batch": 16},
    "cg1": {"cta_group": 1}, "cg1_sb1": {"cta_group": 1, "signal_batch": 1}, "cg1_sb8": {"cta_group": 1, "signal_batch": 8},
    "nvls": {"transport": "nvls"}, "nvls_sb1": {"transport": "nvls", "signal_batch": 1},
    "noreduce": {"ablate": 1}, "nosignal": {"ablate": 3},
}
AG_SETTINGS: dict[str, dict] = {
    "default": {},
    "gr128": {"gather_rows": 128}, "gr2048": {"gather_rows": 2048}, "gr4096": {"gather_rows": 4096},
    "item8": {"item_rows": 8},
    "gw2": {"gather_warps": 2}, "gw3": {"gather_warps": 3}, "v32": {"vec32": True}, "gw2_v32": {"gather_warps": 2, "vec32": True},
    "gw2_v32_gm16": {"gather_warps": 2, "vec32": True, "group_m": 16},
    "gw2_gm16": {"gather_warps": 2, "group_m": 16}, "gw2_gm16_gr2048": {"gather_warps": 2, "group_m": 16, "gather_rows": 2048},
    "gw2_gr4096": {"gather_warps": 2, "gather_rows": 4096}, "gm16_gr2048": {"group_m": 16, "gather_rows": 2048},
    "gm4": {"group_m": 4}, "gm16": {"group_m": 16},
    "cg1": {"cta_group": 1},
    "push": {"transport": "push"},
    "nowait": {"ablate": 4}, "nocomm": {"comm_enabled": False},
}
TIMING_ONLY = {"noreduce", "nosignal", "nowait", "nocomm"}


def knobs_string(kw: dict, base: dict) -> str:
    full = dict(base)
    full.update({k: int(v) if isinstance(v, bool) else v for k, v in kw.items()})
    return "|".join(f"{k}={v}" for k, v in full.items())


def _sweep(op, names, settings, build, baseline, heap, args, roof, dims, base_knobs, rank, world):
    """Builds the plans (collectively), times them in turn, prints and records the table."""
    plans, skipped = {}, []
    for n in names:
        try:
            plans[n] = build(settings[n])
        except ValueError as e:          # a setting that does not tile this shape
            skipped.append(f"{n}: {e}")
    ok = G.all_gather_object(sorted(plans))
    common = [n for n in names if all(n in o for o in ok)]
    runners = {n: plans[n] for n in common}
    runners["nccl"] = baseline
    bar = ew.DeviceBarrier(heap)
    def check_all():
        bar.check()
        for n in common:
            try:
                plans[n].check()
            except Exception as e:  # noqa: BLE001
                raise RuntimeError(f"setting {n}: {type(e).__name__}: {e}") from e

    series = C.timed_interleaved(runners, args.iters, args.warmup, before=bar, flush=L2Flusher(), check=check_all)
    torch.cuda.synchronize()
    bar.check()
    for n in common:
        plans[n].check()
    mine = {n: C.stats_of(v).mean for n, v in series.items()}
    allr = G.all_gather_object(mine)
    if rank != 0:
        return
    M, N, K = dims
    worst = {n: max(r[n] for r in allr) for n in mine}
    nccl = worst.pop("nccl")
    print(f"# tune_fused {op} M={M} N={N} K={K} (per rank) world={world} iters={args.iters} [{C.device_line()}]")
    for s in skipped:
        print(f"# skipped {s}")
    print(f"{'setting':14s} | {'us (max over ranks)':>20s} | vs NCCL+cuBLAS | vs default | % roofline (burst cuBLAS rate)")
    csv = csvio.CsvAppender(args.csv, csvio.EXP3_FUSED_COLUMNS)
    dflt = worst.get("default", 0.0)
    for n in sorted(worst, key=worst.get):
        t = worst[n]
        print(f"{n:14s} | {t:20.1f} | {nccl / t:14.3f} | {dflt / t if dflt else 0:10.3f} | {100 * roof['roofline_burst_us'] / t:9.1f}"
              + ("   (timing only)" if n in TIMING_ONLY else ""))
        csv.row(m=M, n=N, k=K, world=world, rank=0, fused_us=mine[n], order="|".join(runners), iters=args.iters, max_over_ranks_us=t,
                nccl_cublas_us=nccl, speedup=nccl / t, roofline_us=roof["roofline_burst_us"], pct_roofline=100 * roof["roofline_burst_us"] / t,
                dtype="bf16", knobs=f"op={op}|setting={n}|" + knobs_string(settings[n], base_knobs))
    csv.close()
    print(f"nccl+cublas    | {nccl:20.1f}")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--ops", default="rs,ag")
    ap.add_argument("--m", type=C.parse_size, default=32768)
    ap.add_argument("--n", type=C.parse_size, default=8192, help="N of the GEMM+RS")
    ap.add_argument("--k", type=C.parse_size, default=0, help="GEMM+RS: K per rank")
    ap.add_argument("--k-global", type=C.parse_size, default=8192, help="GEMM+RS: global K, sharded (used when --k is 0)")
    ap.add_argument("--k-ag", type=C.parse_size, default=8192)
    ap.add_argument("--n-ag-global", type=C.parse_size, default=28672, help="AG+GEMM: global N, sharded over the ranks")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--only", default=None, help="comma list of setting names (default: all that fit the shape)")
    ap.add_argument("--csv", default=None)
    args = ap.parse_args(argv)
    rank, world, _ = G.init()
    dev = torch.device("cuda", torch.cuda.current_device())
    ops = C.split_csv(args.ops)
    only = C.split_csv(args.only) if args.only else None
    M = args.m

    if "rs" in ops:
        N = args.n
        K = args.k if args.k > 0 else args.k_global // world
        names = [n for n in RS_SETTINGS if only is None or n in only]
        mc_ok = world > 1 and bool(_native.lib().tcl_multicast_supported(torch.cuda.current_device()))
        per_plan = M * N * 2 + (M // world) * N * 2 + (1 << 20)
        n_nvls = sum(1 for n in names if RS_SETTINGS[n].get("transport") == "nvls")
        if not mc_ok:
            names = [n for n in names if RS_SETTINGS[n].get("transport") != "nvls"]
            n_nvls = 0
        heap = SymmetricHeap((len(names) - n_nvls) * per_plan + (64 << 20))
        mc_heap = SymmetricHeap(n_nvls * per_plan + (64 << 20), backend="vmm", multicast=True) if n_nvls else None
        try:
            A = torch.empty(M, K, dtype=torch.bfloat16, device=dev)
            Bt = torch.empty(N, K, dtype=torch.bfloat16, device=dev)
            ew.fill_normal_(A, seed=1000 + rank)
            ew.fill_normal_(Bt, seed=2000 + rank)
            D = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
            out_nccl = torch.empty(M // world, N, dtype=torch.bfloat16, device=dev) if world > 1 else None
            _sweep("gemm_rs", names, RS_SETTINGS, lambda kw: GemmRs(mc_heap if kw.get("transport") == "nvls" else heap, A, Bt, **kw),
                   lambda: base_ops.gemm_rs_baseline(A, Bt, out=out_nccl, full=D), heap, args,
                   roofline.gemm_rs_roofline_us(M, N, K, world), (M, N, K),
                   {"cta_group": 2, "transport": "p2p", "rs_chunks": 0, "group_m": 0, "num_ctas": 0, "st256": 0, "signal_batch": 0, "ablate": 0}, rank, world)
            torch.cuda.synchronize()
            G.host_barrier()
        except BaseException:
            if mc_heap is not None:
                mc_heap.release_multicast()
            raise
        if mc_heap is not None:
            mc_heap.close()
        heap.close()
        del A, Bt, D, out_nccl

    if "ag" in ops:
        K = args.k_ag
        N = args.n_ag_global // world
        names = [n for n in AG_SETTINGS if only is None or n in only]
        heap = SymmetricHeap(len(names) * (M * K * 2 + (2 << 20)) + (64 << 20))
        Bt = torch.empty(N, K, dtype=torch.bfloat16, device=dev)
        ew.fill_normal_(Bt, seed=3000 + rank, std=0.02)
        out = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
        shard = torch.empty(M // world, K, dtype=torch.bfloat16, device=dev)
        ew.fill_normal_(shard, seed=4000 + rank)
        gathered = torch.empty(M, K, dtype=torch.bfloat16, device=dev) if world > 1 else None
        out_b = torch.empty(M, N, dtype=torch.bfloat16, device=dev)

        def build(kw):
            op = AgGemm(heap, M, K, Bt, out=out, **kw)
            op.a_shard.copy_(shard)
            return op

        _sweep("ag_gemm", names, AG_SETTINGS, build, lambda: base_ops.ag_gemm_baseline(shard, Bt, gathered=gathered, out=out_b), heap, args,
               roofline.ag_gemm_roofline_us(M, N, K, world), (M, N, K),
               {"cta_group": 2, "transport": "pull", "gather_rows": 512, "item_rows": 1, "gather_warps": 0, "group_m": 0, "ablate": 0, "comm_enabled": 1}, rank, world)
        torch.cuda.synchronize()
        G.host_barrier()
        heap.close()
    G.shutdown()
    return 0


if __name__ == "__main__":
    sys.exit(main())
