"""exp3 (v2): fused GEMM + reduce-scatter, three variants per rank.

    base   plain tcgen05 GEMM into a local [M, N] buffer
    ctrl   the fused kernel with communication off: same tile order, stores local
    fused  the fused kernel: epilogue pushes partial tiles to their owners,
           reduce warps sum them

and the library baseline ``nccl`` = cuBLAS GEMM + ncclReduceScatter.  Derived:
struct = ctrl/base, comm = fused/ctrl, total = fused/base, speedup =
nccl/fused (max over ranks), % of roofline.  A device barrier precedes every
timed iteration; times are per-iteration CUDA events.

Run under torchrun, one process per GPU:
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 \\
        -m tileccl_b200.bench.exp3_gemm_rs_fused --m 32768 --n 8192 --k 1024 --verify --csv out.csv

Reference parity: comm_comp/exp3_gemm_rs_fused.cu (flags :108-131, variants
:423-442, timing :278-331, verify :519-545, CSV :574-634).  ``--k`` is K per
rank as in the reference; ``--k-global`` shards a global K over the ranks.
"""
from __future__ import annotations

import argparse
import sys

import torch

from ..ops import baseline as base_ops
from ..ops import elementwise as ew
from ..ops.gemm import GemmPlan
from ..ops.gemm_rs import GemmRs
from ..parallel import group as G
from ..parallel.heap import SymmetricHeap
from ..utils import csvio, roofline
from ..utils.timing import L2Flusher
from . import _common as C


def build_parser():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--m", type=C.parse_size, default=8192)
    ap.add_argument("--n", type=C.parse_size, default=8192)
    ap.add_argument("--k", type=C.parse_size, default=0, help="K per rank")
    ap.add_argument("--k-global", type=C.parse_size, default=8192, help="global K, sharded (used when --k is 0)")
    ap.add_argument("--iters", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--order", default="base,ctrl,fused,nccl")
    ap.add_argument("--cta-group", type=int, default=2)
    ap.add_argument("--rs-chunks", type=int, default=0)
    ap.add_argument("--group-m", type=int, default=0)
    ap.add_argument("--num-ctas", type=int, default=0, help="CTAs of the fused and ctrl variants (0 = one per SM)")
    ap.add_argument("--ablate", type=int, default=0, help="timing-only knobs of the fused variant: 1 = no reduce warps, 2 or 3 = no tile signals and no reduce warps")
    ap.add_argument("--transport", default="p2p", choices=["p2p", "nvls"], help="p2p: epilogue pushes partial tiles to the owner; nvls: partials stay local, the owner pulls sums with multimem.ld_reduce")
    ap.add_argument("--st256", action="store_true", help="fused variant: 32-byte epilogue stores (st.global.v8.b32) instead of 16-byte ones")
    ap.add_argument("--verify", action="store_true")
    ap.add_argument("--no-flush", action="store_true", help="do not flush L2 between iterations")
    ap.add_argument("--csv", default=None)
    ap.add_argument("--dump-iters", default=None, help="prefix of per-rank per-iteration CSV files")
    return ap


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    rank, world, _ = G.init()
    M, N = args.m, args.n
    K = args.k if args.k > 0 else args.k_global // world
    dev = torch.device("cuda", torch.cuda.current_device())
    # A rank's segment must hold whole tiles: 256 rows for CTA pairs, 128 for single CTAs.
    if M % world == 0 and (M // world) % (128 * args.cta_group) and (M // world) % 128 == 0:
        if rank == 0:
            print(f"# M / world = {M // world} rows is not a multiple of {128 * args.cta_group}: using --cta-group 1")
        args.cta_group = 1
    if M % world or (M // world) % 128 or N % 256 or K % 8:
        if rank == 0:
            print(f"# skipped: M={M} N={N} K/rank={K} world={world} does not tile (M/world % 128, N % 256, K % 8)")
        G.shutdown()
        return 0
    nvls = args.transport == "nvls" and world > 1
    heap = SymmetricHeap(2 * (M * N * 2 + (M // world) * N * 2) + (64 << 20), backend="vmm" if nvls else "ipc", multicast=nvls)
    try:
        A = torch.empty(M, K, dtype=torch.bfloat16, device=dev)
        Bt = torch.empty(N, K, dtype=torch.bfloat16, device=dev)
        ew.fill_normal_(A, seed=1000 + rank)
        ew.fill_normal_(Bt, seed=2000 + rank)
        D = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
        plain = GemmPlan(A, Bt, out=D, cta_group=args.cta_group)
        fused = GemmRs(heap, A, Bt, cta_group=args.cta_group, rs_chunks=args.rs_chunks, group_m=args.group_m, num_ctas=args.num_ctas,
                       ablate=args.ablate, transport=args.transport, st256=args.st256)
        ctrl = GemmRs(heap, A, Bt, cta_group=args.cta_group, rs_chunks=args.rs_chunks, group_m=args.group_m, num_ctas=args.num_ctas,
                      comm_enabled=False)
        bar = ew.DeviceBarrier(heap)
        out_nccl = torch.empty(M // world, N, dtype=torch.bfloat16, device=dev) if world > 1 else None
        flush = None if args.no_flush else L2Flusher()

        runners = {
            "base": lambda: plain(),
            "fused": lambda: fused(),
            "nccl": lambda: base_ops.gemm_rs_baseline(A, Bt, out=out_nccl, full=D),
        }
        if ctrl is not None:
            runners["ctrl"] = lambda: ctrl()
        order = [o for o in C.split_csv(args.order) if o in runners]
        # One iteration of every variant in turn, so that all see the same clocks.
        series = C.timed_interleaved({n: runners[n] for n in order}, args.iters, args.warmup, before=bar, flush=flush, rotate=False)   # --order is the experiment
        torch.cuda.synchronize()
        bar.check()
        fused.check()
        plain.check()
        if ctrl is not None:
            ctrl.check()

        max_rel = float("nan")
        if args.verify:
            fused()
            ref = base_ops.gemm_rs_baseline(A, Bt, out=out_nccl, full=D).float() if world > 1 else None
            if world == 1:
                plain()
                ref = D.float()
            torch.cuda.synchronize()
            max_rel = ((fused.out.float() - ref).abs() / (ref.abs() + 1)).max().item()

        st = {k: C.stats_of(v) for k, v in series.items()}
        zero = C.stats_of([])
        b, c, f, n = (st.get(k, zero) for k in ("base", "ctrl", "fused", "nccl"))
        mine = {"rank": rank, "b": b, "c": c, "f": f, "n": n, "max_rel": max_rel}
        allr = G.all_gather_object(mine)

        if args.dump_iters:
            d = csvio.CsvAppender(f"{args.dump_iters}.rank{rank}.csv", csvio.EXP3_ITER_COLUMNS)
            for name, v in series.items():
                for i, us in enumerate(v):
                    d.row(m=M, n=N, k=K, world=world, rank=rank, variant=name, iter=i, us=us)
            d.close()

        if rank == 0:
            flop = 2.0 * M * N * K
            roof = roofline.gemm_rs_roofline_us(M, N, K, world)
            ctrl_max = max(r["c"].mean for r in allr)
            fused_max = max(r["f"].mean for r in allr)
            nccl_max = max(r["n"].mean for r in allr)
            print(f"# exp3 fused GEMM+RS  M={M} N={N} K/rank={K} world={world} cta_group={args.cta_group} "
                  f"transport={fused.transport} iters={args.iters}  [{C.device_line()}]")
            print("rank |  base us   TF/s |  ctrl us | fused us   TF/s | struct   comm  total | push GB/s | nccl+cublas us | verify")
            csv = csvio.CsvAppender(args.csv, csvio.EXP3_FUSED_COLUMNS)
            for r in allr:
                b, c, f, n = r["b"], r["c"], r["f"], r["n"]
                sd_struct = c.mean / b.mean if b.mean > 0 and c.mean > 0 else 0.0
                sd_comm = f.mean / c.mean if c.mean > 0 else 0.0
                sd_total = f.mean / b.mean if b.mean > 0 else 0.0
                gbps = (world - 1) / world * M * N * 2 / (f.mean * 1e-6) / 1e9 if f.mean > 0 else 0.0
                ver = "-" if not args.verify else ("ok" if r["max_rel"] <= 0.5 else "FAIL") + f" (rel {r['max_rel']:.3g})"
                print(f"{r['rank']:4d} | {b.mean:9.1f} {flop / max(b.mean, 1e-9) / 1e6:6.0f} | {c.mean:8.1f} | {f.mean:8.1f} "
                      f"{flop / max(f.mean, 1e-9) / 1e6:6.0f} | {sd_struct:6.3f} {sd_comm:6.3f} {sd_total:6.3f} | {gbps:9.1f} | "
                      f"{n.mean:14.1f} | {ver}")
                csv.row(m=M, n=N, k=K, world=world, rank=r["rank"], base_us=b.mean, base_p95=b.p95, ctrl_us=c.mean,
                        ctrl_p95=c.p95, fused_us=f.mean, fused_p95=f.p95, struct_sd=sd_struct, comm_sd=sd_comm,
                        total_sd=sd_total, pull_gbps=gbps, max_rel_diff=r["max_rel"], base_p50=b.p50, ctrl_p50=c.p50,
                        fused_p50=f.p50, base_min=b.min, ctrl_min=c.min, fused_min=f.min,
                        comm_sd_p50=(f.p50 / c.p50 if c.p50 > 0 else 0.0),
                        comm_sd_skew=(f.mean / ctrl_max if ctrl_max > 0 else 0.0), comm_abs_us=f.mean - c.mean,
                        order="|".join(order), iters=args.iters, max_over_ranks_us=fused_max, nccl_cublas_us=nccl_max,
                        speedup=(nccl_max / fused_max if fused_max > 0 else 0.0), roofline_us=roof["roofline_burst_us"],
                        pct_roofline=(100.0 * roof["roofline_burst_us"] / fused_max if fused_max > 0 else 0.0), dtype="bf16",
                        knobs=f"cta_group={args.cta_group}|transport={fused.transport}|rs_chunks={args.rs_chunks}|group_m={args.group_m}|"
                              f"num_ctas={args.num_ctas}|st256={int(args.st256)}|ablate={args.ablate}")
            csv.close()
            if fused_max > 0:
                print(f"max over ranks: fused {fused_max:.1f} us | nccl+cublas {nccl_max:.1f} us | speedup "
                      f"{nccl_max / fused_max if nccl_max else 0:.3f}x | roofline {roof['roofline_burst_us']:.1f} us "
                      f"({100 * roof['roofline_burst_us'] / fused_max:.1f} % of {roof['peaks']} peaks, burst cuBLAS rate)")
    except BaseException:
        # no rank may leave with its memory still bound to a multicast object: unbind locally, then re-raise
        heap.release_multicast()
        raise
    torch.cuda.synchronize()
    G.host_barrier()
    heap.close()
    G.shutdown()
    return 0


if __name__ == "__main__":
    sys.exit(main())
