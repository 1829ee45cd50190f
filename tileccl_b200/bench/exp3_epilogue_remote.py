"""exp3 (v1): what it costs to point the GEMM's epilogue at a peer.

The same tcgen05 GEMM, with only its output pointer changed:

    local          D in this GPU's memory (the control)
    remote         all of D in one peer's memory
    scatter-local  D cut into `world` row segments that all stay local (control for `scatter`)
    scatter        row segment s goes to rank s's memory (the reduce-scatter write pattern)

The default epilogue is tcgen05.ld -> bf16 -> shared-memory transpose -> 16-byte st.global
(``st16`` in the `epi` column); ``--epi st16,st256,tma`` adds the 32-byte store form and the TMA-store
form (cp.async.bulk.tensor from the same staging buffer), the counterparts of the reference's
direct-store and TMA-store epilogues.  slowdown = time / time of `local` with the same epilogue.
Verification is bit-wise against the local result.

Reference parity: comm_comp/exp3_epilogue_remote.cu (modes :147-156,311-328, timing :185-204,
verify :366-395, CSV :255-257,403-406).
"""
from __future__ import annotations

import argparse
import sys

import torch

from ..ops import elementwise as ew
from ..ops.gemm import GemmPlan
from ..parallel import group as G
from ..parallel.heap import SymmetricHeap
from ..utils import csvio
from ..utils.timing import L2Flusher
from . import _common as C


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--sizes", default="8192", help="comma list of N or MxNxK")
    ap.add_argument("--modes", default="local,remote,scatter-local,scatter")
    ap.add_argument("--peer", type=int, default=-1, help="rank that receives `remote` (default: next rank)")
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--cta-group", type=int, default=2)
    ap.add_argument("--epi", default="st16", help="comma list of epilogues: st16 (16-byte st.global), st256 (32-byte st.global), tma (TMA store)")
    ap.add_argument("--verify", action="store_true")
    ap.add_argument("--csv", default=None)
    args = ap.parse_args(argv)
    rank, world, _ = G.init()
    dev = torch.device("cuda", torch.cuda.current_device())
    shapes = [C.parse_shape(s) for s in C.split_csv(args.sizes)]
    modes = C.split_csv(args.modes)
    epis = C.split_csv(args.epi)
    for e in epis:
        if e not in ("st16", "st256", "tma"):
            ap.error(f"unknown epilogue {e!r}")
    peer = args.peer if args.peer >= 0 else (rank + 1) % world
    max_mn = max(m * n for m, n, _ in shapes)
    heap = SymmetricHeap(2 * max_mn * 2 + (64 << 20))
    bar = ew.DeviceBarrier(heap)
    flush = L2Flusher()
    csv = csvio.CsvAppender(args.csv if rank == 0 else None, csvio.EXP3_EPILOGUE_COLUMNS)
    if rank == 0:
        print(f"# exp3 epilogue remote write, world={world}, peer of rank 0 = {peer}, cta_group={args.cta_group} [{C.device_line()}]")
        print("      shape        mode        | iter us    p95 |  TF/s | slowdown | D write GB/s | verify")
    for (M, N, K) in shapes:
        heap.reset()
        bar = ew.DeviceBarrier(heap)
        D = heap.empty((M, N), torch.bfloat16)          # symmetric: every rank has one, peers can write it
        A = torch.empty(M, K, dtype=torch.bfloat16, device=dev)
        Bt = torch.empty(N, K, dtype=torch.bfloat16, device=dev)
        # With --verify every rank computes the same product, so whichever rank wrote a row of a
        # shared destination last, its bits are known.
        ew.fill_normal_(A, seed=31 + (0 if args.verify else rank))
        ew.fill_normal_(Bt, seed=41 + (0 if args.verify else rank))
        seg = M // world if world > 1 and M % (world * 128 * args.cta_group) == 0 else M
        nseg = M // seg
        plans = {}          # (mode, epilogue) -> plan
        for epi in epis:
            kw = dict(out=D, cta_group=args.cta_group, store=epi)
            for mode in modes:
                if mode == "local":
                    plans[mode, epi] = GemmPlan(A, Bt, **kw)
                elif mode == "remote" and world > 1:
                    plans[mode, epi] = GemmPlan(A, Bt, dst_ptrs=[heap.peer_ptr(D, peer)], seg_rows=M, **kw)
                elif mode == "scatter-local" and nseg > 1:
                    plans[mode, epi] = GemmPlan(A, Bt, seg_rows=seg, dst_ptrs=[D.data_ptr() + s * seg * N * 2 for s in range(nseg)], **kw)
                elif mode == "scatter" and nseg > 1:
                    # segment s lands in rank s's D, in the row block of this (source) rank's ... same rows
                    plans[mode, epi] = GemmPlan(A, Bt, seg_rows=seg, dst_ptrs=[heap.peer_ptr(D, s) + s * seg * N * 2 for s in range(nseg)], **kw)
        series = C.timed_interleaved(plans, args.iters, args.warmup, before=bar, flush=flush)
        for p in plans.values():
            p.check()
        verify = {}
        if args.verify and ("local", epis[0]) in plans:
            plans["local", epis[0]]()
            torch.cuda.synchronize()
            ref = D.clone()
            for (mode, epi), p in plans.items():
                if (mode, epi) == ("local", epis[0]):
                    continue
                torch.cuda.synchronize()
                G.host_barrier()
                D.zero_()
                torch.cuda.synchronize()
                G.host_barrier()
                p()
                torch.cuda.synchronize()
                G.host_barrier()
                if mode == "remote":
                    # my result as it landed in the peer's buffer
                    got = heap.peer_tensor(D, peer)
                    verify[mode, epi] = "ok" if torch.equal(got, ref) else "FAIL"
                elif mode == "scatter":
                    # every rank wrote its segment `rank` of rows into my D: those rows must be the reference's
                    mine = slice(rank * seg, (rank + 1) * seg)
                    verify[mode, epi] = "ok" if torch.equal(D[mine], ref[mine]) else "FAIL"
                else:
                    verify[mode, epi] = "ok" if torch.equal(D, ref) else "FAIL"
                G.host_barrier()
        stats = {m: C.stats_of(v) for m, v in series.items()}
        allr = G.all_gather_object({m: (s.mean, s.p95) for m, s in stats.items()})
        if rank == 0:
            flop = 2.0 * M * N * K
            for (mode, epi) in plans:
                # slow-down against the local run with the same epilogue, as in the reference
                base = max(r["local", epi][0] for r in allr) if ("local", epi) in stats else 0.0
                mean = max(r[mode, epi][0] for r in allr)
                p95 = max(r[mode, epi][1] for r in allr)
                slow = mean / base if base > 0 else 0.0
                gbps = M * N * 2 / (mean * 1e-6) / 1e9
                ver = verify.get((mode, epi), "-")
                name = mode if len(epis) == 1 else f"{mode}/{epi}"
                print(f" {M:6d}x{N:5d}x{K:5d} {name:14s} | {mean:8.1f} {p95:6.1f} | {flop / mean / 1e6:5.0f} | {slow:8.3f} | {gbps:12.1f} | {ver}")
                csv.row(m=M, n=N, k=K, epi=epi, mode=mode, peer=peer, iter_us=mean, iter_p95=p95, slowdown=slow,
                        tflops=flop / mean / 1e6, d_write_gbps=gbps, verify=ver, max_over_ranks_us=mean, dtype="bf16")
    csv.close()
    torch.cuda.synchronize()
    G.host_barrier()
    heap.close()
    G.shutdown()
    return 0


if __name__ == "__main__":
    sys.exit(main())
