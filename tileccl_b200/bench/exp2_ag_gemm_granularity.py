"""exp2: all-gather -> GEMM at configurable gather granularity.

Every rank holds a row shard of A and a local B; the GEMM needs all of A.
Compared, per granularity (rows per gather tile, i.e. S = shard rows / rows
chunks per shard):

    fused  one kernel: gather warps pull peer rows with P2P loads, the TMA
           producer starts on a row block when its counter says it landed
    ce     the reference's design: one copy-engine peer copy + event per chunk
           on a high-priority stream, the compute stream waits on the event and
           launches a pre-built segment GEMM (local shard first)
    nccl   ncclAllGather, then one cuBLAS GEMM (the baseline)

with t_full (one GEMM on pre-gathered A), t_seg (the same segmentation with no
communication), t_comm (the transfers alone), t_ovl (the dependent pipeline),
seg_eff = t_full / t_seg, overlap_eff = max(t_seg, t_comm) / t_ovl.

Reference parity: comm_comp/exp2_ag_gemm_granularity.cu (flags :72-88, pipeline
:168-300, metrics :553-559, verify with a 0x55 scrub :511-533, CSV :446-448).
"""
from __future__ import annotations

import argparse
import ctypes as C_
import sys

import torch

from .. import _native
from ..ops import baseline as base_ops
from ..ops import elementwise as ew
from ..ops.ag_gemm import AgGemm
from ..ops.gemm import GemmPlan
from ..parallel import group as G
from ..parallel.heap import SymmetricHeap
from ..utils import csvio, roofline
from ..utils.timing import L2Flusher
from . import _common as C


def build_parser():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--m", type=C.parse_size, default=32768, help="gathered rows")
    ap.add_argument("--k", type=C.parse_size, default=8192)
    ap.add_argument("--n", type=C.parse_size, default=0, help="local N (columns of this rank's B)")
    ap.add_argument("--n-global", type=C.parse_size, default=28672, help="global N, sharded (used when --n is 0)")
    ap.add_argument("--gather-rows", default="128,512,2048,4096")
    ap.add_argument("--modes", default="fused,ce,nccl")
    ap.add_argument("--transport", default="pull", choices=["push", "pull"], help="fused mode: gather warps store the own shard to every peer (push) or load the peers' shards (pull)")
    ap.add_argument("--iters", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--cta-group", type=int, default=2)
    ap.add_argument("--ablate", type=int, default=0, help="timing-only knob of the fused mode: 4 = the TMA producer does not wait for gathered rows")
    ap.add_argument("--item-rows", type=int, default=1, help="rows per gather work item of the fused mode")
    ap.add_argument("--verify", action="store_true")
    ap.add_argument("--csv", default=None)
    return ap


def gather_tiles(asked, seg: int) -> tuple[list[int], list[int]]:
    """(tiles to run, tiles skipped) for a segment of ``seg`` rows.  A tile larger than the segment becomes the
    segment.  A CTA's TMA producer waits for the 128 rows it loads itself, also in a CTA pair, so 128 rows is the
    finest tile; a tile must divide the segment."""
    want = sorted(set(min(int(g), seg) for g in asked))
    run = [g for g in want if g == seg or (seg % g == 0 and g % 128 == 0)]
    return run, [g for g in want if g not in run]


class CePipeline:
    """Segmented launch + copy-engine transfers (the reference's exp2 design)."""

    def __init__(self, heap, a_full, Bt, out, chunk_rows, cta_group):
        self.heap, self.a_full, self.out = heap, a_full, out
        self.lib = _native.lib()
        world, rank = heap.world, heap.rank
        M, K = a_full.shape
        seg = M // world
        self.chunk_rows = chunk_rows
        self.comm = torch.cuda.Stream(priority=-1)
        if chunk_rows % (128 * cta_group) != 0:
            cta_group = 1        # a 128-row chunk is one single-CTA tile high
        self.chunks = []     # (row0, src_ptr, dst_ptr, bytes, src_dev, event, plan)
        order = [(rank + s) % world for s in range(world)]
        for s in order:
            for c in range(seg // chunk_rows):
                row0 = s * seg + c * chunk_rows
                rows = a_full[row0:row0 + chunk_rows]
                plan = GemmPlan(rows, Bt, out=out[row0:row0 + chunk_rows], cta_group=cta_group)
                src = heap.peer_ptr(rows, s)
                ev = torch.cuda.Event() if s != rank else None
                self.chunks.append((s, src, rows.data_ptr(), rows.numel() * 2, ev, plan))
        self.gate = torch.cuda.Event()

    def copies(self):
        dev = torch.cuda.current_device()
        for s, src, dst, nbytes, ev, _ in self.chunks:
            if ev is None:
                continue
            _native.check(self.lib.tcl_memcpy_async(C_.c_void_p(dst), C_.c_void_p(src), nbytes,
                                                    C_.c_void_p(self.comm.cuda_stream)), "peer copy")
            ev.record(self.comm)

    def run(self, comm: bool = True, compute: bool = True):
        cur = torch.cuda.current_stream()
        if comm:
            self.gate.record(cur)
            self.comm.wait_event(self.gate)     # transfers of this iteration start when the previous one is done
            self.copies()
        if compute:
            for s, _, _, _, ev, plan in self.chunks:
                if comm and ev is not None:
                    cur.wait_event(ev)
                plan()
        elif comm:
            cur.wait_stream(self.comm)


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    rank, world, _ = G.init()
    M, K = args.m, args.k
    N = args.n if args.n > 0 else args.n_global // world
    seg = M // world
    dev = torch.device("cuda", torch.cuda.current_device())
    modes = C.split_csv(args.modes)
    grains, skipped = gather_tiles(C.split_csv(args.gather_rows), seg)
    if rank == 0:
        for g in skipped:
            print(f"# gather tile {g} rows skipped: it must divide the {seg}-row segment and be a multiple of 128")
    heap = SymmetricHeap((3 * len(grains) + 1) * (M * K * 2 + (8 << 20)) + (64 << 20))
    Bt = torch.empty(N, K, dtype=torch.bfloat16, device=dev)
    ew.fill_normal_(Bt, seed=500 + rank, std=0.02)
    shard = torch.empty(seg, K, dtype=torch.bfloat16, device=dev)
    ew.fill_normal_(shard, seed=600 + rank)
    out = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
    out_ref = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
    bar = ew.DeviceBarrier(heap)
    flush = L2Flusher()

    # t_full: one GEMM on a pre-gathered A (also the verification reference).
    gathered = torch.empty(M, K, dtype=torch.bfloat16, device=dev)
    if world > 1:
        torch.distributed.all_gather_into_tensor(gathered, shard)
    else:
        gathered.copy_(shard)
    full_plan = GemmPlan(gathered, Bt, out=out_ref, cta_group=args.cta_group)
    g2 = torch.empty(M, K, dtype=torch.bfloat16, device=dev)
    common = {"full": full_plan}
    if "nccl" in modes:
        common["nccl"] = lambda: base_ops.ag_gemm_baseline(shard, Bt, gathered=g2, out=out)
    full_plan()
    torch.cuda.synchronize()
    t_full_all, t_nccl_all = [], []

    rows_out = []
    for g in grains:
        S = seg // g
        for mode in [m for m in modes if m in ("fused", "ce")]:
            if mode == "fused":
                op = AgGemm(heap, M, K, Bt, cta_group=args.cta_group, gather_rows=g, out=out, ablate=args.ablate, transport=args.transport, item_rows=args.item_rows)
                ctrl = None
                a_full = op.a_full
                op.a_shard.copy_(shard)
                run_ovl = lambda: op()
                # t_seg: same kernel, same tile order, no waiting (data already gathered)
                seg_op = AgGemm(heap, M, K, Bt, cta_group=args.cta_group, gather_rows=g, out=out, comm_enabled=False, transport=args.transport)
                seg_op.a_full.copy_(gathered)
                run_seg = lambda: seg_op()
                run_comm = None
            else:
                a_full = heap.empty((M, K), torch.bfloat16)
                a_full[rank * seg:(rank + 1) * seg].copy_(shard)
                pipe = CePipeline(heap, a_full, Bt, out, g, args.cta_group)
                run_ovl = lambda: pipe.run(True, True)
                run_seg = lambda: pipe.run(False, True)
                run_comm = lambda: pipe.run(True, False)
            torch.cuda.synchronize()
            G.host_barrier()
            verify = "-"
            if args.verify:
                # scrub the peers' rows so that a broken dependency shows up as garbage
                scrub = a_full.view(-1).view(torch.uint8)
                scrub[: rank * seg * K * 2].fill_(0x55)
                scrub[(rank + 1) * seg * K * 2:].fill_(0x55)
                torch.cuda.synchronize()
                G.host_barrier()
                out.zero_()
                run_ovl()
                torch.cuda.synchronize()
                G.host_barrier()
                verify = "ok" if torch.equal(out, out_ref) else "FAIL"
            if mode == "ce":
                a_full.copy_(gathered)
            # One iteration of every variant in turn: same clocks for all of them.
            fns = dict(common)
            fns["seg"] = run_seg
            fns["ovl"] = run_ovl
            ser = C.timed_interleaved(fns, args.iters, args.warmup, before=bar, flush=flush)
            t_seg, t_ovl = C.stats_of(ser["seg"]), C.stats_of(ser["ovl"])
            t_full_all += ser["full"]
            t_nccl_all += ser.get("nccl", [])
            t_comm = C.stats_of(C.timed_series(run_comm, max(5, args.iters // 3), 2, before=bar)) if run_comm else C.stats_of([])
            if mode == "fused":
                op.check()
                seg_op.check()
            rows_out.append(dict(mode=mode, S=S, chunk_rows=g, t_seg=t_seg.mean, t_ovl=t_ovl.mean, t_comm=t_comm.mean, verify=verify,
                                 t_full=C.stats_of(ser["full"]).mean, t_nccl=C.stats_of(ser.get("nccl", [])).mean))
    bar.check()

    mine = {"rank": rank, "t_full": C.stats_of(t_full_all).mean, "t_nccl": C.stats_of(t_nccl_all).mean, "rows": rows_out}
    allr = G.all_gather_object(mine)
    if rank == 0:
        flop = 2.0 * M * N * K
        roof = roofline.ag_gemm_roofline_us(M, N, K, world)
        tf = max(r["t_full"] for r in allr)
        tn = max(r["t_nccl"] for r in allr)
        print(f"# exp2 AG+GEMM  M={M} N/rank={N} K={K} world={world} cta_group={args.cta_group} iters={args.iters} [{C.device_line()}]")
        print(f"t_full {tf:.1f} us ({flop / tf / 1e6:.0f} TF/s) | nccl+cublas {tn:.1f} us | roofline {roof['roofline_burst_us']:.1f} us  (max over ranks)")
        print(" mode      S  chunk_rows chunk_MiB |  t_seg us  t_comm us   t_ovl us | seg_eff ovl_eff  bubble | e2e TF/s  speedup  %roof | verify")
        csv = csvio.CsvAppender(args.csv, csvio.EXP2_COLUMNS)
        for i, row in enumerate(rows_out):
            ts = max(r["rows"][i]["t_seg"] for r in allr)
            to = max(r["rows"][i]["t_ovl"] for r in allr)
            tc = max(r["rows"][i]["t_comm"] for r in allr)
            tf_i = max(r["rows"][i]["t_full"] for r in allr)
            tn_i = max(r["rows"][i]["t_nccl"] for r in allr)
            ver = "FAIL" if any(r["rows"][i]["verify"] == "FAIL" for r in allr) else row["verify"]
            mib = row["chunk_rows"] * K * 2 / 2**20
            seg_eff = tf_i / ts if ts > 0 else 0.0
            ovl_eff = max(ts, tc) / to if to > 0 else 0.0
            bubble = (to - max(ts, tc)) / to if to > 0 else 0.0
            gbps = (world - 1) / world * M * K * 2 / (tc * 1e-6) / 1e9 if tc > 0 else 0.0
            print(f" {row['mode']:6s} {row['S']:5d} {row['chunk_rows']:10d} {mib:9.1f} | {ts:9.1f} {tc:10.1f} {to:10.1f} | "
                  f"{seg_eff:7.3f} {ovl_eff:7.3f} {bubble:7.3f} | {flop / to / 1e6:8.0f} {tn_i / to if tn_i else 0:8.3f} "
                  f"{100 * roof['roofline_burst_us'] / to:6.1f} | {ver}")
            csv.row(m=M, n=N, k=K, world=world, S=row["S"], chunk_rows=row["chunk_rows"], chunk_mib=mib, mode=row["mode"],
                    streams=1, t_full_us=tf_i, t_seg_us=ts, t_comm_us=tc, t_ovl_us=to, seg_eff=seg_eff, comm_gbps=gbps,
                    overlap_eff=ovl_eff, e2e_tflops=flop / to / 1e6, verify=ver, max_over_ranks_us=to, nccl_cublas_us=tn_i,
                    speedup=(tn_i / to if tn_i else 0.0), roofline_us=roof["roofline_burst_us"],
                    pct_roofline=100 * roof["roofline_burst_us"] / to, dtype="bf16")
        csv.close()
    torch.cuda.synchronize()
    G.host_barrier()
    heap.close()
    G.shutdown()
    return 0


if __name__ == "__main__":
    sys.exit(main())
