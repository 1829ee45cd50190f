"""End-to-end tensor-parallel MLP block: AG+GEMM(gate|up) -> SiLU*mul -> GEMM+RS(down), forward only.

Default shape: Llama-3-70B block, hidden 8192, ffn 28672, 16384 tokens, bf16, weights N(0, 0.02).
Compared against the same block on NCCL + cuBLAS (all_gather -> matmul -> SiLU*mul (same fused
kernel) -> matmul -> reduce_scatter), one iteration of each in turn, device-timed, max over ranks.
The reference has no end-to-end model; this is the pipeline named by the benchmark configuration.
"""
from __future__ import annotations

import argparse
import sys

import torch
import torch.distributed as dist

from ..models.tp_mlp import TpMlp, heap_bytes
from ..ops import elementwise as ew
from ..parallel import group as G
from ..parallel.heap import SymmetricHeap
from ..utils import csvio, roofline
from ..utils.timing import L2Flusher
from . import _common as C


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--tokens", type=C.parse_size, default=16384)
    ap.add_argument("--hidden", type=C.parse_size, default=8192)
    ap.add_argument("--ffn", type=C.parse_size, default=28672)
    ap.add_argument("--iters", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--cta-group", type=int, default=2)
    ap.add_argument("--gather-rows", type=int, default=512)
    ap.add_argument("--no-fuse-silu", action="store_true", help="keep SiLU*mul as its own kernel")
    ap.add_argument("--graph", action="store_true", help="also time the block replayed from a CUDA graph (call numbers kept in device memory)")
    ap.add_argument("--verify", action="store_true")
    ap.add_argument("--csv", default=None)
    args = ap.parse_args(argv)
    rank, world, _ = G.init()
    T, H, F = args.tokens, args.hidden, args.ffn
    f = F // world
    dev = torch.device("cuda", torch.cuda.current_device())
    heap = SymmetricHeap(heap_bytes(T, H, F, world) + (64 << 20))
    mlp = TpMlp(heap, T, H, F, cta_group=args.cta_group, gather_rows=args.gather_rows, fuse_silu=not args.no_fuse_silu, graph=args.graph)
    x = torch.empty(T // world, H, dtype=torch.bfloat16, device=dev)
    ew.fill_normal_(x, seed=77 + rank)
    mlp.x_shard.copy_(x)
    bar = ew.DeviceBarrier(heap)
    flush = L2Flusher()
    w_gu_plain = mlp.gate_up_plain()      # the baseline uses the plain gate|up layout and the stand-alone SiLU*mul kernel
    # baseline buffers
    xg = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
    hb = torch.empty(T, 2 * f, dtype=torch.bfloat16, device=dev)
    ab = torch.empty(T, f, dtype=torch.bfloat16, device=dev)
    yb_full = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
    yb = torch.empty(T // world, H, dtype=torch.bfloat16, device=dev)

    def baseline():
        if world > 1:
            dist.all_gather_into_tensor(xg, x)
            src = xg
        else:
            src = x
        torch.matmul(src, w_gu_plain.t(), out=hb)
        ew.silu_mul(hb, ab)
        torch.matmul(ab, mlp.w_down.t(), out=yb_full)
        if world > 1:
            dist.reduce_scatter_tensor(yb, yb_full)
            return yb
        return yb_full

    torch.cuda.synchronize()
    G.host_barrier()
    max_rel = float("nan")
    if args.verify:
        y = mlp()
        mlp.check()
        ref = baseline()
        torch.cuda.synchronize()
        max_rel = ((y.float() - ref.float()).abs() / (ref.float().abs() + 1)).max().item()
    variants = {"fused": mlp, "nccl": baseline}
    if args.graph:
        mlp.capture()
        variants["graph"] = mlp.replay
    ser = C.timed_interleaved(variants, args.iters, args.warmup, before=bar, flush=flush)
    mlp.check()
    # stage breakdown of the fused path
    parts = C.timed_interleaved({"ag": mlp.ag, "silu": lambda: ew.silu_mul(hb, ab), "rs": mlp.rs},
                                max(5, args.iters // 3), 2, before=bar, flush=flush)
    mine = {k: C.stats_of(v) for k, v in {**ser, **parts}.items()}
    allr = G.all_gather_object({k: (s.mean, s.p95) for k, s in mine.items()} | {"rel": max_rel})
    if rank == 0:
        mx = lambda k, i=0: max(r[k][i] for r in allr)
        fused, nccl = mx("fused"), mx("nccl")
        r_ag = roofline.ag_gemm_roofline_us(T, 2 * f, H, world)
        r_rs = roofline.gemm_rs_roofline_us(T, H, f, world)
        roof = r_ag["roofline_burst_us"] + r_rs["roofline_burst_us"] + T * f * 2 * 3 / (roofline.peaks()["hbm_gbs"] * 1e9) * 1e6
        rel = max(r["rel"] for r in allr) if args.verify else float("nan")
        print(f"# mlp_e2e tokens={T} hidden={H} ffn={F} tp={world} cta_group={args.cta_group} [{C.device_line()}]")
        print(f"fused {fused:.1f} us (p95 {mx('fused', 1):.1f}) = AG+GEMM{"+SiLU*mul" if mlp.fuse_silu else ""} {mx('ag'):.1f} + GEMM+RS {mx('rs'):.1f} (stages timed alone; stand-alone SiLU*mul kernel: {mx('silu'):.1f})")
        print(f"nccl+cublas {nccl:.1f} us | speedup {nccl / fused:.3f}x | roofline {roof:.1f} us ({100 * roof / fused:.1f} % of {r_ag['peaks']} peaks, burst cuBLAS rate) | max rel diff {rel:.3g}")
        if args.graph:
            print(f"replayed from a CUDA graph: {mx('graph'):.1f} us (p95 {mx('graph', 1):.1f}), {fused / mx('graph'):.3f}x of the eager launches")
        csv = csvio.CsvAppender(args.csv, csvio.MLP_E2E_COLUMNS)
        csv.row(tokens=T, hidden=H, ffn=F, world=world, fused_us=fused, fused_p95=mx("fused", 1), ag_us=mx("ag"), silu_us=mx("silu"),
                rs_us=mx("rs"), nccl_cublas_us=nccl, speedup=nccl / fused, roofline_us=roof, pct_roofline=100 * roof / fused,
                max_rel_diff=rel, iters=args.iters, dtype="bf16", graph_us=(mx("graph") if args.graph else ""))
        csv.close()
    torch.cuda.synchronize()
    G.host_barrier()
    heap.close()
    G.shutdown()
    return 0


if __name__ == "__main__":
    sys.exit(main())
