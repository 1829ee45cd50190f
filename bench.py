#!/usr/bin/env python
"""Headline benchmark: fused GEMM->reduce-scatter and all-gather->GEMM against
NCCL + cuBLAS on the same GPUs.

One step = one fused GEMM+RS (global M=32768, N=8192, K=8192 sharded over the
N GPUs) followed by one fused AG+GEMM (A shard [32768/N, 8192], local B
[8192, 28672/N]); bf16 N(0,1) activations, N(0,0.02) AG weights, synthetic.
The same step is also timed on the baseline path (torch.matmul = cuBLAS, then /
preceded by the NCCL collective).  Every time is device-timed with CUDA events
and reported as the max over ranks.  Ahead of every timed operation (of both paths) the L2 is flushed and a
device barrier over all ranks runs, untimed, so that an operation's time does not include waiting for a rank
that was still busy with the previous one (the reference times its fused kernel the same way:
comm_comp/exp3_gemm_rs_fused.cu:278-331).

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \\
        --master-port 29500 bench.py --gpus 8 --steps 20 --warmup 5

Prints one JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

REF_UNAVAILABLE = ("reference is 13 stand-alone CUDA programs, not an installable package (pip: neither setup.py "
                   "nor pyproject.toml); its GEMM+RS / AG+GEMM programs need the empty CUTLASS submodule and are "
                   "sm_90a wgmma kernels that cannot run on sm_100")


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="tileccl", choices=["tileccl", "reference"])
    ap.add_argument("--m", type=int, default=32768)
    ap.add_argument("--n-rs", type=int, default=8192)
    ap.add_argument("--k-rs", type=int, default=8192, help="global K of the GEMM+RS, sharded over the GPUs")
    ap.add_argument("--k-ag", type=int, default=8192)
    ap.add_argument("--n-ag", type=int, default=28672, help="global N of the AG+GEMM, sharded over the GPUs")
    ap.add_argument("--gather-rows", type=int, default=512)
    ap.add_argument("--cta-group", type=int, default=2)
    ap.add_argument("--rs-cta-group", type=int, default=0, help="CTA form of the GEMM+RS alone (0 = --cta-group)")
    ap.add_argument("--signal-batch", type=int, default=0, help="GEMM+RS: finished tiles per system-scope fence (0 = library default)")
    ap.add_argument("--gather-warps", type=int, default=0, help="AG+GEMM: gather warps per CTA (0 = library default)")
    ap.add_argument("--ag-group-m", type=int, default=0, help="AG+GEMM: raster group height (0 = library default)")
    ap.add_argument("--ag-vec32", type=int, default=-1, help="AG+GEMM: 32-byte gather moves, 0 or 1 (-1 = library default)")
    ap.add_argument("--pre-barrier", type=int, default=1, help="1: a device barrier over all ranks runs (untimed) ahead of every timed operation; "
                                                                "0: operations follow each other directly and rank skew is charged to the next one")
    ap.add_argument("--no-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    return ap.parse_args()


def main():
    args = parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": REF_UNAVAILABLE}))
        return 0

    import torch
    import torch.distributed as dist

    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from tileccl_b200 import _native
    from tileccl_b200.ops import baseline as base
    from tileccl_b200.ops import elementwise as ew
    from tileccl_b200.ops.ag_gemm import AgGemm
    from tileccl_b200.ops.gemm_rs import GemmRs
    from tileccl_b200.parallel import group as G
    from tileccl_b200.parallel.heap import SymmetricHeap
    from tileccl_b200.utils import roofline
    from tileccl_b200.utils.clocks import make_sampler
    from tileccl_b200.utils.timing import L2Flusher

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the kernels have no CPU fallback")
    _native.lib()  # fail loudly if the native library is missing

    rank, world, local = G.init()
    # Clock / throttle sampling runs from here to the end of the fused timing;
    # the summary keeps the samples taken under load.
    sampler = None            # started right before the timed loop
    if world != args.gpus and rank == 0:
        print(f"warning: --gpus {args.gpus} but WORLD_SIZE is {world}", file=sys.stderr)
    tp = world
    M = args.m
    N_rs, K_rs = args.n_rs, args.k_rs // tp
    K_ag, N_ag = args.k_ag, args.n_ag // tp
    steps, warmup = args.steps, max(3, args.warmup)
    dev = torch.device("cuda", torch.cuda.current_device())

    heap_bytes = 3 * (M * N_rs * 2 + (M // tp) * N_rs * 2 + M * K_ag * 2) + (64 << 20)
    heap = SymmetricHeap(heap_bytes)

    # Inputs: synthetic, seeded per rank.
    A_rs = torch.empty(M, K_rs, dtype=torch.bfloat16, device=dev)
    Bt_rs = torch.empty(N_rs, K_rs, dtype=torch.bfloat16, device=dev)
    Bt_ag = torch.empty(N_ag, K_ag, dtype=torch.bfloat16, device=dev)
    ew.fill_normal_(A_rs, seed=10 + rank)
    ew.fill_normal_(Bt_rs, seed=110 + rank)
    ew.fill_normal_(Bt_ag, seed=210 + rank, std=0.02)
    rs_kw = dict(cta_group=args.rs_cta_group or args.cta_group, signal_batch=args.signal_batch)
    ag_kw = dict(cta_group=args.cta_group, gather_rows=args.gather_rows, gather_warps=args.gather_warps, group_m=args.ag_group_m)
    if args.ag_vec32 >= 0:
        ag_kw["vec32"] = bool(args.ag_vec32)
    rs = GemmRs(heap, A_rs, Bt_rs, **rs_kw)
    ag = AgGemm(heap, M, K_ag, Bt_ag, **ag_kw)
    ew.fill_normal_(ag.a_shard, seed=310 + rank)
    torch.cuda.synchronize()
    G.host_barrier()

    def fused_step():
        rs()
        ag()

    # Baseline path (cuBLAS + NCCL), same inputs.
    run_base = not args.no_baseline
    if run_base:
        full = torch.empty(M, N_rs, dtype=torch.bfloat16, device=dev)
        out_b = torch.empty(M // tp, N_rs, dtype=torch.bfloat16, device=dev) if tp > 1 else full
        gathered = torch.empty(M, K_ag, dtype=torch.bfloat16, device=dev) if tp > 1 else None
        out_ag_b = torch.empty(M, N_ag, dtype=torch.bfloat16, device=dev)
        shard_b = ag.a_shard.clone()

        def base_rs():
            return base.gemm_rs_baseline(A_rs, Bt_rs, out=out_b if tp > 1 else None, full=full)

        def base_ag():
            return base.ag_gemm_baseline(shard_b, Bt_ag, gathered=gathered, out=out_ag_b)

    # ---- verification (untimed) ----
    # GEMM+RS: against an fp32 computation of sampled rows of this rank's shard (every 16th row: all tile rows,
    # all four epilogue warps, every tile column).  Each rank's partial product crosses NVLink as bf16 and the
    # sum is rounded once more, so |out - ref| <= 2^-8 * (sum_r |partial_r| + |ref|) (+5 % and a small absolute
    # term for the fp32 reference's own rounding).  AG+GEMM: against cuBLAS on the NCCL-gathered input.
    verified = None
    fused_step()
    rs.check()
    ag.check()
    seg = M // tp
    rows_local = torch.arange(0, seg, 16, device=dev)
    if tp > 1:
        want_rows = torch.cat([r * seg + rows_local for r in range(tp)])            # every rank's sample, in rank order
        a_rows = [torch.empty(want_rows.numel(), K_rs, dtype=torch.bfloat16, device=dev) for _ in range(tp)]
        b_all = [torch.empty_like(Bt_rs) for _ in range(tp)]
        dist.all_gather(a_rows, A_rs[want_rows].contiguous())
        dist.all_gather(b_all, Bt_rs)
        mine = slice(rank * rows_local.numel(), (rank + 1) * rows_local.numel())
        parts = [a[mine].float() @ b.float().t() for a, b in zip(a_rows, b_all)]
        del a_rows, b_all
    else:
        parts = [A_rs[rows_local].float() @ Bt_rs.float().t()]
    ref = sum(parts)
    bound = 1.05 * 2.0 ** -8 * (sum(p.abs() for p in parts) + ref.abs()) + 1e-2
    got = rs.out[rows_local].float()
    e_rs = ((got - ref).abs() / bound).max().item()                                  # <= 1 passes
    e_rs_rel = ((got - ref).abs() / (ref.abs() + 1)).max().item()
    del parts, ref, bound, got
    errs = {"gemm_rs_err_over_bf16_rounding_bound": e_rs, "gemm_rs_max_rel": e_rs_rel}
    ok_local = e_rs <= 1.0
    if run_base:
        oa = base_ag()
        torch.cuda.synchronize()
        e_ag = ((ag.out.float() - oa.float()).abs() / (oa.float().abs() + 1)).max().item()
        errs["ag_gemm_max_rel_vs_cublas"] = e_ag
        ok_local = ok_local and e_ag < 0.02
    else:
        if tp > 1:
            shards = [torch.empty_like(ag.a_shard) for _ in range(tp)]
            dist.all_gather(shards, ag.a_shard.contiguous())
            full_x = torch.cat(shards)
            del shards
        else:
            full_x = ag.a_full
        sample = torch.arange(0, M, 64, device=dev)
        ref_ag = full_x[sample].float() @ Bt_ag.float().t()
        e_ag = ((ag.out[sample].float() - ref_ag).abs() / (ref_ag.abs() + 1)).max().item()
        errs["ag_gemm_max_rel_vs_fp32_rows"] = e_ag
        ok_local = ok_local and e_ag < 0.02
    verified = bool(G.max_over_ranks(0.0 if ok_local else 1.0) == 0.0)
    errs = {k: G.max_over_ranks(v) for k, v in errs.items()}

    flush = L2Flusher()

    bar = ew.DeviceBarrier(heap)

    def before_op():
        flush()
        if args.pre_barrier:
            bar()

    def timed(variants, n_steps, n_warm):
        """variants: {name: [fn, ...]}.  Per-step device times (us) of each
        function, one step of every variant in turn so that the fused path and
        the baseline see the same clocks and temperature."""
        names = list(variants)
        for _ in range(n_warm):
            for n in names:
                for f in variants[n]:
                    before_op()
                    f()
        torch.cuda.synchronize()
        G.host_barrier()
        own0 = rs.launches + ag.launches + bar.epoch          # kernels of this library launched so far
        ev = {n: [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in variants[n]]
                  for _ in range(n_steps)] for n in names}
        for i in range(n_steps):
            # the two paths take turns at going first, so that neither always starts right after the other's
            # last (power-hungry) kernel
            for n in (names if i % 2 == 0 else names[::-1]):
                for j, f in enumerate(variants[n]):
                    before_op()
                    ev[n][i][j][0].record()
                    f()
                    ev[n][i][j][1].record()
        torch.cuda.synchronize()
        G.host_barrier()
        own = rs.launches + ag.launches + bar.epoch - own0   # fused kernels and device barriers inside the timed loop
        return {n: [[ev[n][i][j][0].elapsed_time(ev[n][i][j][1]) * 1e3 for i in range(n_steps)]
                    for j in range(len(variants[n]))] for n in names}, own

    variants = {"fused": [rs, ag]}
    if run_base:
        variants["base"] = [base_rs, base_ag]
    # A run that saw a hardware or thermal slow-down is not a measurement: take it once more.
    bad_reasons = {"hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown"}
    for attempt in range(2):
        # Clock / throttle sampling (read-only) spans exactly the timed loop of this attempt.
        if rank == 0:
            phys = int(os.environ.get("CUDA_VISIBLE_DEVICES", "").split(",")[local]) if os.environ.get("CUDA_VISIBLE_DEVICES", "").replace(",", "").isdigit() else local
            sampler = make_sampler(phys).start()
        res, gpu_launches = timed(variants, steps, warmup)
        clocks = sampler.summary() if sampler else None
        throttled = torch.tensor([1 if clocks and bad_reasons & set(clocks.get("reasons", [])) else 0], device=dev)
        if world > 1:
            dist.broadcast(throttled, src=0)
        if not int(throttled) or attempt == 1:
            break
        if rank == 0:
            print(f"clock record shows {clocks['reasons']}: measuring once more", file=sys.stderr)
        time.sleep(2.0)
    if clocks is not None:
        clocks["attempts"] = attempt + 1
    rs.check()
    ag.check()
    bar.check()
    per = res["fused"]
    rs_us = G.max_over_ranks(sum(per[0]) / steps)
    ag_us = G.max_over_ranks(sum(per[1]) / steps)
    step_us = G.max_over_ranks(sum(a + b for a, b in zip(per[0], per[1])) / steps)

    b_rs_us = b_ag_us = b_step_us = None
    if run_base:
        perb = res["base"]
        b_rs_us = G.max_over_ranks(sum(perb[0]) / steps)
        b_ag_us = G.max_over_ranks(sum(perb[1]) / steps)
        b_step_us = G.max_over_ranks(sum(a + b for a, b in zip(perb[0], perb[1])) / steps)

    # ---- end to end through the public API: every step copies its inputs host -> device from
    # pinned memory, runs the two fused ops, and reads a result metric back to the host.  Two sets
    # of device input buffers (and of plans bound to them) let the copy of step i+1 run on a copy
    # stream while step i computes; each step still waits for its own inputs and its own result.
    e2e = None
    if not args.no_e2e:
        a_host = torch.empty(M, K_rs, dtype=torch.bfloat16).pin_memory()
        x_host = torch.empty(M // tp, K_ag, dtype=torch.bfloat16).pin_memory()
        a_host.copy_(A_rs)
        x_host.copy_(ag.a_shard)
        A_rs2 = torch.empty_like(A_rs)
        rs2 = GemmRs(heap, A_rs2, Bt_rs, **rs_kw)
        ag2 = AgGemm(heap, M, K_ag, Bt_ag, out=ag.out, **ag_kw)
        sets = [(A_rs, rs, ag), (A_rs2, rs2, ag2)]
        copy_stream = torch.cuda.Stream()
        ready = [torch.cuda.Event() for _ in sets]       # inputs of the set have landed
        free = [torch.cuda.Event() for _ in sets]        # the set's kernels are done with its inputs
        metric_host = torch.empty(2, dtype=torch.float32).pin_memory()
        main_stream = torch.cuda.current_stream()

        def stage_inputs(i):
            a_dev, _, ag_i = sets[i % 2]
            copy_stream.wait_event(free[i % 2])
            with torch.cuda.stream(copy_stream):
                a_dev.copy_(a_host, non_blocking=True)
                ag_i.a_shard.copy_(x_host, non_blocking=True)
                ready[i % 2].record(copy_stream)

        def compute(i):
            _, rs_i, ag_i = sets[i % 2]
            main_stream.wait_event(ready[i % 2])
            rs_i()
            ag_i()
            free[i % 2].record(main_stream)
            m = torch.stack([rs_i.out[0].float().sum(), ag_i.out[0].float().sum()])
            metric_host.copy_(m, non_blocking=True)
            main_stream.synchronize()
            return float(metric_host[0]) + float(metric_host[1])

        def e2e_loop(n):
            for ev in free:
                ev.record(main_stream)
            stage_inputs(0)
            for i in range(n):
                if i + 1 < n:
                    stage_inputs(i + 1)
                compute(i)

        e2e_loop(4)
        torch.cuda.synchronize()
        G.host_barrier()
        t0 = time.perf_counter()
        e2e_loop(steps)
        torch.cuda.synchronize()
        dt = (time.perf_counter() - t0) / steps * 1e6
        G.host_barrier()
        e2e = {"value": round(G.max_over_ranks(dt), 2), "unit": "us_per_step",
               "h2d_bytes_per_step": a_host.numel() * 2 + x_host.numel() * 2,
               "d2h_bytes_per_step": metric_host.numel() * 4,
               "how": "wall clock over the timed steps; H2D of step i+1 overlaps the kernels of step i (two input buffer sets)"}
        for op in (rs, ag, rs2, ag2):
            op.check()

    roof_rs = roofline.gemm_rs_roofline_us(M, N_rs, K_rs, tp)
    roof_ag = roofline.ag_gemm_roofline_us(M, N_ag, K_ag, tp)
    flops = 2.0 * M * N_rs * K_rs * tp + 2.0 * M * N_ag * K_ag * tp
    # Which cuBLAS peak bounds this run depends on the clock it held: both fractions are given, `pct` is the one that applies.
    f_rs = roofline.fractions(roof_rs, rs_us, clocks)
    f_ag = roofline.fractions(roof_ag, ag_us, clocks)
    which = "burst" if "burst" in (f_rs["of"], f_ag["of"]) else "sustained"
    roof_us = (roof_rs["roofline_burst_us"] + roof_ag["roofline_burst_us"]) if which == "burst" else (roof_rs["roofline_us"] + roof_ag["roofline_us"])

    rc = 0
    if rank == 0:
        out = {
            "metric": "fused GEMM+RS + AG+GEMM step time (device-timed, max over ranks)",
            "value": round(step_us, 2), "unit": "us_per_step", "n_gpus": world, "steps": steps, "warmup": warmup,
            "ms_per_step": round(step_us / 1e3, 4), "higher_is_better": False, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic N(0,1) bf16 activations, N(0,0.02) AG weights, random init",
            "config": {"model": "flux-style TP GEMM pair (Llama-3-70B MLP shapes)",
                       "gemm_rs": {"M": M, "N": N_rs, "K_global": args.k_rs, "K_per_rank": K_rs},
                       "ag_gemm": {"M": M, "K": K_ag, "N_global": args.n_ag, "N_per_rank": N_ag, "gather_rows": args.gather_rows},
                       "global_batch": M, "seq_len": None, "parallelism": f"tp{tp}", "cta_group": args.cta_group, "knobs": {"gemm_rs": rs_kw, "ag_gemm": {k: v for k, v in ag_kw.items() if k != "gather_rows"}},
                       "l2": "flushed ahead of every timed operation (256 MiB write); inputs also exceed L2",
                       "timing": ("fused and NCCL+cuBLAS steps alternate inside one timed loop and take turns at going first; a step is the sum of its two operations, each timed by "
                                  "its own pair of CUDA events" + (", behind an untimed device barrier over all ranks" if args.pre_barrier else ""))},
            "gemm_rs_us": round(rs_us, 2), "ag_gemm_us": round(ag_us, 2),
            "nccl_cublas_us": None if b_step_us is None else round(b_step_us, 2),
            "nccl_cublas_gemm_rs_us": None if b_rs_us is None else round(b_rs_us, 2),
            "nccl_cublas_ag_gemm_us": None if b_ag_us is None else round(b_ag_us, 2),
            "speedup_vs_nccl_cublas": None if b_step_us is None else round(b_step_us / step_us, 4),
            "speedup_gemm_rs": None if b_rs_us is None else round(b_rs_us / rs_us, 4),
            "speedup_ag_gemm": None if b_ag_us is None else round(b_ag_us / ag_us, 4),
            "tflops_aggregate": round(flops / (step_us * 1e-6) / 1e12, 1),
            "roofline_us": round(roof_us, 2),
            "roofline": {"gemm_rs": roof_rs, "ag_gemm": roof_ag,
                         "of": f"{roof_rs['peaks']} peaks: cuBLAS bf16 {which} rate (chosen from the SM clock sampled under load), "
                               f"{roof_rs['link_gbs']:.0f} GB/s NVLink per direction ({roof_rs['link_file']})"},
            "pct_roofline": round(100.0 * roof_us / step_us, 1),
            "pct_roofline_gemm_rs": f_rs["pct"], "pct_roofline_ag_gemm": f_ag["pct"],
            "pct_roofline_detail": {"gemm_rs": f_rs, "ag_gemm": f_ag},
            "wave_efficiency": {"gemm_rs": round(roofline.wave_efficiency(M, N_rs, rs_kw["cta_group"])["efficiency"], 4),
                                "ag_gemm": round(roofline.wave_efficiency(M, N_ag, args.cta_group)["efficiency"], 4),
                                "note": "share of the persistent grid's tile slots that hold a tile; not folded into the roofline"},
            "verified": verified, "verify_errors": errs,
            "clocks": clocks, "e2e": e2e, "gpu_launches": gpu_launches, "impl": "tileccl_b200",
            "host_numa": G.numa_info,
        }
        if not verified:
            # A wrong result is not a measurement: no value, and a failing exit code.
            out["invalid"] = "verification failed: " + json.dumps(errs)
            for k in ("value", "ms_per_step", "gemm_rs_us", "ag_gemm_us", "speedup_vs_nccl_cublas", "speedup_gemm_rs", "speedup_ag_gemm", "pct_roofline"):
                out[k] = None
            out["e2e"] = None
        print(json.dumps(out), flush=True)
    if not verified:
        rc = 3
    torch.cuda.synchronize()
    G.host_barrier()
    heap.close()
    G.shutdown()
    return rc


if __name__ == "__main__":
    sys.exit(main())
