"""Bandwidth sweep of the NVSwitch paths, 4 KB ... 1 GB, every rank active at once.

    p2p_st      plain 16-byte stores into the next rank's heap (ring)
    p2p_ld      plain 16-byte loads from the next rank's heap
    p2p_a2a     plain 16-byte stores of 1/world of the payload into EVERY peer's heap at once (the traffic pattern
                of the fused GEMM + reduce-scatter epilogue; GB/s counts the (world-1)/world that leaves the GPU)
    mc_bcast    multimem.st: one store lands on every GPU (all-gather building block)
    mc_ldreduce multimem.ld_reduce: one load returns the sum over all GPUs, added inside the switch
    mc_red      multimem.red: one instruction adds into every GPU's copy
    nccl_ag / nccl_rs   ncclAllGather / ncclReduceScatter of the same payload (baseline)
    barrier_p2p / barrier_mc   all-ranks device barrier: one red.release per peer, or one multimem.red.release
                               per rank (bytes = 0; us is the launch-to-exit time of the barrier kernel)
    rtt_st_release / rtt_red_release / rtt_mc_red   flag ping-pong between ranks 0 and 1, timed inside the kernel
                               with %globaltimer: us is one round trip (two signals)

GB/s is payload bytes per rank per second (for nccl_*: the bus-bandwidth convention, (w-1)/w of the
full buffer).  Needs a symmetric heap on the VMM back end bound to a multicast object; when the
device or the driver offers none, the mc_* rows are reported as unavailable.

The reference has no multicast path; its bandwidth sweep is tests/pk_bw_sweep.cu (ce / tma / reg).
"""
from __future__ import annotations

import argparse
import ctypes as C_
import sys

import torch
import torch.distributed as dist

from .. import _native
from ..ops import elementwise as ew
from ..parallel import group as G
from ..parallel.heap import SymmetricHeap
from ..utils import csvio
from . import _common as C

COLUMNS = "mover,bytes,world,us,gbps,verify".split(",")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--sizes", default="4K,64K,1M,16M,128M,1G")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--blocks", type=int, default=0)
    ap.add_argument("--no-multicast", action="store_true")
    ap.add_argument("--csv", default=None)
    args = ap.parse_args(argv)
    rank, world, _ = G.init()
    lib = _native.lib()
    sizes = [C.parse_size(s) for s in C.split_csv(args.sizes)]
    mx = max(sizes)
    use_mc = world > 1 and not args.no_multicast and bool(lib.tcl_multicast_supported(torch.cuda.current_device()))
    why = ""
    try:
        heap = SymmetricHeap(2 * mx + (8 << 20), backend="vmm", multicast=use_mc)
    except Exception as e:  # noqa: BLE001
        why = f"{type(e).__name__}: {e}"
        use_mc = False
        heap = None
    # every rank must take the same path
    flag = torch.tensor([1 if heap is not None else 0], device="cuda")
    if world > 1:
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if int(flag) == 0:
        if heap is not None:
            heap.close()
        use_mc = False
        heap = SymmetricHeap(2 * mx + (8 << 20), backend="ipc")
        if rank == 0:
            print(f"# VMM/multicast heap unavailable ({why or 'on a peer'}): IPC heap, p2p rows only")
    try:
        sym = heap.empty((mx,), torch.uint8)      # symmetric buffer
        loc = torch.empty(mx, dtype=torch.uint8, device="cuda")
        loc.view(torch.bfloat16).fill_(1.0)
        bar = ew.DeviceBarrier(heap)
        sym_ptrs = (C_.c_void_p * _native.MAX_WORLD)(*[heap.peer_ptr(sym, r) for r in range(world)])
        nxt = (rank + 1) % world
        st = lambda: C_.c_void_p(torch.cuda.current_stream().cuda_stream)  # noqa: E731
        vp = C_.c_void_p
        csv = csvio.CsvAppender(args.csv if rank == 0 else None, COLUMNS)
        if rank == 0:
            print(f"# nvls_bw world={world} multicast={'yes' if use_mc else 'no'} [{C.device_line()}]")
            print(f"{'mover':12s} {'bytes':>11s} | {'us':>10s} {'GB/s':>9s} | verify")
        movers = ["p2p_st", "p2p_ld"] + (["p2p_a2a"] if world > 1 else []) + (["mc_bcast", "mc_ldreduce", "mc_red"] if use_mc else []) + (["nccl_ag", "nccl_rs"] if world > 1 else [])
        full = torch.empty(mx, dtype=torch.uint8, device="cuda")
        for n in sizes:
            for mv in movers:
                per = n // world // 16 * 16 if mv.startswith("nccl") else n
                if per < 16:
                    continue

                def run():
                    if mv == "p2p_st":
                        _native.check(lib.tcl_p2p_copy(vp(heap.peer_ptr(sym, nxt)), vp(loc.data_ptr()), n, args.blocks, st()), mv)
                    elif mv == "p2p_ld":
                        _native.check(lib.tcl_p2p_copy(vp(loc.data_ptr()), vp(heap.peer_ptr(sym, nxt)), n, args.blocks, st()), mv)
                    elif mv == "p2p_a2a":
                        sl = n // world // 16 * 16
                        _native.check(lib.tcl_p2p_scatter(sym_ptrs, vp(loc.data_ptr()), sl, world, rank, args.blocks, st()), mv)
                    elif mv == "mc_bcast":
                        # each rank broadcasts its 1/world slice: together an all-gather of n bytes
                        sl = n // world // 16 * 16
                        _native.check(lib.tcl_nvls_bcast(vp(heap.mc_ptr(sym) + rank * sl), vp(loc.data_ptr() + rank * sl), sl, args.blocks, st()), mv)
                    elif mv == "mc_ldreduce":
                        sl = n // world // 16 * 16
                        _native.check(lib.tcl_nvls_ld_reduce(vp(heap.mc_ptr(sym) + rank * sl), vp(loc.data_ptr() + rank * sl), sl, args.blocks, st()), mv)
                    elif mv == "mc_red":
                        sl = n // world // 16 * 16
                        _native.check(lib.tcl_nvls_red(vp(heap.mc_ptr(sym) + rank * sl), vp(loc.data_ptr() + rank * sl), sl, args.blocks, st()), mv)
                    elif mv == "nccl_ag":
                        dist.all_gather_into_tensor(full[: per * world], loc[:per])
                    else:
                        dist.reduce_scatter_tensor(loc[:per].view(torch.bfloat16), full[: per * world].view(torch.bfloat16))

                verify = "-"
                if mv == "mc_ldreduce":
                    sym.view(torch.bfloat16).fill_(float(rank + 1))
                    loc.zero_()
                    torch.cuda.synchronize(); G.host_barrier()
                    run()
                    torch.cuda.synchronize(); G.host_barrier()
                    sl = n // world // 16 * 16
                    got = loc[rank * sl: rank * sl + sl].view(torch.bfloat16)
                    verify = "ok" if bool((got == world * (world + 1) / 2).all()) else "FAIL"
                    loc.view(torch.bfloat16).fill_(1.0)
                elif mv == "p2p_a2a":
                    loc.view(torch.bfloat16).fill_(float(rank + 1))
                    sym.zero_()
                    torch.cuda.synchronize(); G.host_barrier()
                    run()
                    torch.cuda.synchronize(); G.host_barrier()
                    sl = n // world // 16 * 16
                    got = sym[: sl * world].view(world, sl).view(torch.bfloat16)[:, 0::max(1, sl // 2 // 64)].float()
                    want = torch.arange(1, world + 1, device="cuda", dtype=torch.float32)[:, None].expand_as(got).clone()
                    want[rank] = 0.0   # the own slot is not written
                    verify = "ok" if bool((got == want).all()) and bool((sym[: sl * world].view(world, sl).view(torch.bfloat16)[:, -1].float() == want[:, 0]).all()) else "FAIL"
                    loc.view(torch.bfloat16).fill_(1.0)
                elif mv == "mc_bcast":
                    loc.view(torch.bfloat16).fill_(1.0)
                    sym.zero_()
                    torch.cuda.synchronize(); G.host_barrier()
                    run()
                    torch.cuda.synchronize(); G.host_barrier()
                    sl = n // world // 16 * 16
                    verify = "ok" if bool((sym[: sl * world].view(torch.bfloat16) == 1.0).all()) else "FAIL"
                us = C.stats_of(C.timed_series(run, args.iters, 3, before=bar)).p50
                us = G.max_over_ranks(us)
                moved = (world - 1) / world * per * world if mv.startswith("nccl") else (n // world // 16 * 16 * (world - 1) if mv in ("mc_bcast", "mc_red", "p2p_a2a") else
                                                                                            (n // world // 16 * 16 if mv == "mc_ldreduce" else n))
                gbps = moved / us / 1e3
                bad = torch.tensor([1 if verify == "FAIL" else 0], device="cuda")
                if world > 1:
                    dist.all_reduce(bad)
                if int(bad):
                    verify = "FAIL"
                if rank == 0:
                    print(f"{mv:12s} {n:11d} | {us:10.2f} {gbps:9.1f} | {verify}")
                    csv.row(mover=mv, bytes=n, world=world, us=us, gbps=gbps, verify=verify)
        # barrier latency: world stores per rank against one multicast store per rank
        flavours = [("barrier_p2p", ew.DeviceBarrier(heap, transport="p2p"))] + ([("barrier_mc", ew.DeviceBarrier(heap, transport="nvls"))] if use_mc else [])
        for name, b in flavours:
            us = G.max_over_ranks(C.stats_of(C.timed_series(b, max(args.iters, 50), 5, before=bar)).p50)
            torch.cuda.synchronize()
            b.check()
            if rank == 0:
                print(f"{name:12s} {0:11d} | {us:10.2f} {'-':>9s} | -")
                csv.row(mover=name, bytes=0, world=world, us=us, gbps=0.0, verify="-")
        # signal round trip between ranks 0 and 1 (the other ranks idle): plain, reduction and multicast signals
        if world > 1:
            rounds = 2000
            pp_status = torch.zeros(4, dtype=torch.int32, device="cuda")
            ns = torch.zeros(1, dtype=torch.float32, device="cuda")
            for mode, name in enumerate(["rtt_st_release", "rtt_red_release", "rtt_mc_red"]):
                if mode == 2 and not use_mc:
                    continue
                flag = heap.zeros((32,), torch.int32)
                torch.cuda.synchronize(); G.host_barrier()
                base = 0
                for _ in range(3):   # the first call warms the path; the last one is reported
                    if rank < 2:
                        remote = heap.mc_ptr(flag) if mode == 2 else heap.peer_ptr(flag, 1 - rank)
                        _native.check(lib.tcl_signal_pingpong(vp(flag.data_ptr()), vp(remote), mode, 1 if rank == 0 else 0, base, rounds,
                                                              vp(ns.data_ptr()), vp(pp_status.data_ptr()), 0, st()), name)
                    torch.cuda.synchronize(); G.host_barrier()
                    base += (2 if mode == 2 else 1) * rounds
                if int(pp_status[0]) != 0:
                    raise RuntimeError(f"{name}: wait ran out: {pp_status.tolist()}")
                if rank == 0:
                    us = float(ns.item()) / 1e3
                    print(f"{name:15s} {0:8d} | {us:10.3f} {'-':>9s} | -")
                    csv.row(mover=name, bytes=0, world=world, us=us, gbps=0.0, verify="-")
        bar.check()
        csv.close()
        torch.cuda.synchronize()
        G.host_barrier()
    except BaseException:
        # no rank may leave with its memory still bound to the multicast object: unbind locally, then re-raise
        heap.release_multicast()
        raise
    heap.close()
    G.shutdown()
    return 0


if __name__ == "__main__":
    sys.exit(main())
