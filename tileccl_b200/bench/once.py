"""Single-GPU "once" runner: launches one kernel a few times and exits, for
profiling with ncu (small case, few launches).

    python -m tileccl_b200.bench.once gemm --m 8192 --n 8192 --k 8192 --cta-group 2 --launches 3
    python -m tileccl_b200.bench.once gemm_rs --m 8192 --n 8192 --k 1024      (world of one, staged path)
    python -m tileccl_b200.bench.once silu_mul --m 16384 --n 3584
    python -m tileccl_b200.bench.once ag_gemm --m 8192 --n 7168 --k 8192 --epi silu_mul   (world of one: flag-gated
                                                    producer, gather warps idle, fused SiLU(gate)*up epilogue)
    python -m tileccl_b200.bench.once barrier                      (the device barrier kernel, world of one)
    python -m tileccl_b200.bench.once p2p_copy --m 16384 --n 8192  (the flat 16-byte mover of nvls_bw, local to local)

The reference's counterpart is ``peer_l2_probe --modes once`` (l2_peer_cache/peer_l2_probe.cu:53-58).
"""
from __future__ import annotations

import argparse
import sys

import torch

from ..ops import elementwise as ew
from ..ops.ag_gemm import AgGemm
from ..ops.gemm import GemmPlan
from ..ops.gemm_rs import GemmRs
from ..parallel.heap import SymmetricHeap
from . import _common as C


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("what", choices=["gemm", "gemm_rs", "silu_mul", "ag_gemm", "barrier", "p2p_copy"])
    ap.add_argument("--m", type=C.parse_size, default=8192)
    ap.add_argument("--n", type=C.parse_size, default=8192)
    ap.add_argument("--k", type=C.parse_size, default=8192)
    ap.add_argument("--cta-group", type=int, default=2)
    ap.add_argument("--launches", type=int, default=3)
    ap.add_argument("--epi", default=None, choices=["silu_mul"], help="ag_gemm: fused activation epilogue")
    args = ap.parse_args(argv)
    dev = torch.device("cuda", torch.cuda.current_device())
    M, N, K = args.m, args.n, args.k
    if args.what == "barrier":
        heap = SymmetricHeap(8 << 20)
        bar = ew.DeviceBarrier(heap)
        run, check = bar, bar.check
    elif args.what == "p2p_copy":
        import ctypes as C_

        from .. import _native
        src = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
        dst = torch.empty_like(src)
        ew.fill_normal_(src, seed=3)
        lib = _native.lib()
        run = lambda: _native.check(lib.tcl_p2p_copy(C_.c_void_p(dst.data_ptr()), C_.c_void_p(src.data_ptr()), src.numel() * 2, 0,
                                                     C_.c_void_p(torch.cuda.current_stream().cuda_stream)), "p2p_copy")
        check = lambda: None
    elif args.what == "silu_mul":
        gu = torch.empty(M, 2 * N, dtype=torch.bfloat16, device=dev)
        ew.fill_normal_(gu, seed=1)
        out = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
        run = lambda: ew.silu_mul(gu, out)
        check = lambda: None
    else:
        A = torch.empty(M, K, dtype=torch.bfloat16, device=dev)
        Bt = torch.empty(N, K, dtype=torch.bfloat16, device=dev)
        ew.fill_normal_(A, seed=1)
        ew.fill_normal_(Bt, seed=2)
        if args.what == "gemm":
            plan = GemmPlan(A, Bt, cta_group=args.cta_group)
            run, check = plan, plan.check
        elif args.what == "ag_gemm":
            heap = SymmetricHeap(M * K * 2 + (64 << 20))
            op = AgGemm(heap, M, K, Bt, cta_group=args.cta_group, epi=args.epi)
            op.a_shard.copy_(A)
            run, check = op, op.check
        else:
            heap = SymmetricHeap(2 * M * N * 2 + (64 << 20))
            op = GemmRs(heap, A, Bt, cta_group=args.cta_group, force_staged=True)
            run, check = op, op.check
    s = torch.cuda.Event(enable_timing=True)
    e = torch.cuda.Event(enable_timing=True)
    run()
    torch.cuda.synchronize()
    s.record()
    for _ in range(args.launches):
        run()
    e.record()
    torch.cuda.synchronize()
    check()
    print(f"{args.what} {M}x{N}x{K}: {s.elapsed_time(e) * 1e3 / args.launches:.1f} us per launch")
    return 0


if __name__ == "__main__":
    sys.exit(main())
