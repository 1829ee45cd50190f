#!/usr/bin/env python
"""Entry script for the Python experiment drivers, usable as a torchrun target:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \\
        tileccl_b200/bench/run.py exp3_gemm_rs_fused --m 32768 --n 8192 --k 1024 --verify

The first argument names a module of ``tileccl_b200.bench``; the rest are its flags.
"""
import importlib
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

EXPERIMENTS = ("exp1_ce_interference", "exp2_ag_gemm_granularity", "exp3_epilogue_remote",
               "exp3_gemm_rs_fused", "mlp_e2e", "nvls_bw", "gemm_vs_cublas", "once", "tune_gemm_rs")


def main() -> int:
    if len(sys.argv) < 2 or sys.argv[1] not in EXPERIMENTS:
        print(f"usage: run.py <{'|'.join(EXPERIMENTS)}> [flags]", file=sys.stderr)
        return 1
    mod = importlib.import_module(f"tileccl_b200.bench.{sys.argv[1]}")
    return int(mod.main(sys.argv[2:]) or 0)


if __name__ == "__main__":
    sys.exit(main())
