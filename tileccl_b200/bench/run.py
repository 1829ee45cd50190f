#!/usr/bin/env python
"""Entry script for the Python experiment drivers, usable as a torchrun target:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \\
        tileccl_b200/bench/run.py exp3_gemm_rs_fused --m 32768 --n 8192 --k 1024 --verify

The first argument names a module of ``tileccl_b200.bench``; the rest are its flags.

Several experiments can share one set of rank processes (one start-up, one NCCL rendezvous): separate
them with ``--then``, optionally naming each with ``--as NAME``.  With ``--manifest FILE`` rank 0 appends
one line per experiment (``NAME rc=... seconds=...``, the orchestrator's manifest format) and with
``--logs DIR`` each experiment's rank-0 output goes to ``DIR/NAME.log``.  An experiment that raises is
recorded and the batch goes on with the next one only if every rank agrees that it is still in step.

    run.py --manifest out/manifest.txt --logs out exp3_gemm_rs_fused --m 512 ... --as exp3_m512 \\
           --then exp3_gemm_rs_fused --m 1024 ... --as exp3_m1024
"""
import contextlib
import importlib
import os
import sys
import time
import traceback

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

EXPERIMENTS = ("exp1_ce_interference", "exp2_ag_gemm_granularity", "exp3_epilogue_remote",
               "exp3_gemm_rs_fused", "mlp_e2e", "nvls_bw", "gemm_vs_cublas", "once", "tune_fused")


def split_batch(argv: list[str]) -> tuple[dict, list[tuple[str, str, list[str]]]]:
    """(options, [(name, module, flags), ...]) from a command line with ``--then`` separators."""
    opts = {"manifest": None, "logs": None}
    while argv and argv[0] in ("--manifest", "--logs"):
        opts[argv[0][2:]] = argv[1]
        argv = argv[2:]
    jobs, cur = [], []
    for a in argv + ["--then"]:
        if a == "--then":
            if cur:
                name = cur[0]
                if "--as" in cur:
                    i = cur.index("--as")
                    name = cur[i + 1]
                    cur = cur[:i] + cur[i + 2:]
                jobs.append((name, cur[0], cur[1:]))
            cur = []
        else:
            cur.append(a)
    return opts, jobs


class StallDump:
    """With TILECCL_STALL_DUMP_S=<seconds> set, an experiment that is still running after that long gets the
    Python stack of every thread of every rank written to ``stall.<experiment>.rank<r>.txt`` (in
    TILECCL_STALL_DUMP_DIR, default: the log directory or the working directory), again every <seconds>: where
    each rank sits when a collective never completes.  Nothing is written, and the file is removed, when the
    experiment ends in time."""

    def __init__(self, name: str, where: str | None):
        self.file = None
        try:
            self.seconds = float(os.environ.get("TILECCL_STALL_DUMP_S", "0") or 0)
        except ValueError:
            self.seconds = 0.0
        if self.seconds > 0:
            d = os.environ.get("TILECCL_STALL_DUMP_DIR") or where or "."
            self.path = os.path.join(d, f"stall.{name}.rank{os.environ.get('RANK', '0')}.txt")

    def __enter__(self):
        if self.seconds > 0:
            import faulthandler
            self.file = open(self.path, "w")
            faulthandler.dump_traceback_later(self.seconds, repeat=True, file=self.file)
        return self

    def __exit__(self, *exc):
        if self.file is not None:
            import faulthandler
            faulthandler.cancel_dump_traceback_later()
            self.file.close()
            if os.path.getsize(self.path) == 0:
                os.remove(self.path)
        return False


def main() -> int:
    opts, jobs = split_batch(sys.argv[1:])
    if not jobs or any(mod not in EXPERIMENTS for _, mod, _ in jobs):
        print(f"usage: run.py [--manifest FILE] [--logs DIR] <{'|'.join(EXPERIMENTS)}> [flags] [--as NAME] [--then <experiment> [flags] ...]", file=sys.stderr)
        return 1
    if len(jobs) == 1 and not opts["manifest"] and not opts["logs"]:
        mod = importlib.import_module(f"tileccl_b200.bench.{jobs[0][1]}")
        with StallDump(jobs[0][0], None):
            return int(mod.main(jobs[0][2]) or 0)

    import torch
    from tileccl_b200.parallel import group as G
    rank, world, _ = G.init()
    G.hold()
    worst = 0
    try:
        for name, modname, flags in jobs:
            t0 = time.time()
            log = open(os.path.join(opts["logs"], f"{name}.log"), "w", buffering=1) if (opts["logs"] and rank == 0) else None
            rc = 0
            try:
                with contextlib.ExitStack() as st:
                    st.enter_context(StallDump(name, opts["logs"]))
                    if log:
                        log.write(f"$ {modname} {' '.join(flags)}\n")
                        log.flush()
                        st.enter_context(contextlib.redirect_stdout(log))
                    mod = importlib.import_module(f"tileccl_b200.bench.{modname}")
                    rc = int(mod.main(list(flags)) or 0)
            except SystemExit as e:
                rc = int(e.code or 0) if isinstance(e.code, int) else 1
            except Exception:  # noqa: BLE001  (recorded; whether the batch can go on is decided below)
                rc = 1
                text = traceback.format_exc()
                (log or sys.stderr).write(text)
                if log:
                    sys.stderr.write(f"[{name}] {text.splitlines()[-1]}\n")
            finally:
                if log:
                    log.close()
            # every rank must have left the experiment the same way, else the ranks are out of step
            flag = torch.tensor([rc, -rc], device="cuda")
            if world > 1:
                import torch.distributed as dist
                dist.all_reduce(flag, op=dist.ReduceOp.MAX)
            rc_all, rc_min = int(flag[0]), -int(flag[1])
            worst = max(worst, rc_all)
            if rank == 0:
                print(f"  {name}: rc={rc_all} in {time.time() - t0:.1f} s", flush=True)
                if opts["manifest"]:
                    with open(opts["manifest"], "a") as mf:
                        mf.write(f"{name} rc={rc_all} seconds={time.time() - t0:.1f}\n")
            if rc_all != rc_min:
                break          # the ranks left this experiment in different ways: stop rather than run out of step
            if rc_all != 0:
                torch.cuda.synchronize()
    finally:
        G.release()
        G.shutdown()
    return 0 if worst == 0 else 1


if __name__ == "__main__":
    sys.exit(main())
