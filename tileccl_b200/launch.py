"""Starts an experiment with one process per GPU on this node.

    python -m tileccl_b200.launch -n 8 exp3_gemm_rs_fused --m 32768 --n 8192 --k 1024 --verify

is the same as running ``tileccl_b200/bench/run.py`` under
``python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1``
with a ``--`` in front of the script (so that torchrun does not try to read
the experiment's own flags).  The reference forks its ranks itself
(comm_comp/ipc_multiproc.cuh:105-136); the native counterpart of that launcher
is csrc/runtime/launcher.cpp.
"""
from __future__ import annotations

import os
import subprocess
import sys


def main() -> int:
    argv = sys.argv[1:]
    nproc, port = 1, 29540
    while argv and argv[0] in ("-n", "--nproc", "--port"):
        if argv[0] == "--port":
            port = int(argv[1])
        else:
            nproc = int(argv[1])
        argv = argv[2:]
    if not argv:
        print(__doc__, file=sys.stderr)
        return 1
    script = os.path.join(os.path.dirname(os.path.abspath(__file__)), "bench", "run.py")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), "--", script, *argv]
    return subprocess.call(cmd)


if __name__ == "__main__":
    sys.exit(main())
