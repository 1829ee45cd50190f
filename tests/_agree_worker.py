"""Rank program of tests/test_agree_cpu.py: only the last rank's check fails; every rank must raise."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from tileccl_b200.bench import _common as C  # noqa: E402
from tileccl_b200.parallel import group as G  # noqa: E402

rank, world, _ = G.init(backend="gloo")


def check():
    if rank == world - 1:
        raise ValueError("setting gw9: wait ran out")


try:
    C.agree_no_failure(check, "warm-up")
    print(f"AGREE_MISSED rank {rank}")
except RuntimeError as e:
    ok = f"rank {world - 1}: ValueError: setting gw9: wait ran out" in str(e) and "warm-up" in str(e)
    print(("AGREE_OK" if ok else "AGREE_BAD") + f" rank {rank}: {e}")
C.agree_no_failure(lambda: None)          # a clean check passes on every rank, and the ranks are still in step
print(f"AGREE_CLEAN rank {rank}")
G.shutdown()
