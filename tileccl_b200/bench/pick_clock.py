"""Which SM clock does this GPU hold under a sustained GEMM?  (Report only, by default.)

For each candidate clock the reference pins the GPU with ``nvidia-smi -lgc``, soaks it with the
8192^3 GEMM, and keeps the highest clock that holds for >= 98 % of the samples
(comm_comp/pick_clock.sh:32-101).  On shared machines nothing may change a GPU setting, so this
tool's default is to *observe*: it soaks at whatever clock policy the GPU has, reports mean / min /
p10 / hold %, and tells which candidate would be picked.  The code that applies a clock exists
(`apply=True`) but is off unless both ``--apply`` and ``TILECCL_ALLOW_CLOCK_LOCK=1`` are given, and
it always restores the previous state; it is exercised only against a fake NVML in the tests.
"""
from __future__ import annotations

import argparse
import os
import statistics
import sys
import time


class NvmlBackend:
    """The subset of NVML this tool needs; tests substitute a fake."""

    def sm_clock(self, index: int) -> int: raise NotImplementedError
    def max_sm_clock(self, index: int) -> int: raise NotImplementedError
    def lock_clocks(self, index: int, mhz: int) -> None: raise NotImplementedError
    def reset_clocks(self, index: int) -> None: raise NotImplementedError


class RealNvml(NvmlBackend):
    def __init__(self):
        import pynvml
        self.n = pynvml
        pynvml.nvmlInit()

    def _h(self, i):
        return self.n.nvmlDeviceGetHandleByIndex(i)

    def sm_clock(self, index):
        return int(self.n.nvmlDeviceGetClockInfo(self._h(index), self.n.NVML_CLOCK_SM))

    def max_sm_clock(self, index):
        return int(self.n.nvmlDeviceGetMaxClockInfo(self._h(index), self.n.NVML_CLOCK_SM))

    def lock_clocks(self, index, mhz):
        self.n.nvmlDeviceSetGpuLockedClocks(self._h(index), mhz, mhz)

    def reset_clocks(self, index):
        self.n.nvmlDeviceResetGpuLockedClocks(self._h(index))


def soak_stats(samples: list[int], target: int) -> dict:
    s = sorted(samples)
    hold = sum(1 for x in samples if abs(x - target) <= 0.02 * target) / max(1, len(samples))
    return {"target": target, "n": len(samples), "mean": statistics.mean(s) if s else 0, "min": s[0] if s else 0,
            "p10": s[len(s) // 10] if s else 0, "hold_pct": 100.0 * hold}


def pick(results: list[dict], need_pct: float = 98.0) -> int | None:
    """Highest candidate whose clock held within +-2 % for at least need_pct of the samples."""
    ok = [r["target"] for r in results if r["hold_pct"] >= need_pct]
    return max(ok) if ok else None


def soak(nvml: NvmlBackend, index: int, seconds: float, load, period_s: float = 0.1) -> list[int]:
    """Samples the SM clock while `load()` (non-blocking: enqueues work) keeps the GPU busy."""
    out = []
    t0 = time.time()
    while time.time() - t0 < seconds:
        load()
        out.append(nvml.sm_clock(index))
        time.sleep(period_s)
    return out


def run(nvml: NvmlBackend, index: int, candidates: list[int], seconds: float, load, apply: bool) -> list[dict]:
    results = []
    if not apply:
        samples = soak(nvml, index, seconds, load)
        # One observation serves every candidate: would the clock we saw have held it?
        for c in candidates:
            results.append(soak_stats(samples, c))
        return results
    for c in candidates:
        nvml.lock_clocks(index, c)
        try:
            results.append(soak_stats(soak(nvml, index, seconds, load), c))
        finally:
            nvml.reset_clocks(index)      # never leave a lock behind
    return results


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpu", type=int, default=0)
    ap.add_argument("--candidates", default="1965,1830,1700,1590,1500,1400,1305,1200")
    ap.add_argument("--soak-s", type=float, default=5.0)
    ap.add_argument("--apply", action="store_true", help="pin each candidate clock (needs TILECCL_ALLOW_CLOCK_LOCK=1 and admin rights)")
    args = ap.parse_args(argv)
    apply = args.apply and os.environ.get("TILECCL_ALLOW_CLOCK_LOCK") == "1"
    if args.apply and not apply:
        print("--apply ignored: set TILECCL_ALLOW_CLOCK_LOCK=1 as well (never on a shared machine)", file=sys.stderr)
    import torch
    torch.cuda.set_device(args.gpu)
    a = torch.randn(8192, 8192, device="cuda", dtype=torch.bfloat16)
    b = a.clone()

    def load():
        for _ in range(20):
            torch.matmul(a, b)

    res = run(RealNvml(), args.gpu, [int(c) for c in args.candidates.split(",")], args.soak_s, load, apply)
    torch.cuda.synchronize()
    print(f"{'target':>7} {'mean':>7} {'min':>6} {'p10':>6} {'hold%':>6}")
    for r in res:
        print(f"{r['target']:7d} {r['mean']:7.0f} {r['min']:6d} {r['p10']:6d} {r['hold_pct']:6.1f}")
    best = pick(res)
    print(f"highest clock that holds >= 98 %: {best if best else 'none'}" + ("" if apply else "  (observed, nothing was changed)"))
    return 0


if __name__ == "__main__":
    sys.exit(main())
