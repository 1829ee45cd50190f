"""Device timing: per-iteration CUDA events with an L2 flush between iterations."""
from __future__ import annotations

import torch


class L2Flusher:
    """Overwrites a buffer larger than the 126 MB L2 so the next iteration starts cold."""

    def __init__(self, nbytes: int = 256 << 20):
        self.buf = torch.empty(nbytes // 4, dtype=torch.int32, device="cuda")
        self.v = 0

    def __call__(self) -> None:
        self.v += 1
        self.buf.fill_(self.v)


def time_iters(fn, iters: int, warmup: int = 3, flush: L2Flusher | None = None, before=None) -> list[float]:
    """Runs ``fn`` ``warmup`` + ``iters`` times; returns the device time of each
    timed call in microseconds (events on the current stream).  ``before`` runs
    untimed ahead of every call (e.g. a device barrier)."""
    for _ in range(warmup):
        if before:
            before()
        fn()
    torch.cuda.synchronize()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(iters)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(iters)]
    for i in range(iters):
        if flush:
            flush()
        if before:
            before()
        starts[i].record()
        fn()
        ends[i].record()
    torch.cuda.synchronize()
    return [s.elapsed_time(e) * 1000.0 for s, e in zip(starts, ends)]
