"""Summary statistics of timing series (mean / p50 / p95 / p99 / min / max).

Same definitions as the reference's make_stats (comm_comp/common.cuh:130-146)
and the signalling bench's percentiles (signalling/signal_fanin.cu:399-410):
percentiles are order statistics of the sorted series, no interpolation.
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass
class Stats:
    n: int
    mean: float
    p50: float
    p95: float
    p99: float
    min: float
    max: float


def percentile(sorted_vals: list[float], q: float) -> float:
    if not sorted_vals:
        return 0.0
    i = min(len(sorted_vals) - 1, int(q * len(sorted_vals)))
    return sorted_vals[i]


def make_stats(vals) -> Stats:
    v = sorted(float(x) for x in vals)
    if not v:
        return Stats(0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0)
    return Stats(len(v), sum(v) / len(v), percentile(v, 0.50), percentile(v, 0.95), percentile(v, 0.99), v[0], v[-1])


def iters_for_ms(one_iter_us: float, window_ms: float, lo: int = 5, hi: int = 2000) -> int:
    """Iterations that fill a wall-clock window (comm_comp/common.cuh:120-128)."""
    if one_iter_us <= 0:
        return lo
    return max(lo, min(hi, int(window_ms * 1000.0 / one_iter_us)))
