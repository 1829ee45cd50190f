"""Shared plumbing of the Python experiment drivers (one process per GPU)."""
from __future__ import annotations

import argparse
import os

import torch

from ..parallel import group as G
from ..utils.stats import make_stats


def parse_shape(text: str) -> tuple[int, int, int]:
    """``N`` -> (N, N, N); ``MxNxK`` -> (M, N, K)  (comm_comp/common.cuh:80-105)."""
    parts = text.lower().split("x")
    if len(parts) == 1:
        v = parse_size(parts[0])
        return v, v, v
    if len(parts) != 3:
        raise argparse.ArgumentTypeError(f"bad shape {text!r}: want N or MxNxK")
    return tuple(parse_size(p) for p in parts)  # type: ignore[return-value]


def parse_size(text: str) -> int:
    """Integer with an optional K/M/G suffix, powers of 1024 (comm_comp/common.cuh:52-66)."""
    t = text.strip()
    mult = 1
    if t and t[-1].upper() in "KMG":
        mult = 1024 ** ("KMG".index(t[-1].upper()) + 1)
        t = t[:-1]
    try:
        return int(float(t) * mult)
    except ValueError as e:
        raise argparse.ArgumentTypeError(f"bad size {text!r}") from e


def split_csv(text: str) -> list[str]:
    return [p for p in (x.strip() for x in text.split(",")) if p]


def timed_series(fn, iters: int, warmup: int, before=None, flush=None) -> list[float]:
    """Device time of each of ``iters`` calls in microseconds; ``before`` (e.g. a
    device barrier) and ``flush`` run untimed ahead of every call."""
    for _ in range(warmup):
        if before:
            before()
        fn()
    torch.cuda.synchronize()
    G.host_barrier()
    s = [torch.cuda.Event(enable_timing=True) for _ in range(iters)]
    e = [torch.cuda.Event(enable_timing=True) for _ in range(iters)]
    for i in range(iters):
        if flush:
            flush()
        if before:
            before()
        s[i].record()
        fn()
        e[i].record()
    torch.cuda.synchronize()
    return [a.elapsed_time(b) * 1e3 for a, b in zip(s, e)]


def turn_order(names: list, i: int) -> list:
    """The order of the variants in iteration ``i``: a different start and a different stride every iteration
    (strides coprime to the count), so that over a run no variant keeps the same predecessor.  A plain rotation
    would change who goes first but leave every variant behind the same neighbour, and a kernel that always
    follows the power-hungry library GEMM always starts at a lower clock.  Deterministic: every rank gets the
    same order."""
    n = len(names)
    if n < 3:
        return names[i % n:] + names[:i % n] if n else []
    import math
    strides = [s for s in range(1, n) if math.gcd(s, n) == 1]
    s = strides[i % len(strides)]
    return [names[(i + j * s) % n] for j in range(n)]


def agree_no_failure(check, what: str = "step") -> None:
    """Runs ``check()`` on this rank, then lets all ranks agree: if it raised anywhere, every rank raises the
    same RuntimeError naming the ranks and their messages.  A failure seen by one rank only would otherwise
    leave the others waiting for it in their next collective."""
    err = None
    try:
        check()
    except Exception as e:  # noqa: BLE001  (reported on every rank below)
        err = f"{type(e).__name__}: {e}"
    errs = G.all_gather_object(err)
    if any(errs):
        raise RuntimeError(f"failed during {what}: " + "; ".join(f"rank {r}: {e}" for r, e in enumerate(errs) if e))


def timed_interleaved(fns: dict, iters: int, warmup: int, before=None, flush=None, rotate: bool = True, check=None) -> dict:
    """Like :func:`timed_series` for several variants at once, taking one
    iteration of each in turn, so that all of them see the same clocks and
    temperature (the paired-baseline discipline of the reference,
    comm_comp/exp1_ce_interference.cu:545-548).  With ``rotate`` the turn starts
    one variant later every iteration, so that no variant always runs right
    after the same neighbour (a kernel that follows a power-hungry one starts at
    a lower clock, see :func:`turn_order`); every rank orders alike.

    ``check`` (optional) is called on every rank after the warm-up and should raise if a variant
    reported a failure (a bounded wait that ran out).  The ranks then agree on the outcome and all of
    them raise, naming rank and variant, before the timed loop starts: a variant whose every launch
    sits out its time-out would otherwise hold the GPUs for iterations x time-out."""
    names = list(fns)
    for _ in range(warmup):
        for n in names:
            if before:
                before()
            fns[n]()
    torch.cuda.synchronize()
    if check is not None:
        agree_no_failure(check, "warm-up")
    G.host_barrier()
    ev = {n: ([torch.cuda.Event(enable_timing=True) for _ in range(iters)],
              [torch.cuda.Event(enable_timing=True) for _ in range(iters)]) for n in names}
    for i in range(iters):
        for n in turn_order(names, i) if rotate else names:
            if flush:
                flush()
            if before:
                before()
            ev[n][0][i].record()
            fns[n]()
            ev[n][1][i].record()
    torch.cuda.synchronize()
    return {n: [a.elapsed_time(b) * 1e3 for a, b in zip(*ev[n])] for n in names}


def stats_of(series):
    return make_stats(series)


def device_line() -> str:
    p = torch.cuda.get_device_properties(torch.cuda.current_device())
    return f"{p.name}, {p.multi_processor_count} SMs, {p.total_memory / 2**30:.0f} GiB, cc {p.major}.{p.minor}"


def out_path(path: str | None) -> str | None:
    if path:
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    return path
