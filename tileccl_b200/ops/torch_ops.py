"""``torch.ops.tileccl.*``: the thin PyTorch op layer.

    import tileccl_b200 as tc
    tc.init(heap_bytes=4 << 30)                      # once per process, after torch.distributed is up
    y_shard = torch.ops.tileccl.gemm_rs(a, w_t)      # a [M, K/tp], w_t [N, K/tp]  ->  [M/tp, N]
    y       = torch.ops.tileccl.ag_gemm(x_shard, w_t)  # x_shard [M/tp, K], w_t [N/tp, K]  ->  [M, N/tp]
    c       = torch.ops.tileccl.gemm(a, b_t)         # plain tcgen05 GEMM, a @ b_t.T
    h       = torch.ops.tileccl.silu_mul(gate_up)
    torch.ops.tileccl.barrier()                      # device barrier over all ranks, on the current stream

Plans (tensor maps, staging buffers, counters) are built on first use for a given operand *layout* (shapes,
row pitches) and are cached; the operands' addresses are not part of the key.  Every call points the cached
plan at the tensors it was given (a host-side re-encoding of two tensor maps) and keeps no reference to them,
so a loop that allocates fresh activations every step reuses one plan and one set of staging buffers, and
every rank builds the same plans in the same order whatever addresses its allocator hands out.  Results live
in buffers owned by the cached plan: a result is valid until the next call with operands of the same layout.
Inputs that must be peer-visible (the AG shard) are copied into the plan's slot of the symmetric heap when
they are not already there.  Building a fused plan allocates from the symmetric heap and is collective: all
ranks must make the same sequence of first calls.

The reference stops at C++ programs; this layer is what the north star adds.
"""
from __future__ import annotations

import torch

from ..parallel.heap import SymmetricHeap
from . import elementwise as ew
from .ag_gemm import AgGemm
from .gemm import GemmPlan
from .gemm_rs import GemmRs

_ctx: dict = {"heap": None, "plans": {}, "barrier": None, "cta_group": 2}


def init(heap_bytes: int = 2 << 30, backend: str = "ipc", multicast: bool = False, cta_group: int = 2) -> SymmetricHeap:
    """Creates the process-wide symmetric heap (collective: every rank calls it with the same size)."""
    if _ctx["heap"] is None:
        _ctx["heap"] = SymmetricHeap(heap_bytes, backend=backend, multicast=multicast)
        _ctx["cta_group"] = cta_group
    return _ctx["heap"]


def heap() -> SymmetricHeap:
    if _ctx["heap"] is None:
        raise RuntimeError("call tileccl_b200.init(heap_bytes) first (collectively on every rank)")
    return _ctx["heap"]


def shutdown() -> None:
    _ctx["plans"].clear()
    _ctx["barrier"] = None
    if _ctx["heap"] is not None:
        _ctx["heap"].close()
        _ctx["heap"] = None


def symm_empty(shape, dtype=torch.bfloat16) -> torch.Tensor:
    """A tensor in the symmetric heap (same offset on every rank; collective)."""
    return heap().empty(shape, dtype)


def _key(kind, *tensors, extra=()):
    """Cache key: the operands' layout only (never their addresses)."""
    return (kind,) + tuple((tuple(t.shape), tuple(t.stride()), str(t.dtype)) for t in tensors) + tuple(extra)


def check_all() -> None:
    """Synchronises and raises if any cached plan recorded a time-out."""
    for p in _ctx["plans"].values():
        p.check() if hasattr(p, "check") else None


_lib = torch.library.Library("tileccl", "DEF")
_lib.define("gemm(Tensor a, Tensor b_t) -> Tensor")
_lib.define("gemm_rs(Tensor a, Tensor b_t) -> Tensor")
_lib.define("ag_gemm(Tensor a_shard, Tensor b_t, int gather_rows=512) -> Tensor")
_lib.define("silu_mul(Tensor gate_up) -> Tensor")
_lib.define("barrier() -> ()")


def _gemm(a: torch.Tensor, b_t: torch.Tensor) -> torch.Tensor:
    k = _key("gemm", a, b_t)
    plan = _ctx["plans"].get(k)
    if plan is None:
        plan = _ctx["plans"][k] = GemmPlan(a, b_t, cta_group=_ctx["cta_group"] if a.shape[0] % 256 == 0 else 1, hold_operands=False)
    else:
        plan.set_operands(a, b_t)
    return plan()


def _gemm_rs(a: torch.Tensor, b_t: torch.Tensor) -> torch.Tensor:
    k = _key("gemm_rs", a, b_t)
    op = _ctx["plans"].get(k)
    if op is None:
        h = heap()
        g = _ctx["cta_group"] if (a.shape[0] // h.world) % 256 == 0 else 1
        op = _ctx["plans"][k] = GemmRs(h, a, b_t, cta_group=g, hold_operands=False)
    else:
        op.plan.set_operands(a, b_t)
    return op()


def _ag_gemm(a_shard: torch.Tensor, b_t: torch.Tensor, gather_rows: int = 512) -> torch.Tensor:
    h = heap()
    M, K = a_shard.shape[0] * h.world, a_shard.shape[1]
    k = _key("ag_gemm", b_t, extra=(M, K, gather_rows))
    op = _ctx["plans"].get(k)
    if op is None:
        g = _ctx["cta_group"] if a_shard.shape[0] % 256 == 0 else 1
        op = _ctx["plans"][k] = AgGemm(h, M, K, b_t, cta_group=g, gather_rows=gather_rows, hold_operands=False)
    else:
        op.plan.set_operands(op.a_full, b_t)
    if a_shard.data_ptr() != op.a_shard.data_ptr():
        op.a_shard.copy_(a_shard)
    return op()


def _barrier() -> None:
    if _ctx["barrier"] is None:
        _ctx["barrier"] = ew.DeviceBarrier(heap())
    _ctx["barrier"]()


_lib.impl("gemm", _gemm, "CUDA")
_lib.impl("gemm_rs", _gemm_rs, "CUDA")
_lib.impl("ag_gemm", _ag_gemm, "CUDA")
_lib.impl("silu_mul", lambda gu: ew.silu_mul(gu), "CUDA")
_lib.impl("barrier", _barrier, "CompositeExplicitAutograd")
