"""Fused all-gather -> GEMM (tensor-parallel column-parallel linear).

Every rank holds a row shard ``A_r`` [M/world, K] and a local ``Bt`` [N_local,
K]; the result on every rank is ``concat_r(A_r) @ Bt.T`` = [M, N_local].  The
shard lives inside the rank's gathered buffer (symmetric heap), so the local
part needs no copy; gather warps of the GEMM kernel pull the peers' shards with
P2P loads and the TMA producer starts on a row block as soon as its counter
says it has landed.  ``gather_rows`` is the granularity of those counters,
``item_rows`` the rows one gather warp moves at a time (one row by default, so
that rows land progressively in the order the tile schedule consumes them).
``transport="push"`` makes every rank store its shard into all peers' buffers
instead; measured at 8 GPUs it is slower than pull (2.0 ms against 1.38 ms on
the 32768 x 3584 x 8192 case) and is kept as the measured alternative.

Co-residency: the gather work is dealt over the gather warps of every CTA of the grid, and every CTA's
TMA producer waits for row blocks that other CTAs gather.  The kernel therefore needs all its CTAs resident
at the same time: one CTA per SM, grid <= number of SMs that are free.  If another kernel holds SMs while
this one runs (an NCCL kernel, a copy kernel on a second stream), resident CTAs wait for CTAs that cannot
start, and the call ends with the "gathered row block never arrived" status after the time-out instead of
hanging.  Callers that overlap other kernels pass ``num_ctas`` (a multiple of ``cta_group``) small enough to
leave those kernels their SMs.  The fused GEMM + reduce-scatter has the same requirement across ranks only
(its reduce warps wait for peers, not for other CTAs of the same grid).

Reference parity: comm_comp/exp2_ag_gemm_granularity.cu:168-300 (the
segmented-launch + copy-engine pipeline; its chunk count S is this op's
``gather_rows``), and :15-20 of that file for the in-kernel form built here.
"""
from __future__ import annotations

import torch

from .. import _native
from ..parallel import group as G
from ..parallel.heap import SymmetricHeap
from ._plan import Plan, require_bf16_rowmajor


class AgGemm:
    def __init__(self, heap: SymmetricHeap, M: int, K: int, Bt: torch.Tensor, cta_group: int = 2,
                 gather_rows: int = 512, out: torch.Tensor | None = None, group_m: int = 0,
                 num_ctas: int = 0, comm_enabled: bool = True, timeout_ms: float = 4000.0, ablate: int = 0, transport: str = "pull", item_rows: int = 1, epi: str | None = None,
                 device_epoch: bool = False, hold_operands: bool = True, gather_warps: int = 0, vec32: bool = False):
        require_bf16_rowmajor(Bt, "Bt")
        self.heap = heap
        world, rank = heap.world, heap.rank
        if transport not in ("push", "pull"):
            raise ValueError("transport must be 'push' or 'pull'")
        self.transport = transport
        N = Bt.shape[0]
        if Bt.shape[1] != K:
            raise ValueError("Bt must be [N, K]")
        seg = M // world
        if M % world or seg % (128 * cta_group):
            raise ValueError("M / world must be a multiple of 128 * cta_group")
        gather_rows = min(gather_rows, seg)
        self.a_full = heap.empty((M, K), torch.bfloat16)
        self.flags = heap.zeros((M // 128 + 32,), torch.int32)
        self.done = heap.zeros((32,), torch.int32)       # [0] gather warps done, [16] peers done reading
        self.barrier = heap.zeros((32,), torch.int32)
        self.a_shard = self.a_full[rank * seg:(rank + 1) * seg]
        if epi not in (None, "silu_mul"):
            raise ValueError("epi must be None or 'silu_mul'")
        n_out = N // 2 if epi == "silu_mul" else N      # silu_mul: Bt in the interleave_gate_up layout
        if out is None:
            out = torch.empty(M, n_out, dtype=torch.bfloat16, device=Bt.device)
        if tuple(out.shape) != (M, n_out):
            raise ValueError(f"out must be [{M}, {n_out}]")
        self.out = out
        d = _native.GemmDesc()
        d.mode, d.cta_group = _native.MODE_AG_GEMM, cta_group
        d.M, d.N, d.K = M, N, K
        d.lda, d.ldb, d.ldc = K, Bt.stride(0), out.stride(0)
        d.A, d.B = self.a_full.data_ptr(), Bt.data_ptr()
        d.world, d.rank = world, rank
        d.seg_rows = M            # the output is one local segment
        d.comm_enabled = 1 if comm_enabled else 0
        d.dst_base[0] = out.data_ptr()
        d.dst_row_off[0] = 0
        d.seg_rows = seg
        for s in range(world):
            d.dst_base[s] = out.data_ptr()
            d.dst_row_off[s] = s * seg
            d.ag_src[s] = heap.peer_ptr(self.a_full, s) + s * seg * K * 2
            d.ag_read_done[s] = heap.peer_ptr(self.done, s) + 16 * 4
            d.barrier[s] = heap.peer_ptr(self.barrier, s)
            d.ag_dst[s] = heap.peer_ptr(self.a_full, s)
            d.ag_flag_peer[s] = heap.peer_ptr(self.flags, s)
        d.ag_push = 1 if transport == "push" else 0
        d.epi_silu_mul = 1 if epi == "silu_mul" else 0
        d.ag_flags = self.flags.data_ptr()
        for s in range(world):   # debug build: the only memory of rank s this plan may touch is its heap
            d.range_lo[s] = heap.base[s]
            d.range_hi[s] = heap.base[s] + heap.nbytes
        d.gather_rows = gather_rows
        d.ag_item_rows = item_rows
        d.ag_warps = gather_warps          # gather warps per CTA that take part (0 = all four)
        d.ag_vec32 = 1 if vec32 else 0     # 32-byte gather loads and stores instead of 16-byte ones
        self.item_rows = item_rows
        d.ag_done = self.done.data_ptr()
        d.timeout_ns = int(timeout_ms * 1e6)
        d.group_m, d.num_ctas = group_m, num_ctas
        d.ablate = ablate
        own = (out, self.a_full, self.flags, self.done, self.barrier)
        self.plan = Plan(d, keep_alive=((Bt,) + own) if hold_operands else own, device_epoch=device_epoch)
        self.gather_rows = gather_rows
        # Construction is collective.  It ends with a host barrier behind a device synchronise: the counters
        # zeroed above are zero on every rank before any rank's first launch can signal them.
        if world > 1:
            torch.cuda.synchronize()
            G.host_barrier(heap.group)

    def __call__(self, stream=None) -> torch.Tensor:
        self.plan.run(stream)
        return self.out

    def check(self) -> None:
        self.plan.check()

    def audit(self) -> None:
        """Flag audit after a run: every gathered row block of a peer segment stands at
        epoch * (gather_rows / item_rows) arrivals, the local segment's flags were never touched, and all
        peers reported that they finished reading this rank's shard.  Synchronises."""
        h = self.heap
        if h.world == 1 or not self.plan.desc.comm_enabled or self.plan.desc.ablate:
            return
        M = self.a_full.shape[0]
        seg = M // h.world
        per = self.gather_rows // self.item_rows * self.plan.epoch
        flags = self.flags[: M // self.gather_rows].tolist()
        for b, v in enumerate(flags):
            own = (b * self.gather_rows) // seg == h.rank
            if v != (0 if own else per):
                raise AssertionError(f"gather flag {b} is {v}, expected {0 if own else per}")
        if self.transport == "pull" and int(self.done[16]) != self.plan.epoch * (h.world - 1):
            raise AssertionError("not every peer reported the end of its reads")

    @property
    def launches(self) -> int:
        return self.plan.launches
