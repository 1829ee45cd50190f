"""Fused GEMM -> reduce-scatter (tensor-parallel row-parallel linear).

Every rank holds ``A_r`` [M, K_local] and ``Bt_r`` [N, K_local]; the result is
``sum_r A_r @ Bt_r.T`` with the M rows scattered: rank r gets rows
[r*M/world, (r+1)*M/world).  One kernel per rank does both: the GEMM epilogue
pushes bf16 partial tiles into the owner's staging slot over NVLink and the
owner's reduce warps sum them in fp32 as tiles complete.

Reference parity: comm_comp/exp3_gemm_rs_fused.cu:195-238,423-442 (RsRunner and
its base / ctrl / fused variants), comm_comp/rs_dma_sm90.cuh:93-176.
"""
from __future__ import annotations

import torch

from .. import _native
from ..parallel import group as G
from ..parallel.heap import SymmetricHeap
from ._plan import Plan, require_bf16_rowmajor


def staging_bytes(M: int, N: int, world: int) -> int:
    """Symmetric-heap bytes a :class:`GemmRs` of this shape takes per rank."""
    tiles = (M // world // 128) * (N // 256)
    return M * N * 2 + (M // world) * N * 2 + tiles * 4 + 4096 + 8 * 1024


class GemmRs:
    def __init__(self, heap: SymmetricHeap, A: torch.Tensor, Bt: torch.Tensor, cta_group: int = 2,
                 rs_chunks: int = 0, comm_enabled: bool = True, group_m: int = 0, num_ctas: int = 0,
                 timeout_ms: float = 4000.0, ablate: int = 0, force_staged: bool = False, transport: str = "p2p",
                 st256: bool = False, device_epoch: bool = False, hold_operands: bool = True, signal_batch: int = 0):
        require_bf16_rowmajor(A, "A")
        require_bf16_rowmajor(Bt, "Bt")
        self.heap = heap
        world, rank = heap.world, heap.rank
        if transport not in ("p2p", "nvls"):
            raise ValueError("transport must be 'p2p' or 'nvls'")
        nvls = transport == "nvls" and world > 1 and comm_enabled
        if nvls and heap.mc_base is None:
            raise ValueError("transport='nvls' needs a heap with a multicast mapping (backend='vmm', multicast=True)")
        self.transport = "nvls" if nvls else "p2p"
        M, K = A.shape
        N = Bt.shape[0]
        if M % world:
            raise ValueError("M must be divisible by the world size")
        seg = M // world
        tile_m = 128 * cta_group
        if seg % tile_m:
            raise ValueError(f"M / world must be a multiple of {tile_m}")
        # Symmetric objects: staging [world][seg][N], per-tile counters, barrier counter.
        self.stage = heap.empty((world, seg, N), torch.bfloat16)
        self.tile_cnt = heap.zeros(((seg // 128) * (N // 256),), torch.int32)
        self.barrier = heap.zeros((32,), torch.int32)
        self.out = heap.empty((seg, N), torch.bfloat16)
        d = _native.GemmDesc()
        d.mode, d.cta_group = _native.MODE_GEMM_RS, cta_group
        d.M, d.N, d.K = M, N, K
        d.lda, d.ldb, d.ldc = A.stride(0), Bt.stride(0), N
        d.A, d.B = A.data_ptr(), Bt.data_ptr()
        d.world, d.rank = world, rank
        d.seg_rows = seg
        if world == 1 and comm_enabled and not force_staged:
            # One rank: nothing to reduce, the epilogue writes the result itself.
            comm_enabled = False
            self._direct = True
        else:
            self._direct = False
        d.comm_enabled = 1 if comm_enabled else 0
        for s in range(world):
            if self._direct:
                d.dst_base[s] = self.out.data_ptr()
                d.dst_row_off[s] = 0
            elif nvls:
                # NVLS: partial tiles stay in this rank's own staging at their global row; owners pull sums
                d.dst_base[s] = self.stage.data_ptr()
                d.dst_row_off[s] = s * seg
            elif comm_enabled:
                # Segment s goes to rank s's staging, slot `rank`.
                d.dst_base[s] = heap.peer_ptr(self.stage, s)
                d.dst_row_off[s] = rank * seg
            else:
                # ctrl variant: same schedule, every store stays local.
                d.dst_base[s] = self.stage.data_ptr()
                d.dst_row_off[s] = s * seg
            d.rs_tile_cnt[s] = heap.peer_ptr(self.tile_cnt, s)
            d.barrier[s] = heap.peer_ptr(self.barrier, s)
        d.rs_stage = self.stage.data_ptr()
        for s in range(world):   # debug build: the only memory of rank s this plan may touch is its heap
            d.range_lo[s] = heap.base[s]
            d.range_hi[s] = heap.base[s] + heap.nbytes
        d.rs_out = self.out.data_ptr()
        d.ld_out = N
        d.rs_chunks = rs_chunks
        d.rs_mc_stage = heap.mc_ptr(self.stage) if nvls else None
        d.timeout_ns = int(timeout_ms * 1e6)
        d.group_m, d.num_ctas = group_m, num_ctas
        d.ablate = ablate
        d.rs_signal_batch = signal_batch      # finished tiles per system-scope fence of the signalling warp (0 = default)
        d.epi_st256 = 1 if st256 else 0    # 32-byte epilogue stores (st.global.v8.b32) instead of 16-byte ones
        # hold_operands=False: the caller re-points the plan with plan.set_operands() and owns the operands' lifetime
        own = (self.stage, self.tile_cnt, self.barrier, self.out)
        self.plan = Plan(d, keep_alive=((A, Bt) + own) if hold_operands else own, device_epoch=device_epoch)
        self.rs_chunks = rs_chunks
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
        """Flag audit after a run: every per-tile counter of this rank stands at epoch * world (each
        producer signalled each tile exactly once per call).  Synchronises."""
        if self._direct or not self.plan.desc.comm_enabled or self.plan.desc.ablate:
            return
        want = self.plan.epoch * self.heap.world
        bad = (self.tile_cnt != want).nonzero()
        if bad.numel():
            i = int(bad[0])
            raise AssertionError(f"tile counter {i} is {int(self.tile_cnt[i])}, expected {want}")

    @property
    def launches(self) -> int:
        return self.plan.launches
