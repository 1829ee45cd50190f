"""Plain bf16 GEMM on the tcgen05 kernel: ``D = A @ Bt.T``.

``A`` is [M, K], ``Bt`` is [N, K] (the K-major "column-major B[K, N]" that the
reference's GEMM takes, comm_comp/gemm_sm90.cuh:40-46), ``D`` is [M, N].  This
is the in-repo control GEMM; the baseline GEMM is cuBLAS (``torch.matmul``).
"""
from __future__ import annotations

import torch

from .. import _native
from ._plan import Plan, require_bf16_rowmajor


class GemmPlan(Plan):
    def __init__(self, A: torch.Tensor, Bt: torch.Tensor, out: torch.Tensor | None = None,
                 cta_group: int = 2, group_m: int = 0, num_ctas: int = 0, timeout_ms: float = 4000.0,
                 dst_ptrs: list[int] | None = None, seg_rows: int | None = None, epi: str | None = None,
                 store: str = "st16", hold_operands: bool = True):
        """``dst_ptrs``/``seg_rows`` route row segments of D to other addresses
        (a peer's buffer): the epilogue-remote experiment.  ``store`` picks how the epilogue leaves the
        SM: ``st16`` (16-byte st.global, the default), ``st256`` (32-byte st.global.v8.b32) or ``tma``
        (cp.async.bulk.tensor stores from the staging buffer), the counterparts of the reference's
        direct-store and TMA-store epilogues (comm_comp/gemm_sm90.cuh:83-88)."""
        if store not in ("st16", "st256", "tma"):
            raise ValueError("store must be st16, st256 or tma")
        require_bf16_rowmajor(A, "A")
        require_bf16_rowmajor(Bt, "Bt")
        M, K = A.shape
        N, K2 = Bt.shape
        if K2 != K:
            raise ValueError("A is [M, K] and Bt is [N, K]: K differs")
        if epi not in (None, "silu_mul"):
            raise ValueError("epi must be None or 'silu_mul'")
        n_out = N // 2 if epi == "silu_mul" else N
        if out is None:
            out = torch.empty(M, n_out, dtype=torch.bfloat16, device=A.device)
        if out.shape != (M, n_out):
            raise ValueError(f"out must be [{M}, {n_out}]")
        require_bf16_rowmajor(out, "out")
        d = _native.GemmDesc()
        d.mode, d.cta_group = _native.MODE_PLAIN, cta_group
        d.M, d.N, d.K = M, N, K
        d.lda, d.ldb, d.ldc = A.stride(0), Bt.stride(0), out.stride(0)
        d.A, d.B = A.data_ptr(), Bt.data_ptr()
        d.world, d.rank = 1, 0
        d.seg_rows = seg_rows or M
        nseg = M // d.seg_rows
        for s in range(nseg):
            d.dst_base[s] = dst_ptrs[s] if dst_ptrs else out.data_ptr()
            # With an explicit pointer per segment the segment starts at row 0 of it.
            d.dst_row_off[s] = 0 if dst_ptrs else s * d.seg_rows
        d.timeout_ns = int(timeout_ms * 1e6)
        d.group_m, d.num_ctas = group_m, num_ctas
        d.epi_silu_mul = 1 if epi == "silu_mul" else 0
        d.epi_st256 = 1 if store == "st256" else 0
        d.epi_tma_store = 1 if store == "tma" else 0
        # hold_operands=False: the caller re-points the plan with set_operands() and owns the operands' lifetime
        super().__init__(d, keep_alive=(A, Bt, out) if hold_operands else (out,))
        self.out = out

    def __call__(self, stream=None) -> torch.Tensor:
        self.run(stream)
        return self.out


def interleave_gate_up(w_gate: torch.Tensor, w_up: torch.Tensor) -> torch.Tensor:
    """[F, K] gate and up weights -> one [2F, K] weight whose 256-row blocks hold 128 gate rows
    followed by the 128 up rows of the same features: the layout the ``silu_mul`` epilogue expects
    (every 256-column output tile then carries matching gate and up columns).  F % 128 == 0."""
    F, K = w_gate.shape
    if w_up.shape != (F, K) or F % 128:
        raise ValueError("gate and up must both be [F, K] with F a multiple of 128")
    return torch.stack([w_gate.view(F // 128, 128, K), w_up.view(F // 128, 128, K)], dim=1).reshape(2 * F, K).contiguous()


def deinterleave_gate_up(w: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Inverse of :func:`interleave_gate_up`."""
    two_f, K = w.shape
    v = w.view(two_f // 256, 2, 128, K)
    return v[:, 0].reshape(two_f // 2, K), v[:, 1].reshape(two_f // 2, K)


def gemm(A: torch.Tensor, Bt: torch.Tensor, cta_group: int = 2) -> torch.Tensor:
    """One-shot convenience wrapper (builds a plan per call)."""
    plan = GemmPlan(A, Bt, cta_group=cta_group)
    out = plan()
    plan.check()
    return out
