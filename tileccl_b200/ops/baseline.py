"""The baseline every fused op is measured against: cuBLAS + NCCL, sequential.

``torch.matmul`` (cuBLAS/cuBLASLt) followed or preceded by the NCCL collective
of ``torch.distributed``.  Nothing here is on a product path.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def gemm_rs_baseline(A: torch.Tensor, Bt: torch.Tensor, out: torch.Tensor | None = None,
                     full: torch.Tensor | None = None, group=None) -> torch.Tensor:
    """cuBLAS GEMM into a full [M, N] buffer, then ncclReduceScatter."""
    M, N = A.shape[0], Bt.shape[0]
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if full is None:
        full = torch.empty(M, N, dtype=A.dtype, device=A.device)
    torch.matmul(A, Bt.t(), out=full)
    if world == 1:
        return full
    if out is None:
        out = torch.empty(M // world, N, dtype=A.dtype, device=A.device)
    dist.reduce_scatter_tensor(out, full, group=group)
    return out


def ag_gemm_baseline(A_shard: torch.Tensor, Bt: torch.Tensor, gathered: torch.Tensor | None = None,
                     out: torch.Tensor | None = None, group=None) -> torch.Tensor:
    """ncclAllGather of the row shards, then one cuBLAS GEMM."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        gathered = A_shard
    else:
        if gathered is None:
            gathered = torch.empty(A_shard.shape[0] * world, A_shard.shape[1], dtype=A_shard.dtype, device=A_shard.device)
        dist.all_gather_into_tensor(gathered, A_shard, group=group)
    if out is None:
        out = torch.empty(gathered.shape[0], Bt.shape[0], dtype=A_shard.dtype, device=A_shard.device)
    torch.matmul(gathered, Bt.t(), out=out)
    return out
