"""CPU oracles (plain fp32) for the fused ops, world simulated in-process.

The reference has no CPU oracle: it verifies on the GPU against an fp32
re-computation (comm_comp/exp3_gemm_rs_fused.cu:248-270) or bit-wise against
its own un-fused run (comm_comp/exp2_ag_gemm_granularity.cu:511-533).
"""
from __future__ import annotations

import numpy as np


def normal_inputs(world: int, M: int, N: int, K_local: int, seed: int = 0, dtype=np.float32):
    """Per-rank A_r [M, K_local] and B_r [K_local, N] ~ N(0, 1), one generator, fixed order."""
    rng = np.random.default_rng(seed)
    A = [rng.standard_normal((M, K_local)).astype(dtype) for _ in range(world)]
    B = [rng.standard_normal((K_local, N)).astype(dtype) for _ in range(world)]
    return A, B


def gemm_rs(A_list, B_list):
    """sum_r A_r @ B_r, rows scattered: returns one [M/world, N] shard per rank."""
    world = len(A_list)
    total = np.zeros((A_list[0].shape[0], B_list[0].shape[1]), dtype=np.float64)
    for a, b in zip(A_list, B_list):
        total += a.astype(np.float64) @ b.astype(np.float64)
    M = total.shape[0]
    if M % world:
        raise ValueError("M must be divisible by world")
    seg = M // world
    return [total[r * seg:(r + 1) * seg].astype(np.float32) for r in range(world)]


def ag_gemm(A_shards, B_list):
    """concat_r(A_r) @ B_r for every rank r: returns one [M, N_r] block per rank."""
    A_full = np.concatenate([a.astype(np.float64) for a in A_shards], axis=0)
    return [(A_full @ b.astype(np.float64)).astype(np.float32) for b in B_list]


def silu_mul(gate_up: np.ndarray) -> np.ndarray:
    """silu(gate) * up with gate = left half of the columns, up = right half."""
    f = gate_up.shape[1] // 2
    g = gate_up[:, :f].astype(np.float64)
    u = gate_up[:, f:].astype(np.float64)
    return (g / (1.0 + np.exp(-g)) * u).astype(np.float32)


def tp_mlp(x_shards, w_gate_up_list, w_down_list):
    """Tensor-parallel gated MLP forward, sequence-sharded in and out.

    x_shards[r]: [T/world, H]; w_gate_up_list[r]: [H, 2*F/world] (gate | up);
    w_down_list[r]: [F/world, H].  Returns the [T/world, H] shard of every rank.
    """
    hs = ag_gemm(x_shards, w_gate_up_list)
    acts = [silu_mul(h) for h in hs]
    return gemm_rs(acts, w_down_list)


def max_rel_err(got: np.ndarray, ref: np.ndarray) -> float:
    """The reference's metric: max |got - ref| / (|ref| + 1)."""
    return float(np.max(np.abs(got.astype(np.float64) - ref) / (np.abs(ref) + 1.0)))
