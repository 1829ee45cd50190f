"""Python mirror of the device tile schedule (csrc/gemm/tile_sched.hpp) and of
the index arithmetic the fused kernels use for owners, counters and flags.

Used by host-side planning, by the analysis scripts (ns per tile) and by the
CPU tests that cross-check the native schedule.  The reference's counterpart is
the XOR segment swizzle of its fused kernel
(comm_comp/rs_gemm_kernel_sm90.cuh:321-330), which needs a power-of-two world.
"""
from __future__ import annotations

ORDER_PLAIN, ORDER_RS_PUSH, ORDER_AG_PULL, ORDER_AG_PUSH = 0, 1, 2, 3
TILE_N = 256
CTA_M = 128


def m_of_row(p: int, m_tiles: int, order: int = ORDER_PLAIN, world: int = 1, rank: int = 0, rs_chunks: int = 1) -> int:
    """Schedule row ``p`` -> tile row, for one rank."""
    st = m_tiles // world
    if order == ORDER_RS_PUSH:
        cpr = st // rs_chunks
        per_round = world * cpr
        g, q = divmod(p, per_round)
        step, i = divmod(q, cpr)
        seg = (rank + 1 + step) % world
        return seg * st + g * cpr + i
    if order == ORDER_AG_PUSH:
        if p < st:
            return rank * st + p
        i, step = divmod(p - st, world - 1)
        return ((rank + step + 1) % world) * st + i
    if order == ORDER_AG_PULL:
        step, i = divmod(p, st)
        return ((rank + step) % world) * st + i
    return p


def schedule(m_tiles: int, n_tiles: int, group_m: int, order: int = ORDER_PLAIN, world: int = 1,
             rank: int = 0, rs_chunks: int = 1) -> list[tuple[int, int]]:
    """The whole work list [(m_blk, n_blk)] in execution order."""
    out = []
    per_group = group_m * n_tiles
    for t in range(m_tiles * n_tiles):
        grp, rem = divmod(t, per_group)
        first = grp * group_m
        gm = min(group_m, m_tiles - first)
        n, r = divmod(rem, gm)
        out.append((m_of_row(first + r, m_tiles, order, world, rank, rs_chunks), n))
    return out


def owner_of_row(row: int, seg_rows: int) -> int:
    return row // seg_rows


def rs_counter_index(row: int, col: int, seg_rows: int, n_cols: int) -> int:
    """Index of the owner's counter for the 128x256 tile holding (row, col)."""
    return (row % seg_rows) // CTA_M * (n_cols // TILE_N) + col // TILE_N


def gather_flag_index(row: int, gather_rows: int) -> int:
    return row // gather_rows
