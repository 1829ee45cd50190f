"""The persistent tile schedule: bijection, raster grouping and the
collective-aware M orders (host build of csrc/gemm/tile_sched.hpp)."""
import ctypes as C

import pytest

from tileccl_b200 import _native
from tileccl_b200.parallel import tiling


def _tiles(lib, m_tiles, n_tiles, group_m, order, world, rank, chunks):
    out = []
    m, n = C.c_int(), C.c_int()
    for t in range(m_tiles * n_tiles):
        lib.tcl_sched_tile(m_tiles, n_tiles, group_m, order, world, rank, chunks, t, C.byref(m), C.byref(n))
        out.append((m.value, n.value))
    return out


@pytest.mark.parametrize("order,world,chunks", [
    (_native.ORDER_PLAIN, 1, 1), (_native.ORDER_RS_PUSH, 2, 2), (_native.ORDER_RS_PUSH, 8, 4),
    (_native.ORDER_RS_PUSH, 3, 1), (_native.ORDER_AG_PULL, 4, 1), (_native.ORDER_AG_PULL, 7, 1),
    (_native.ORDER_AG_PUSH, 2, 1), (_native.ORDER_AG_PUSH, 8, 1), (_native.ORDER_AG_PUSH, 5, 1)])
@pytest.mark.parametrize("group_m", [1, 3, 8])
def test_schedule_is_a_bijection(native_lib, order, world, chunks, group_m):
    seg_tiles = 4 * chunks
    m_tiles, n_tiles = world * seg_tiles, 5
    for rank in range(world):
        tiles = _tiles(native_lib, m_tiles, n_tiles, group_m, order, world, rank, chunks)
        assert sorted(tiles) == [(m, n) for m in range(m_tiles) for n in range(n_tiles)]
        assert tiles == tiling.schedule(m_tiles, n_tiles, group_m, order, world, rank, chunks)


def test_rs_order_own_segment_last_and_peers_balanced():
    world, seg_tiles, chunks = 4, 4, 2
    rows = {r: [tiling.m_of_row(p, world * seg_tiles, order=_native.ORDER_RS_PUSH, world=world, rank=r, rs_chunks=chunks)
                for p in range(world * seg_tiles)] for r in range(world)}
    cpr = seg_tiles // chunks
    for r in range(world):
        segs = [m // seg_tiles for m in rows[r]]
        # inside every round the own segment comes last
        for g in range(chunks):
            rnd = segs[g * world * cpr:(g + 1) * world * cpr]
            assert rnd[-1] == r and rnd[0] == (r + 1) % world
    # at every schedule position the ranks target pairwise different owners
    for p in range(world * seg_tiles):
        assert len({rows[r][p] // seg_tiles for r in range(world)}) == world


def test_rs_rounds_complete_chunks_in_order():
    world, seg_tiles, chunks = 4, 8, 4
    cpr = seg_tiles // chunks
    for r in range(world):
        ms = [tiling.m_of_row(p, world * seg_tiles, _native.ORDER_RS_PUSH, world, r, chunks) for p in range(world * seg_tiles)]
        for g in range(chunks):
            rnd = ms[g * world * cpr:(g + 1) * world * cpr]
            assert {m % seg_tiles // cpr for m in rnd} == {g}


def test_ag_order_own_segment_first():
    world, seg_tiles = 4, 3
    for r in range(world):
        ms = [tiling.m_of_row(p, world * seg_tiles, _native.ORDER_AG_PULL, world, r, 1) for p in range(world * seg_tiles)]
        assert [m // seg_tiles for m in ms[:seg_tiles]] == [r] * seg_tiles
        assert ms[seg_tiles] // seg_tiles == (r + 1) % world


def test_owner_and_counter_index():
    # tile row -> owner rank and the owner's per-tile counter index
    assert tiling.owner_of_row(row=4096 + 130, seg_rows=4096) == 1
    assert tiling.rs_counter_index(row=4096 + 256, col=512, seg_rows=4096, n_cols=8192) == 2 * 32 + 2
    assert tiling.gather_flag_index(row=5000, gather_rows=512) == 9


def test_ag_push_order_follows_arrival():
    world, seg_tiles = 4, 3
    for r in range(world):
        ms = [tiling.m_of_row(p, world * seg_tiles, _native.ORDER_AG_PUSH, world, r, 1) for p in range(world * seg_tiles)]
        assert [m // seg_tiles for m in ms[:seg_tiles]] == [r] * seg_tiles          # own segment first
        rest = ms[seg_tiles:]
        # then tile row i of every peer before tile row i + 1 of any peer
        assert [m % seg_tiles for m in rest] == [i for i in range(seg_tiles) for _ in range(world - 1)]
        assert {m // seg_tiles for m in rest[:world - 1]} == set(range(world)) - {r}


def test_rs_order_spreads_the_tiles_in_flight_over_all_owners():
    """GEMM+RS at the headline shape (128 tile rows x 32 tile columns, 74 CTA pairs): whatever 74 consecutive
    tiles are in flight, every owner receives the same share of them (+-1), so no rank's ingress is a hot spot."""
    from collections import Counter
    m_tiles, n_tiles, in_flight = 128, 32, 74
    for world in (2, 4, 8):
        st = m_tiles // world
        group_m = world * max(1, 8 // world)            # the plan's default raster group: one round of owners
        for rank in (0, world - 1):
            tiles = tiling.schedule(m_tiles, n_tiles, group_m, tiling.ORDER_RS_PUSH, world, rank, st)
            for t0 in range(0, len(tiles) - in_flight, 7):
                c = Counter(m // st for m, _ in tiles[t0:t0 + in_flight])
                assert max(c.values()) - min(c.get(o, 0) for o in range(world)) <= 1, (world, rank, t0, c)
            # the own segment is the last step of every round
            assert all(tiles[i][0] // st == rank for i in range(world - 1, group_m, world))
