"""Property test of the tile schedule: for any legal parameters it is a bijection and the native
(C++) and Python versions agree."""
import ctypes as C

from hypothesis import given, settings
from hypothesis import strategies as st

from tileccl_b200.parallel import tiling


@settings(max_examples=60, deadline=None)
@given(order=st.sampled_from([0, 1, 2, 3]), world=st.integers(1, 8), seg_mult=st.integers(1, 4), chunk_pick=st.integers(0, 3),
       n_tiles=st.integers(1, 7), group_m=st.integers(1, 20), rank_pick=st.integers(0, 7))
def test_schedule_bijection_and_native_python_agreement(native_lib, order, world, seg_mult, chunk_pick, n_tiles, group_m, rank_pick):
    if order == 0:
        world = 1
    chunks_options = [c for c in (1, 2, 3, 4) if (seg_mult * 2) % c == 0]
    chunks = chunks_options[chunk_pick % len(chunks_options)] if order == 1 else 1
    seg_tiles = seg_mult * 2
    m_tiles = world * seg_tiles
    rank = rank_pick % world
    m, n = C.c_int(), C.c_int()
    got = []
    for t in range(m_tiles * n_tiles):
        native_lib.tcl_sched_tile(m_tiles, n_tiles, group_m, order, world, rank, chunks, t, C.byref(m), C.byref(n))
        got.append((m.value, n.value))
    assert sorted(got) == [(a, b) for a in range(m_tiles) for b in range(n_tiles)]
    assert got == tiling.schedule(m_tiles, n_tiles, group_m, order, world, rank, chunks)
