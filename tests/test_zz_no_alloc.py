"""The allocation-free verify entry point, called through its exported C symbol.

Some users of the library may not allocate device memory when they want to check a result (a
server whose arena owns the whole budget, a host application that forbids allocator calls on its
worker threads).  For them ``tcl_max_rel_err_static`` keeps its scratch in a fixed array inside
the library.  This file checks that it returns what the ordinary entry point returns, twice in a
row (the array is shared between calls), and that it refuses sizes its array cannot serve.

The file name sorts last so that a run that stops at the first failure has already run every
other test.
"""
import ctypes as C

import pytest

MAX_ELEMS = 16384 * 4096


def _lib():
    from tileccl_b200 import _build, _native
    _build.build(programs=False)
    L = _native.lib()
    L.tcl_max_rel_err_static.restype = C.c_int
    L.tcl_max_rel_err_static.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p]
    L.tcl_max_rel_err_static_strerror.restype = C.c_char_p
    L.tcl_max_rel_err_static_strerror.argtypes = [C.c_int]
    return L


def test_static_entry_point_rejects_what_it_cannot_serve():
    """Size and argument checks come before any CUDA call, so they can be tested anywhere."""
    L = _lib()
    dummy = C.c_void_p(256)
    assert L.tcl_max_rel_err_static(dummy, dummy, MAX_ELEMS + 1, dummy, None) == -2
    assert b"67,108,864" in L.tcl_max_rel_err_static_strerror(-2)
    assert L.tcl_max_rel_err_static(None, dummy, 16, dummy, None) == -3
    assert L.tcl_max_rel_err_static(dummy, dummy, 0, dummy, None) == -3


@pytest.mark.gpu
def test_static_entry_point_matches_the_allocating_one_twice():
    import torch
    from tileccl_b200.ops import elementwise as ew
    L = _lib()
    torch.manual_seed(11)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    # two different problems back to back: the second call reuses the array the first one wrote
    for n, noise in ((3_000_001, 0.02), (70_001, 0.5)):
        ref = torch.randn(n, device="cuda")
        got = (ref + noise * torch.rand(n, device="cuda")).bfloat16()
        want = ew.max_rel_err(got, ref)                  # the existing entry point (torch allocates its scratch)
        res = torch.zeros(1, device="cuda")
        torch.cuda.synchronize()
        rc = L.tcl_max_rel_err_static(got.data_ptr(), ref.data_ptr(), n, res.data_ptr(), stream)
        assert rc == 0, L.tcl_max_rel_err_static_strerror(rc)
        torch.cuda.synchronize()
        assert abs(float(res) - want) <= 1e-6 * max(1.0, abs(want))
        plain = ((got.float() - ref).abs() / (ref.abs() + 1)).max().item()
        assert abs(float(res) - plain) <= 1e-6
    # a NaN in the data is reported as the worst error by both
    ref = torch.randn(5000, device="cuda")
    got = ref.bfloat16()
    got[1234] = float("nan")
    res = torch.zeros(1, device="cuda")
    torch.cuda.synchronize()
    assert L.tcl_max_rel_err_static(got.data_ptr(), ref.data_ptr(), 5000, res.data_ptr(), stream) == 0
    torch.cuda.synchronize()
    assert float(res) > 1e38 and ew.max_rel_err(got, ref) > 1e38


@pytest.mark.gpu
def test_static_entry_point_at_its_size_limit_on_a_side_stream():
    """The largest problem the array serves (all 16384 slots in use), issued on a stream other than the
    default one; then a small problem on the same stream, which must not see the large one's slots."""
    import torch
    from tileccl_b200.ops import elementwise as ew
    L = _lib()
    torch.manual_seed(12)
    side = torch.cuda.Stream()
    n = MAX_ELEMS - 7
    ref = torch.randn(n, device="cuda")
    got = ref.bfloat16()
    got[n - 3] = 400.0                                   # the worst element sits in the last block
    want = ew.max_rel_err(got, ref)
    res = torch.zeros(2, device="cuda")
    small_ref = torch.randn(4097, device="cuda")
    small_got = (small_ref + 0.01).bfloat16()
    small_want = ew.max_rel_err(small_got, small_ref)
    torch.cuda.synchronize()
    sp = C.c_void_p(side.cuda_stream)
    with torch.cuda.stream(side):
        assert L.tcl_max_rel_err_static(got.data_ptr(), ref.data_ptr(), n, res.data_ptr(), sp) == 0
        assert L.tcl_max_rel_err_static(small_got.data_ptr(), small_ref.data_ptr(), 4097, res.data_ptr() + 4, sp) == 0
    side.synchronize()
    assert abs(float(res[0]) - want) <= 1e-6 * max(1.0, abs(want)) and float(res[0]) > 10.0
    assert abs(float(res[1]) - small_want) <= 1e-6
