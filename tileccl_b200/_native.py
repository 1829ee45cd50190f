"""ctypes binding of ``libtileccl.so``.

The library is loaded from the source tree (``tileccl_b200/lib``).  If a CUDA
device is present and the library is missing or fails to load, importing this
module raises: there is no PyTorch fallback for the kernels.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

MAX_WORLD = 8
MODE_PLAIN, MODE_GEMM_RS, MODE_AG_GEMM = 0, 1, 2
ORDER_PLAIN, ORDER_RS_PUSH, ORDER_AG_PULL, ORDER_AG_PUSH = 0, 1, 2, 3

import os as _os

# TILECCL_DEBUG=1 selects the build with device-side address checks (libtileccl_debug.so).
_LIB_PATH = Path(__file__).resolve().parent / "lib" / ("libtileccl_debug.so" if _os.environ.get("TILECCL_DEBUG") == "1" else "libtileccl.so")


class GemmDesc(C.Structure):
    """Mirror of ``tcl_gemm_desc`` (csrc/ops/tileccl_ops.h)."""

    _fields_ = [
        ("mode", C.c_int32),
        ("cta_group", C.c_int32),
        ("M", C.c_int32),
        ("N", C.c_int32),
        ("K", C.c_int32),
        ("lda", C.c_int32),
        ("ldb", C.c_int32),
        ("ldc", C.c_int32),
        ("A", C.c_void_p),
        ("B", C.c_void_p),
        ("world", C.c_int32),
        ("rank", C.c_int32),
        ("seg_rows", C.c_int32),
        ("comm_enabled", C.c_int32),
        ("dst_base", C.c_void_p * MAX_WORLD),
        ("dst_row_off", C.c_int64 * MAX_WORLD),
        ("rs_tile_cnt", C.c_void_p * MAX_WORLD),
        ("rs_stage", C.c_void_p),
        ("rs_out", C.c_void_p),
        ("ld_out", C.c_int32),
        ("rs_chunks", C.c_int32),
        ("ag_src", C.c_void_p * MAX_WORLD),
        ("ag_flags", C.c_void_p),
        ("gather_rows", C.c_int32),
        ("ag_item_rows", C.c_int32),
        ("ag_done", C.c_void_p),
        ("ag_read_done", C.c_void_p * MAX_WORLD),
        ("ag_push", C.c_int32),
        ("ag_dst", C.c_void_p * MAX_WORLD),
        ("ag_flag_peer", C.c_void_p * MAX_WORLD),
        ("barrier", C.c_void_p * MAX_WORLD),
        ("status", C.c_void_p),
        ("timeout_ns", C.c_uint64),
        ("group_m", C.c_int32),
        ("num_ctas", C.c_int32),
        ("rs_mc_stage", C.c_void_p),
        ("range_lo", C.c_uint64 * MAX_WORLD),
        ("range_hi", C.c_uint64 * MAX_WORLD),
        ("epi_silu_mul", C.c_int32),
        ("ablate", C.c_int32),
        ("epi_st256", C.c_int32),
        ("epi_tma_store", C.c_int32),
        ("rs_signal_batch", C.c_int32),
        ("ag_vec32", C.c_int32),
        ("ag_warps", C.c_int32),
        ("epoch_dev", C.c_void_p),
    ]


_lib = None


def available() -> bool:
    return _LIB_PATH.exists()


def check_desc_layout(L) -> None:
    """The ctypes restatement of ``tcl_gemm_desc`` must have the size and the field offsets of the C
    struct the library was built with; a stale library or an edited binding fails here, not in a kernel."""
    if L.tcl_gemm_desc_size() != C.sizeof(GemmDesc):
        raise RuntimeError(f"tcl_gemm_desc is {L.tcl_gemm_desc_size()} bytes in the library and {C.sizeof(GemmDesc)} in the binding: rebuild")
    for name, _ in GemmDesc._fields_:
        off = L.tcl_gemm_desc_offset(name.encode())
        if off >= 0 and off != getattr(GemmDesc, name).offset:
            raise RuntimeError(f"tcl_gemm_desc.{name}: offset {off} in the library, {getattr(GemmDesc, name).offset} in the binding")


def lib() -> C.CDLL:
    """The loaded library; raises with a build hint when it is missing."""
    global _lib
    if _lib is not None:
        return _lib
    if not _LIB_PATH.exists():
        raise RuntimeError(
            f"{_LIB_PATH} is missing: build it with `python -m tileccl_b200._build` "
            "(nvcc, sm_100a). There is no fallback path for the CUDA kernels."
        )
    L = C.CDLL(str(_LIB_PATH))
    vp, i32, i64, u64 = C.c_void_p, C.c_int, C.c_int64, C.c_uint64

    def sig(name, res, args):
        f = getattr(L, name)
        f.restype = res
        f.argtypes = args

    sig("tcl_gemm_desc_size", i32, [])
    sig("tcl_gemm_desc_offset", i32, [C.c_char_p])
    check_desc_layout(L)
    sig("tcl_gemm_plan_create", vp, [C.POINTER(GemmDesc), C.c_char_p, i32])
    sig("tcl_gemm_plan_run", i32, [vp, i32, vp])
    sig("tcl_gemm_plan_set_operands", i32, [vp, vp, vp])
    sig("tcl_gemm_plan_destroy", None, [vp])
    sig("tcl_gemm_plan_grid", i32, [vp])
    sig("tcl_gemm_plan_launches", i32, [vp])
    sig("tcl_gemm_smem_bytes", i32, [i32])
    sig("tcl_sched_tile", None, [i32] * 8 + [C.POINTER(i32), C.POINTER(i32)])
    sig("tcl_barrier_all", i32, [C.POINTER(vp), i32, i32, i32, vp, u64, vp])
    sig("tcl_silu_mul", i32, [vp, vp, i64, i64, vp])
    sig("tcl_fill_normal_bf16", i32, [vp, i64, u64, C.c_float, C.c_float, vp])
    sig("tcl_max_rel_err", i32, [vp, vp, i64, vp, vp, vp])
    sig("tcl_status_string", C.c_char_p, [i32])
    sig("tcl_debug_bounds_enabled", i32, [])
    sig("tcl_make_smem_desc_k_sw128", u64, [C.c_uint32])
    sig("tcl_advance_desc_k", u64, [u64, C.c_uint32])
    sig("tcl_make_idesc_bf16_f32", C.c_uint32, [C.c_uint32, C.c_uint32])
    # symmetric heap
    sig("tcl_heap_alloc", i32, [C.c_size_t, C.POINTER(vp)])
    sig("tcl_heap_free", i32, [vp])
    sig("tcl_ipc_handle_size", i32, [])
    sig("tcl_ipc_get_handle", i32, [vp, vp])
    sig("tcl_ipc_open", i32, [vp, C.POINTER(vp)])
    sig("tcl_ipc_close", i32, [vp])
    sig("tcl_enable_peer", i32, [i32])
    sig("tcl_can_access_peer", i32, [i32, i32])
    sig("tcl_memcpy_peer_async", i32, [vp, i32, vp, i32, C.c_size_t, vp])
    sig("tcl_memcpy_async", i32, [vp, vp, C.c_size_t, vp])
    sig("tcl_vmm_granularity", i32, [i32, C.POINTER(C.c_size_t), i32, i32])
    sig("tcl_multicast_supported", i32, [i32])
    sig("tcl_vmm_create", i32, [i32, C.c_size_t, C.c_size_t, C.POINTER(u64), C.POINTER(i32), C.POINTER(vp)])
    sig("tcl_vmm_import", i32, [i32, i32, C.c_size_t, C.c_size_t, C.POINTER(u64), C.POINTER(vp)])
    sig("tcl_vmm_unmap", i32, [vp, C.c_size_t, u64])
    sig("tcl_mc_create", i32, [i32, C.c_size_t, C.POINTER(u64), C.POINTER(i32)])
    sig("tcl_mc_import", i32, [i32, C.POINTER(u64)])
    sig("tcl_mc_add_device", i32, [u64, i32])
    sig("tcl_mc_bind_and_map", i32, [u64, u64, C.c_size_t, C.c_size_t, i32, C.POINTER(vp)])
    sig("tcl_mc_unbind", i32, [u64, i32, C.c_size_t])
    sig("tcl_nvls_bcast", i32, [vp, vp, C.c_size_t, i32, vp])
    sig("tcl_nvls_ld_reduce", i32, [vp, vp, C.c_size_t, i32, vp])
    sig("tcl_nvls_red", i32, [vp, vp, C.c_size_t, i32, vp])
    sig("tcl_p2p_copy", i32, [vp, vp, C.c_size_t, i32, vp])
    sig("tcl_barrier_all_mc", i32, [vp, vp, i32, i32, i32, vp, u64, vp])
    sig("tcl_p2p_scatter", i32, [C.POINTER(vp), vp, C.c_size_t, i32, i32, i32, vp])
    sig("tcl_signal_pingpong", i32, [vp, vp, i32, i32, i32, i32, vp, vp, u64, vp])
    _lib = L
    return L


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what} failed with CUDA error {rc}")


def status_string(code: int) -> str:
    return lib().tcl_status_string(code).decode()
