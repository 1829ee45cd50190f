"""Bit layouts of the tcgen05 shared-memory and instruction descriptors (host build of the encoders)."""


def test_smem_descriptor_fields(native_lib):
    d = native_lib.tcl_make_smem_desc_k_sw128(0x12400)
    assert d & 0x3FFF == 0x12400 >> 4                  # start address >> 4
    assert (d >> 16) & 0x3FFF == 1                      # leading byte offset (unused with swizzle)
    assert (d >> 32) & 0x3FFF == 1024 >> 4              # stride byte offset: 8 rows x 128 B
    assert (d >> 46) & 0x3 == 1                         # descriptor version of sm_100
    assert (d >> 49) & 0x7 == 0                         # base offset
    assert (d >> 61) & 0x7 == 2                         # SWIZZLE_128B
    # stepping 16 bf16 elements along K inside the swizzle atom moves the start address by 32 bytes
    d2 = native_lib.tcl_advance_desc_k(d, 32)
    assert d2 - d == 2 and (d2 >> 16) == (d >> 16)
    # addresses above 256 KiB wrap into the 14-bit field (shared memory is smaller than that anyway)
    assert native_lib.tcl_make_smem_desc_k_sw128(0x40000 + 0x800) & 0x3FFF == 0x800 >> 4


def test_instruction_descriptor_fields(native_lib):
    for m, n in ((128, 256), (256, 256), (128, 64)):
        i = native_lib.tcl_make_idesc_bf16_f32(m, n)
        assert (i >> 4) & 0x3 == 1                      # D format fp32
        assert (i >> 7) & 0x7 == 1 and (i >> 10) & 0x7 == 1   # A and B are bf16
        assert (i >> 15) & 0x1 == 0 and (i >> 16) & 0x1 == 0  # both K-major
        assert (i >> 17) & 0x3F == n >> 3
        assert (i >> 24) & 0x1F == m >> 4
        assert i & 0xF == 0 and (i >> 13) & 0x3 == 0    # dense, no negation


def test_binding_restates_the_c_struct(native_lib):
    """Size and field offsets of the ctypes GemmDesc equal those of tcl_gemm_desc in the built library."""
    import ctypes as C

    from tileccl_b200 import _native
    assert native_lib.tcl_gemm_desc_size() == C.sizeof(_native.GemmDesc)
    checked = 0
    for name, _ in _native.GemmDesc._fields_:
        off = native_lib.tcl_gemm_desc_offset(name.encode())
        if off >= 0:
            assert off == getattr(_native.GemmDesc, name).offset, name
            checked += 1
    assert checked >= 20 and native_lib.tcl_gemm_desc_offset(b"no_such_field") == -1
