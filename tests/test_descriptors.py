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


def _swizzle128(byte_off: int) -> int:
    """The 128-byte swizzle of TMA and of the MMA operand descriptors: address bits 4-6 are XORed with
    bits 7-9 (the 16-byte chunk index with the row index inside an 8-row, 1024-byte atom)."""
    return byte_off ^ (((byte_off >> 7) & 7) << 4)


def test_epilogue_staging_layouts():
    """Index arithmetic of the epilogue's per-warp staging buffer, restated from the kernel:
    * default layout: row `lane`, 16-byte slot k of the 256-byte row at k ^ (lane & 7);
    * TMA layout: two 32 x 128-byte tiles (one per 64-column half) in the canonical 128-byte swizzle,
      so that a tensor-map store with SWIZZLE_128B finds element (row, column) where it expects it;
    * the 32-byte store path reads each row's chunks in an order that keeps a quarter-warp on 8 banks."""
    # ---- writer (both layouts): lane = row, half h in {0,1}, chunk j in 0..7 (8 bf16 columns each)
    default, tma = {}, {}
    for lane in range(32):
        for h in range(2):
            for j in range(8):
                col_chunk = h * 8 + j                                   # 16-byte chunk index inside the 128-column pair
                default[lane * 256 + h * 128 + ((j ^ (lane & 7)) << 4)] = (lane, col_chunk)
                tma[h * 4096 + lane * 128 + ((j ^ (lane & 7)) << 4)] = (lane, col_chunk)
    assert len(default) == 512 and len(tma) == 512                      # no two elements share a slot
    # ---- TMA layout equals the canonical swizzle of a dense [32][128 B] tile per half
    for h in range(2):
        for row in range(32):
            for c in range(8):
                assert tma[h * 4096 + _swizzle128(row * 128 + c * 16)] == (row, h * 8 + c)
    # ---- 16-byte store path: lane (ch = lane & 15, r = 2 i + lane >> 4) reads slot ch ^ (r & 7) of row r
    for i in range(16):
        for lane in range(32):
            ch, r = lane & 15, i * 2 + (lane >> 4)
            assert default[r * 256 + ((ch ^ (r & 7)) << 4)] == (r, ch)
    # ---- 32-byte store path: lane (ch8 = lane & 7, r = 4 i + lane >> 3) needs chunks 2 ch8 and 2 ch8 + 1
    for i in range(8):
        for phase in range(2):                                          # first and second 16-byte read of every lane
            for quarter in range(4):                                    # 8 lanes are served together
                banks = set()
                for lane in range(quarter * 8, quarter * 8 + 8):
                    ch8, r = lane & 7, i * 4 + (lane >> 3)
                    swap = ch8 >> 2
                    k = 2 * ch8 + (swap if phase == 0 else 1 - swap)
                    off = r * 256 + ((k ^ (r & 7)) << 4)
                    assert default[off] == (r, k)
                    banks.add((off // 4) % 32)                          # first bank of the 16-byte access
                assert len(banks) == 8, (i, phase, quarter)             # 8 x 4 banks: conflict free
