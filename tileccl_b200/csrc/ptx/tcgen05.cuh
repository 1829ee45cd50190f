// tcgen05 (5th-generation tensor core) and tensor-memory (TMEM) wrappers for
// sm_100a, plus the shared-memory / instruction descriptor encoders.
//
// The encoders are constexpr host+device functions so that the CPU tests can
// check the bit layouts without a GPU.
//
// The reference has no sm_100 path: its GEMMs are CUTLASS sm90 wgmma kernels
// (comm_comp/gemm_sm90.cuh:48-80).  These wrappers are what replaces them.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace tcl {
namespace ptx {

// ---------------------------------------------------------------------------
// Descriptors
// ---------------------------------------------------------------------------

// 64-bit shared-memory matrix descriptor of a K-major operand tile whose rows
// are exactly one 128-byte swizzle atom wide (64 bf16), rows packed at 128 B,
// 8-row groups packed at 1024 B (what a TMA load with SWIZZLE_128B and an
// inner box of 64 bf16 leaves in shared memory).  The tile base must be
// 1024-byte aligned.
//   [ 0,14) start address >> 4        [16,30) leading byte offset >> 4 (1: unused with swizzle)
//   [32,46) stride byte offset >> 4   [46,48) version = 1 (Blackwell)
//   [49,52) base offset = 0           [61,64) layout type: 2 = SWIZZLE_128B
__host__ __device__ constexpr uint64_t make_smem_desc_k_sw128(uint32_t smem_addr) {
  return (static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4)) |
         (static_cast<uint64_t>(1) << 16) |
         (static_cast<uint64_t>(1024 >> 4) << 32) |
         (static_cast<uint64_t>(1) << 46) |
         (static_cast<uint64_t>(2) << 61);
}

// Advancing a K-major SWIZZLE_128B descriptor by k elements of 2 bytes inside
// the swizzle atom adds (k * 2) >> 4 to the start-address field.
__host__ __device__ constexpr uint64_t advance_desc_k(uint64_t desc, uint32_t bytes) {
  return desc + static_cast<uint64_t>(bytes >> 4);
}

// 32-bit instruction descriptor for tcgen05.mma.kind::f16 with bf16 A/B (both
// K-major) and fp32 accumulation.
//   [4,6) D format: 1 = f32   [7,10) A format: 1 = bf16   [10,13) B format: 1 = bf16
//   [15] A major (0 = K)      [16] B major (0 = K)
//   [17,23) N >> 3            [24,29) M >> 4
__host__ __device__ constexpr uint32_t make_idesc_bf16_f32(uint32_t umma_m, uint32_t umma_n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((umma_n >> 3) << 17) | ((umma_m >> 4) << 24);
}

#ifdef __CUDACC__
// ---------------------------------------------------------------------------
// TMEM allocation (one full warp executes these)
// ---------------------------------------------------------------------------
template <int kCtaGroup>
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
  if constexpr (kCtaGroup == 1)
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem),
                 "r"(ncols)
                 : "memory");
  else
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem),
                 "r"(ncols)
                 : "memory");
}
template <int kCtaGroup>
__device__ __forceinline__ void tmem_relinquish() {
  if constexpr (kCtaGroup == 1)
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  else
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
template <int kCtaGroup>
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  if constexpr (kCtaGroup == 1)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
                 : "memory");
  else
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
                 : "memory");
}

__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ---------------------------------------------------------------------------
// MMA issue + commit (one thread executes these)
// ---------------------------------------------------------------------------
// D[tmem] (+)= A[smem desc] * B[smem desc]; accumulate = 0 overwrites D.
template <int kCtaGroup>
__device__ __forceinline__ void mma_f16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                           uint32_t idesc, uint32_t accumulate) {
  if constexpr (kCtaGroup == 1)
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  else
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Arrive once on `bar` (this CTA) when every tcgen05.mma issued so far by this
// thread has completed.  Implies tcgen05.fence::before_thread_sync.
__device__ __forceinline__ void tc_commit_1cta(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}
// Pair form: arrives on the barrier at the same offset in every CTA of `cta_mask`.
__device__ __forceinline__ void tc_commit_2cta(uint32_t bar, uint16_t cta_mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::
          "r"(bar),
      "h"(cta_mask)
      : "memory");
}

// ---------------------------------------------------------------------------
// TMEM -> registers.  Shape 32x32b: lane t of the warp reads TMEM lane
// (lane field of taddr + t); register j is column (column field + j).  A warp
// may only touch the 32 lanes of its own quarter: (warp index % 4) * 32.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Two fp32 -> packed bf16x2 (round to nearest even); `lo` lands in the low half.
__device__ __forceinline__ uint32_t pack_bf16x2(uint32_t lo_f32_bits, uint32_t hi_f32_bits) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;"
      : "=r"(r)
      : "f"(__uint_as_float(hi_f32_bits)), "f"(__uint_as_float(lo_f32_bits)));
  return r;
}
#endif  // __CUDACC__

}  // namespace ptx
}  // namespace tcl
