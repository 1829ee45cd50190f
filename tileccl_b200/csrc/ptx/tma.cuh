// TMA (cp.async.bulk / cp.async.bulk.tensor) wrappers for sm_100a and the
// host-side tensor-map encoder.
//
// Rules this file keeps:
//   * every tensor copy starts at an x coordinate that is a multiple of 8
//     bf16 elements (16 bytes);
//   * no load carries a cluster-multicast qualifier: in a CTA pair each CTA
//     loads its own half of the operands into its own shared memory.
//
// Reference parity: its bulk-copy helpers (tests/pk_bw_sweep.cu:82-152,
// l2_peer_cache/peer_l2_probe.cu:320-422) and the TMA descriptors CUTLASS
// builds for it (comm_comp/gemm_sm90.cuh:99-130).
#pragma once
#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>

namespace tcl {
namespace ptx {

#ifdef __CUDACC__
// 2-D tiled load global -> this CTA's shared memory, completion on this CTA's mbarrier.
__device__ __forceinline__ void tma_load_2d(uint32_t dst_smem, const CUtensorMap* map, uint32_t bar,
                                            int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::
          "r"(dst_smem),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y)
      : "memory");
}

// Pair form: data lands in this CTA's shared memory, the transaction bytes are
// counted on `cluster_bar`, which may be the leader CTA's barrier (a
// shared::cluster address from mapa).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst_smem, const CUtensorMap* map,
                                                 uint32_t cluster_bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::
          "r"(dst_smem),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(cluster_bar), "r"(x), "r"(y)
      : "memory");
}

// 2-D tiled store this CTA's shared memory -> global, joined to the calling thread's bulk group.
// The box that leaves shared memory is the tensor map's box; rows and columns beyond the tensor's
// extent are clipped by the hardware.  x must be a multiple of 8 bf16 elements; x and y not negative.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src_smem, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(src_smem), "r"(x), "r"(y)
               : "memory");
}

__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// Untiled bulk copies: both addresses 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_load(uint32_t dst_smem, const void* src, uint32_t bytes,
                                          uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          dst_smem),
      "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void bulk_store(void* dst, uint32_t src_smem, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst),
               "r"(src_smem), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// Wait until at most N groups still READ shared memory (buffers reusable).
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
// Wait until at most N groups are incomplete (writes performed).
template <int N>
__device__ __forceinline__ void bulk_wait() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
#endif  // __CUDACC__

// ---------------------------------------------------------------------------
// Host: tensor map for a row-major [rows, cols] bf16 matrix with row pitch
// `ld` elements; box = [box_rows, 64 cols] with 128-byte swizzle.
// Returns 0 on success, a CUresult (or -1 if the driver symbol is missing).
// ---------------------------------------------------------------------------
inline int encode_tmap_bf16_k64(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols,
                                uint64_t ld, uint32_t box_rows) {
  typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                               const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                               const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static EncodeFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess || !p)
      return -1;
    fn = reinterpret_cast<EncodeFn>(p);
  }
  cuuint64_t gdim[2] = {cols, rows};
  cuuint64_t gstride[1] = {ld * 2};
  cuuint32_t box[2] = {64, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), gdim, gstride,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return static_cast<int>(r);
}

}  // namespace ptx
}  // namespace tcl
