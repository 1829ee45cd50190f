// Scoped loads/stores/reductions on global memory (local or a peer's, over
// NVLink), 128-bit movers with cache qualifiers written in the source, and the
// NVLS multimem forms.
//
// Reference parity: comm_comp/rs_barrier.cuh:41-157 (system/gpu-scope flag
// barriers, vector red), signalling/signal_fanin.cu:98-112,
// tests/sync_cost.cu:60-74 (ld.acquire.sys / st.release.sys helpers).  The
// reference selects the L1 policy with a second build (-Xptxas -dlcm=cg,
// l2_peer_cache/Makefile:28-32); here the qualifier is in the instruction.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace tcl {
namespace ptx {

// ---- flags ----------------------------------------------------------------
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ int ld_relaxed_sys(const int* p) {
  int v;
  asm volatile("ld.relaxed.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_relaxed_sys(int* p, int v) {
  asm volatile("st.relaxed.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_release_sys_add(int* p, int v) {
  asm volatile("red.release.sys.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_release_gpu_add(int* p, int v) {
  asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_relaxed_sys_add(int* p, int v) {
  asm volatile("red.relaxed.sys.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int atom_add_acq_rel_sys(int* p, int v) {
  int old;
  asm volatile("atom.acq_rel.sys.global.add.s32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
  return old;
}
__device__ __forceinline__ int atom_add_acq_rel_gpu(int* p, int v) {
  int old;
  asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
  return old;
}
__device__ __forceinline__ void fence_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }
__device__ __forceinline__ void fence_gpu() { asm volatile("fence.acq_rel.gpu;" ::: "memory"); }

// Bounded acquire spin: returns true once *p >= target (signed distance, so
// epoch counters may wrap), false when the deadline passes or the CTA aborts.
// `observed` gets the last value read.
template <bool kSys>
__device__ __forceinline__ bool wait_ge(const int* p, int target, volatile int* abort_flag,
                                        unsigned long long deadline_ns, int* observed,
                                        unsigned sleep_ns = 64) {
  for (unsigned it = 0;; ++it) {
    int v = kSys ? ld_acquire_sys(p) : ld_acquire_gpu(p);
    if (v - target >= 0) {
      if (observed) *observed = v;
      return true;
    }
    if (sleep_ns) __nanosleep(sleep_ns);
    if ((it & 15u) == 15u) {
      unsigned long long now;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
      if ((abort_flag && *abort_flag != 0) || now > deadline_ns) {
        if (observed) *observed = v;
        return false;
      }
    }
  }
}

// ---- 128-bit data movers ----------------------------------------------------
// Streaming load that does not allocate in L1 (peer memory is never cached in
// the reader's L2, so L1 is the only cache that could return stale lines).
__device__ __forceinline__ uint4 ld_v4_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
// Cached-in-L2-only load (the .cg policy of the reference's second build).
__device__ __forceinline__ uint4 ld_v4_cg(const void* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
// Default policy (.ca): may allocate in L1.
__device__ __forceinline__ uint4 ld_v4_ca(const void* p) {
  uint4 v;
  asm volatile("ld.global.ca.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
// Volatile-like load that always goes to the point of coherence.
__device__ __forceinline__ uint4 ld_v4_relaxed_sys(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ void st_v4(void* p, const uint4& v) {
  asm volatile("st.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}
// 256-bit forms (sm_100 and later): one instruction moves 32 bytes; the address must be 32-byte aligned.
struct alignas(32) Vec8 {
  uint32_t w[8];
};
__device__ __forceinline__ Vec8 ld_v8_stream(const void* p) {
  Vec8 v;
  asm volatile("ld.global.L1::no_allocate.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3]), "=r"(v.w[4]), "=r"(v.w[5]), "=r"(v.w[6]), "=r"(v.w[7])
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ void st_v8(void* p, const Vec8& v) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "r"(v.w[0]), "r"(v.w[1]), "r"(v.w[2]),
               "r"(v.w[3]), "r"(v.w[4]), "r"(v.w[5]), "r"(v.w[6]), "r"(v.w[7])
               : "memory");
}
__device__ __forceinline__ void st_v4_stream(void* p, const uint4& v) {
  asm volatile("st.global.L1::no_allocate.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x),
               "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

// ---- shared memory 128-bit ------------------------------------------------------
__device__ __forceinline__ void sts_v4(uint32_t addr, const uint4& v) {
  asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}
__device__ __forceinline__ uint4 lds_v4(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(addr)
               : "memory");
  return v;
}

// ---- NVLS multimem (addresses come from a multicast mapping of the heap) ------
// Store 16 bytes to the same offset on every GPU bound to the multicast object.
__device__ __forceinline__ void multimem_st_v4(void* mc_ptr, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_ptr),
               "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)),
               "f"(__uint_as_float(v.w))
               : "memory");
}
// Load 8 bf16 from every GPU at this offset, summed inside the switch with fp32 accumulation.
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const void* mc_ptr) {
  uint4 v;
  asm volatile(
      "multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
      : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
      : "l"(mc_ptr)
      : "memory");
  return v;
}
// Add 8 bf16 into every GPU's copy at this offset.
__device__ __forceinline__ void multimem_red_bf16x8(void* mc_ptr, const uint4& v) {
  asm volatile("multimem.red.relaxed.sys.global.add.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(mc_ptr),
               "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}
// Signal every GPU's flag at this offset (+v), release at system scope.
__device__ __forceinline__ void multimem_red_release_add(int* mc_ptr, int v) {
  asm volatile("multimem.red.release.sys.global.add.u32 [%0], %1;" ::"l"(mc_ptr), "r"(v) : "memory");
}

}  // namespace ptx
}  // namespace tcl
