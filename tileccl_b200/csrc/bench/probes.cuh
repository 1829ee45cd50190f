// Persistent self-reporting probe kernels for the interference matrices.
//
// A probe keeps one resource busy (tensor pipe through tcgen05, tensor pipe through legacy
// mma.sync, FP32 pipe, HBM, L2, shared memory) and counts its iterations in a per-CTA counter in
// device memory that the host copies out while the kernel runs.  It stops when the host raises a stop
// flag, or by itself at a hard deadline, so it can never outlive its measurement.
//
// Reference parity: tests/interference_matrix.cu:282-377 (probe_ffma/mma/hbm/l2/smem kernels), whose
// mma probe is wmma only; the tcgen05 probe is new here.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>
#include <mma.h>
#include <cuda_bf16.h>

#include "../ptx/ldst_sys.cuh"
#include "../ptx/mbarrier.cuh"
#include "../ptx/tcgen05.cuh"

namespace tcl {
namespace bench {

enum ProbeKind : int { kProbeTc5 = 0, kProbeMma = 1, kProbeFfma = 2, kProbeHbm = 3, kProbeL2 = 4, kProbeSmem = 5, kProbeCount = 6 };
inline const char* probe_name(int k) {
  static const char* n[] = {"tcgen05", "mma", "ffma", "hbm", "l2", "smem"};
  return k >= 0 && k < kProbeCount ? n[k] : "?";
}
inline const char* probe_unit(int k) {
  static const char* n[] = {"Gmma/s", "Gmma/s", "Gffma/s", "GB/s", "GB/s", "Gld/s"};
  return k >= 0 && k < kProbeCount ? n[k] : "?";
}

struct ProbeArgs {
  volatile int* stop;             // device memory: != 0 ends the probe
  unsigned long long* counters;   // device memory, one per CTA: iterations done (the host snapshots it)
  unsigned long long deadline_ns; // %globaltimer value after which the probe ends on its own
  uint4* buf;                     // hbm / l2 working set
  size_t buf_vec;                 // its size in 16-byte vectors (per CTA slice for hbm, whole for l2)
  float* sink;
};

// The stop flag is in device memory (the host raises it with an async copy): polling it costs an
// L2 hit, not a PCIe read per warp.
__device__ __forceinline__ bool probe_should_stop(const ProbeArgs& a) {
  return *a.stop != 0 || ptx::globaltimer_ns() > a.deadline_ns;
}

// Work units per counted iteration, for converting counts to rates on the host.
constexpr int kFfmaPerIter = 512;        // per thread
constexpr int kMmaPerIter = 64;          // per warp (16x16x16)
constexpr int kTc5MmaPerIter = 64;       // per CTA (128x64x16)
constexpr int kSmemLoadsPerIter = 256;   // per thread

__global__ void probe_ffma_kernel(ProbeArgs a) {
  float x = threadIdx.x * 1e-3f, y = 1.0000001f, z = 0.5f;
  unsigned long long n = 0;
  while (true) {
#pragma unroll 64
    for (int i = 0; i < kFfmaPerIter; ++i) x = fmaf(x, y, z);
    ++n;
    if (threadIdx.x == 0) {
      a.counters[blockIdx.x] = n;
    }
    if ((n & 63) == 0 && probe_should_stop(a)) break;
  }
  if (x == 123.456f) a.sink[0] = x;
}

__global__ void probe_mma_kernel(ProbeArgs a) {
  using namespace nvcuda;
  wmma::fragment<wmma::matrix_a, 16, 16, 16, __nv_bfloat16, wmma::row_major> fa;
  wmma::fragment<wmma::matrix_b, 16, 16, 16, __nv_bfloat16, wmma::col_major> fb;
  wmma::fragment<wmma::accumulator, 16, 16, 16, float> fc;
  wmma::fill_fragment(fa, __float2bfloat16(0.001f));
  wmma::fill_fragment(fb, __float2bfloat16(0.002f));
  wmma::fill_fragment(fc, 0.f);
  unsigned long long n = 0;
  while (true) {
#pragma unroll 16
    for (int i = 0; i < kMmaPerIter; ++i) wmma::mma_sync(fc, fa, fb, fc);
    ++n;
    if (threadIdx.x == 0) a.counters[blockIdx.x] = n;
    if ((n & 63) == 0 && probe_should_stop(a)) break;
  }
  if (fc.x[0] == 123.456f) a.sink[0] = fc.x[0];
}

// One warp per CTA drives the 5th-generation tensor core: 128x64x16 bf16 MMAs on a zero-filled
// operand tile in shared memory, accumulator in TMEM, completion through tcgen05.commit.
__global__ void probe_tc5_kernel(ProbeArgs a, int* err) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ __align__(8) unsigned long long bar;
  __shared__ uint32_t tmem_slot;
  const uint32_t raw = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  if (threadIdx.x >= 32) return;
  uint4* z = reinterpret_cast<uint4*>(smem_raw + (base - raw));
  for (int i = threadIdx.x; i < (16384 + 8192) / 16; i += 32) z[i] = make_uint4(0, 0, 0, 0);
  if (threadIdx.x == 0) { ptx::mbar_init(ptx::smem_u32(&bar), 1); ptx::fence_mbar_init(); }
  ptx::fence_proxy_async();
  __syncwarp();
  ptx::tmem_alloc<1>(ptx::smem_u32(&tmem_slot), 64);
  ptx::tmem_relinquish<1>();
  ptx::tc_fence_before_sync();
  __syncwarp();
  ptx::tc_fence_after_sync();
  const uint32_t tmem = tmem_slot;
  if (threadIdx.x == 0) {
    const uint64_t da = ptx::make_smem_desc_k_sw128(base);
    const uint64_t db = ptx::make_smem_desc_k_sw128(base + 16384);
    constexpr uint32_t idesc = ptx::make_idesc_bf16_f32(128, 64);
    unsigned long long n = 0;
    int abort_flag = 0;
    while (true) {
      for (int i = 0; i < kTc5MmaPerIter; ++i)
        ptx::mma_f16_ss<1>(tmem, ptx::advance_desc_k(da, (i & 3) * 32), ptx::advance_desc_k(db, (i & 3) * 32), idesc, i > 0);
      ptx::tc_commit_1cta(ptx::smem_u32(&bar));
      if (!ptx::mbar_wait(ptx::smem_u32(&bar), static_cast<uint32_t>(n & 1), &abort_flag, a.deadline_ns + 1000000000ull)) {
        atomicExch(err, 1);
        break;
      }
      ++n;
      a.counters[blockIdx.x] = n;
      if ((n & 63) == 0 && probe_should_stop(a)) break;
    }
  }
  __syncwarp();
  ptx::tc_fence_after_sync();
  ptx::tmem_dealloc<1>(tmem, 64);
}

// Each CTA streams (read + write) through its private slice of the buffer.
__global__ void probe_hbm_kernel(ProbeArgs a) {
  uint4* p = a.buf + static_cast<size_t>(blockIdx.x) * a.buf_vec;
  unsigned long long n = 0;
  uint4 acc = make_uint4(0, 0, 0, 0);
  while (true) {
    for (size_t i = threadIdx.x; i + 3 * blockDim.x < a.buf_vec; i += 4 * blockDim.x) {
      uint4 v0 = ptx::ld_v4_cg(p + i), v1 = ptx::ld_v4_cg(p + i + blockDim.x);
      uint4 v2 = ptx::ld_v4_cg(p + i + 2 * blockDim.x), v3 = ptx::ld_v4_cg(p + i + 3 * blockDim.x);
      acc.x += v0.x + v1.x + v2.x + v3.x;
      v0.y ^= 1u;
      ptx::st_v4(p + i, v0);
    }
    ++n;
    if (threadIdx.x == 0) a.counters[blockIdx.x] = n;
    if (probe_should_stop(a)) break;
  }
  if (acc.x == 0xdeadbeefu) a.sink[0] = 1.f;
}

// All CTAs scan the same buffer, sized to stay inside L2.
__global__ void probe_l2_kernel(ProbeArgs a) {
  unsigned long long n = 0;
  uint4 acc = make_uint4(0, 0, 0, 0);
  while (true) {
    for (size_t i = threadIdx.x + static_cast<size_t>(blockIdx.x) * 64; i < a.buf_vec; i += 4 * blockDim.x) {
      const uint4 v = ptx::ld_v4_cg(a.buf + i);
      acc.x += v.x;
    }
    ++n;
    if (threadIdx.x == 0) a.counters[blockIdx.x] = n;
    if (probe_should_stop(a)) break;
  }
  if (acc.x == 0xdeadbeefu) a.sink[0] = 1.f;
}

// Dependent shared-memory loads over 32 KiB.
__global__ void probe_smem_kernel(ProbeArgs a) {
  __shared__ uint32_t s[8192];
  for (int i = threadIdx.x; i < 8192; i += blockDim.x) s[i] = (i * 33 + 17) & 8191;
  __syncthreads();
  uint32_t idx = threadIdx.x;
  unsigned long long n = 0;
  while (true) {
#pragma unroll 16
    for (int i = 0; i < kSmemLoadsPerIter; ++i) idx = s[idx];
    ++n;
    if (threadIdx.x == 0) a.counters[blockIdx.x] = n;
    if ((n & 63) == 0 && probe_should_stop(a)) break;
  }
  if (idx == 0xffffffffu) a.sink[0] = 1.f;
}

// Work per counted iteration of one CTA with `threads` threads (unit of probe_unit / 1e9).
inline double probe_work_per_iter(int kind, int threads, size_t buf_vec, int blocks) {
  switch (kind) {
    case kProbeTc5: return kTc5MmaPerIter;
    case kProbeMma: return static_cast<double>(kMmaPerIter) * (threads / 32);
    case kProbeFfma: return static_cast<double>(kFfmaPerIter) * threads;
    case kProbeHbm: return static_cast<double>(buf_vec) * 16 * 1.25;            // 4 reads + 1 write per 4 vectors
    case kProbeL2: return static_cast<double>(buf_vec) * 16 / 4.0 / (blocks > 0 ? 1 : 1);
    case kProbeSmem: return static_cast<double>(kSmemLoadsPerIter) * threads;
    default: return 1;
  }
}

}  // namespace bench
}  // namespace tcl
