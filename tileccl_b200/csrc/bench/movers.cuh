// Data movers shared by the transport benchmarks: pattern fill / verify, the
// register (ld/st) mover, and the bulk-copy (cp.async.bulk through shared
// memory) movers with a multi-stage pipeline driven by one thread per CTA.
//
// None of the bulk copies carries a multicast qualifier; a bulk copy whose
// source or destination is peer memory is the "measured alternative"
// transport, the fused GEMM kernels never use it.  All waits are bounded: a
// mover that gives up sets *err and returns after draining its own copies.
//
// Reference parity: tests/pk_bw_sweep.cu:167-310 (fill/verify, reg_p2p_kernel,
// tma_pipe_kernel<STAGES>, tma_single_kernel), tests/p2p_ce_vs_tma.cu:185-360
// (tma_p2p / store-only / load-only / sm_p2p kernels).
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

#include "../ptx/ldst_sys.cuh"
#include "../ptx/mbarrier.cuh"
#include "../ptx/tma.cuh"

namespace tcl {
namespace bench {

__host__ __device__ inline uint32_t hash_u32(uint32_t x) {
  x ^= x >> 16; x *= 0x7feb352dU; x ^= x >> 15; x *= 0x846ca68bU; x ^= x >> 16;
  return x;
}

__global__ void fill_pattern_kernel(uint32_t* p, size_t nwords, uint32_t seed) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nwords; i += (size_t)gridDim.x * blockDim.x)
    p[i] = hash_u32(static_cast<uint32_t>(i) ^ seed);
}

__global__ void verify_pattern_kernel(const uint32_t* p, size_t nwords, uint32_t seed, unsigned long long* mismatches) {
  unsigned long long bad = 0;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nwords; i += (size_t)gridDim.x * blockDim.x)
    bad += (p[i] != hash_u32(static_cast<uint32_t>(i) ^ seed));
  if (bad) atomicAdd(mismatches, bad);
}

__global__ void fill_const_kernel(uint32_t* p, size_t nwords, uint32_t v) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nwords; i += (size_t)gridDim.x * blockDim.x) p[i] = v;
}

// Register mover.  The payload is `n_msgs` messages of `msg_vec` 16-byte
// vectors.  A message of at most 32 KiB is moved by one warp, a larger one by
// the whole CTA; messages are dealt round-robin to warps / CTAs.
__global__ void reg_copy_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, size_t n_msgs, size_t msg_vec) {
  const int lane = threadIdx.x & 31;
  if (msg_vec <= 2048) {
    const size_t warps_per_cta = blockDim.x >> 5;
    const size_t gw = blockIdx.x * warps_per_cta + (threadIdx.x >> 5);
    const size_t n_gw = gridDim.x * warps_per_cta;
    for (size_t m = gw; m < n_msgs; m += n_gw) {
      const uint4* s = src + m * msg_vec;
      uint4* d = dst + m * msg_vec;
      size_t i = lane;
      for (; i + 96 < msg_vec; i += 128) {
        uint4 a = ptx::ld_v4_stream(s + i), b = ptx::ld_v4_stream(s + i + 32);
        uint4 c = ptx::ld_v4_stream(s + i + 64), e = ptx::ld_v4_stream(s + i + 96);
        ptx::st_v4(d + i, a); ptx::st_v4(d + i + 32, b); ptx::st_v4(d + i + 64, c); ptx::st_v4(d + i + 96, e);
      }
      for (; i < msg_vec; i += 32) ptx::st_v4(d + i, ptx::ld_v4_stream(s + i));
    }
  } else {
    for (size_t m = blockIdx.x; m < n_msgs; m += gridDim.x) {
      const uint4* s = src + m * msg_vec;
      uint4* d = dst + m * msg_vec;
      size_t i = threadIdx.x;
      const size_t st = blockDim.x;
      for (; i + 3 * st < msg_vec; i += 4 * st) {
        uint4 a = ptx::ld_v4_stream(s + i), b = ptx::ld_v4_stream(s + i + st);
        uint4 c = ptx::ld_v4_stream(s + i + 2 * st), e = ptx::ld_v4_stream(s + i + 3 * st);
        ptx::st_v4(d + i, a); ptx::st_v4(d + i + st, b); ptx::st_v4(d + i + 2 * st, c); ptx::st_v4(d + i + 3 * st, e);
      }
      for (; i < msg_vec; i += st) ptx::st_v4(d + i, ptx::ld_v4_stream(s + i));
    }
  }
}

// Register mover with 256-bit loads and stores (ld/st.global.v8.b32, sm_100 and later): the same dealing of
// messages as reg_copy_kernel, 32 bytes per thread per instruction.  `msg_vec8` counts 32-byte vectors;
// the buffers must be 32-byte aligned.
__global__ void reg256_copy_kernel(const ptx::Vec8* __restrict__ src, ptx::Vec8* __restrict__ dst, size_t n_msgs, size_t msg_vec8) {
  const int lane = threadIdx.x & 31;
  if (msg_vec8 <= 1024) {
    const size_t warps_per_cta = blockDim.x >> 5;
    const size_t gw = blockIdx.x * warps_per_cta + (threadIdx.x >> 5);
    const size_t n_gw = gridDim.x * warps_per_cta;
    for (size_t m = gw; m < n_msgs; m += n_gw) {
      const ptx::Vec8* s = src + m * msg_vec8;
      ptx::Vec8* d = dst + m * msg_vec8;
      size_t i = lane;
      for (; i + 32 < msg_vec8; i += 64) {
        const ptx::Vec8 a = ptx::ld_v8_stream(s + i), b = ptx::ld_v8_stream(s + i + 32);
        ptx::st_v8(d + i, a); ptx::st_v8(d + i + 32, b);
      }
      for (; i < msg_vec8; i += 32) ptx::st_v8(d + i, ptx::ld_v8_stream(s + i));
    }
  } else {
    for (size_t m = blockIdx.x; m < n_msgs; m += gridDim.x) {
      const ptx::Vec8* s = src + m * msg_vec8;
      ptx::Vec8* d = dst + m * msg_vec8;
      size_t i = threadIdx.x;
      const size_t st = blockDim.x;
      for (; i + st < msg_vec8; i += 2 * st) {
        const ptx::Vec8 a = ptx::ld_v8_stream(s + i), b = ptx::ld_v8_stream(s + i + st);
        ptx::st_v8(d + i, a); ptx::st_v8(d + i + st, b);
      }
      for (; i < msg_vec8; i += st) ptx::st_v8(d + i, ptx::ld_v8_stream(s + i));
    }
  }
}

// What a bulk mover does with each tile.
enum BulkKind : int { kBulkCopy = 0, kBulkLoadOnly = 1, kBulkStoreOnly = 2 };

// Bulk mover: thread 0 of each CTA runs a kStages-deep ring of shared-memory
// slots; tile i (of tile_bytes, the last one shorter) goes global -> slot ->
// global.  Tiles are dealt round-robin to CTAs.  kStages - 2 loads are in
// flight while a store drains.  Dynamic shared memory: kStages * slot_stride
// + 8 * kStages bytes, slot_stride a multiple of 128.
template <int kStages>
__global__ void bulk_pipe_kernel(const char* __restrict__ src, char* __restrict__ dst, size_t total_bytes,
                                 uint32_t tile_bytes, uint32_t slot_stride, int kind, int* err,
                                 unsigned long long timeout_ns) {
  extern __shared__ __align__(128) uint8_t smem[];
  if (threadIdx.x != 0) return;
  const uint32_t base = ptx::smem_u32(smem);
  const uint32_t bars = base + kStages * slot_stride;
  for (int s = 0; s < kStages; ++s) ptx::mbar_init(bars + 8 * s, 1);
  ptx::fence_mbar_init();
  ptx::fence_proxy_async();
  const unsigned long long deadline = ptx::globaltimer_ns() + timeout_ns;
  int local_abort = 0;
  const size_t n_tiles = (total_bytes + tile_bytes - 1) / tile_bytes;
  const size_t my_n = n_tiles > blockIdx.x ? (n_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  auto tile_off = [&](size_t i) { return (blockIdx.x + i * gridDim.x) * static_cast<size_t>(tile_bytes); };
  auto tile_len = [&](size_t i) {
    const size_t off = tile_off(i);
    return static_cast<uint32_t>(total_bytes - off < tile_bytes ? total_bytes - off : tile_bytes);
  };
  constexpr int kAhead = kStages - 2;
  auto issue_load = [&](size_t i) {
    const int s = static_cast<int>(i % kStages);
    if (kind == kBulkStoreOnly) return;
    ptx::mbar_arrive_expect_tx(bars + 8 * s, tile_len(i));
    ptx::bulk_load(base + s * slot_stride, src + tile_off(i), tile_len(i), bars + 8 * s);
  };
  for (size_t i = 0; i < my_n && i < static_cast<size_t>(kAhead); ++i) issue_load(i);
  size_t loads_waited = 0;
  for (size_t i = 0; i < my_n; ++i) {
    const size_t j = i + kAhead;
    if (j < my_n) {
      // Slot j % kStages was last read by the store of tile i - 2.
      ptx::bulk_wait_read<1>();
      issue_load(j);
    }
    const int s = static_cast<int>(i % kStages);
    if (kind != kBulkStoreOnly) {
      if (!ptx::mbar_wait(bars + 8 * s, static_cast<uint32_t>((i / kStages) & 1), &local_abort, deadline)) {
        atomicExch(err, 1);
        break;
      }
      loads_waited = i + 1;
    }
    if (kind != kBulkLoadOnly) {
      ptx::bulk_store(dst + tile_off(i), base + s * slot_stride, tile_len(i));
      ptx::bulk_commit();
    }
  }
  (void)loads_waited;
  ptx::bulk_wait<0>();
  if (*reinterpret_cast<volatile int*>(err)) {
    // Gave up on a load: let the copies already issued land before smem is released.
    for (int k = 0; k < 50; ++k) __nanosleep(4000);
  }
}

// Grid-stride 16-byte copy (one flat stream, no message structure).
__global__ void flat_copy_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, size_t nvec) {
  size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
  const size_t st = (size_t)gridDim.x * blockDim.x;
  for (; i + 3 * st < nvec; i += 4 * st) {
    uint4 a = ptx::ld_v4_stream(src + i), b = ptx::ld_v4_stream(src + i + st);
    uint4 c = ptx::ld_v4_stream(src + i + 2 * st), d = ptx::ld_v4_stream(src + i + 3 * st);
    ptx::st_v4(dst + i, a); ptx::st_v4(dst + i + st, b); ptx::st_v4(dst + i + 2 * st, c); ptx::st_v4(dst + i + 3 * st, d);
  }
  for (; i < nvec; i += st) ptx::st_v4(dst + i, ptx::ld_v4_stream(src + i));
}

// Load-only mover on the register path: a CTA brings tile after tile of the source into shared memory
// with 16-byte ld.global (L1::no_allocate) + st.shared, four loads in flight per thread.  It is the
// counterpart of kBulkLoadOnly without the bulk-copy engine: what a gather warp of a fused all-gather +
// GEMM pays before the tile can reach the tensor core.  Dynamic shared memory: tile_vec * 16 bytes.
__global__ void ldst_load_only_kernel(const uint4* __restrict__ src, size_t total_vec, uint32_t tile_vec, unsigned* sink) {
  extern __shared__ __align__(16) uint4 ldst_tile[];
  const size_t n_tiles = (total_vec + tile_vec - 1) / tile_vec;
  unsigned acc = 0;
  for (size_t t = blockIdx.x; t < n_tiles; t += gridDim.x) {
    const uint4* p = src + t * tile_vec;
    const uint32_t len = static_cast<uint32_t>(total_vec - t * tile_vec < tile_vec ? total_vec - t * tile_vec : tile_vec);
    uint32_t i = threadIdx.x;
    for (; i + 3 * blockDim.x < len; i += 4 * blockDim.x) {
      const uint4 a = ptx::ld_v4_stream(p + i), b = ptx::ld_v4_stream(p + i + blockDim.x);
      const uint4 c = ptx::ld_v4_stream(p + i + 2 * blockDim.x), d = ptx::ld_v4_stream(p + i + 3 * blockDim.x);
      ldst_tile[i] = a; ldst_tile[i + blockDim.x] = b; ldst_tile[i + 2 * blockDim.x] = c; ldst_tile[i + 3 * blockDim.x] = d;
    }
    for (; i < len; i += blockDim.x) ldst_tile[i] = ptx::ld_v4_stream(p + i);
    __syncthreads();
    acc += ldst_tile[(threadIdx.x * 7u) % len].x;  // the tile is consumed from shared memory
    __syncthreads();
  }
  if (acc == 0xdeadbeefu) *sink = acc;
}

inline cudaError_t launch_ldst_load_only(int blocks, cudaStream_t st, const void* src, size_t total, uint32_t tile_bytes, unsigned* sink) {
  const uint32_t tile_vec = tile_bytes / 16;
  if (tile_vec == 0 || total % 16 != 0) return cudaErrorInvalidValue;
  cudaError_t e = cudaFuncSetAttribute(ldst_load_only_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(tile_vec * 16));
  if (e != cudaSuccess) return e;
  ldst_load_only_kernel<<<blocks, 256, tile_vec * 16, st>>>(static_cast<const uint4*>(src), total / 16, tile_vec, sink);
  return cudaGetLastError();
}

inline size_t bulk_smem_bytes(int stages, uint32_t slot_stride) { return static_cast<size_t>(stages) * slot_stride + 8 * stages; }

// Launch helper: picks the instantiation for `stages` in {3,4,6,8}.
inline cudaError_t launch_bulk_pipe(int stages, int blocks, cudaStream_t st, const void* src, void* dst, size_t total,
                                    uint32_t tile_bytes, int kind, int* err, unsigned long long timeout_ns) {
  const uint32_t slot = (tile_bytes + 127u) & ~127u;
  const size_t smem = bulk_smem_bytes(stages, slot);
  auto go = [&](auto kern) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return e;
    kern<<<blocks, 32, smem, st>>>(static_cast<const char*>(src), static_cast<char*>(dst), total, tile_bytes, slot, kind, err, timeout_ns);
    return cudaGetLastError();
  };
  switch (stages) {
    case 3: return go(bulk_pipe_kernel<3>);
    case 4: return go(bulk_pipe_kernel<4>);
    case 6: return go(bulk_pipe_kernel<6>);
    default: return go(bulk_pipe_kernel<8>);
  }
}

}  // namespace bench
}  // namespace tcl
