// NVLS (NVLink SHARP) data movers: multimem instructions on a multicast mapping of the symmetric heap.
//   bcast      local -> every GPU        multimem.st            (the all-gather building block)
//   ld_reduce  every GPU -> local sum    multimem.ld_reduce     (the reduce-scatter building block; the
//                                                                switch adds the bf16 values in fp32)
//   red        local -> added everywhere multimem.red
//   barrier    one multimem.red.release per rank on a counter, instead of one red per peer
// and a plain peer copy (ld/st through a peer mapping) for comparison.  Simple grid-stride kernels: they
// are the movers of the NVLS bandwidth sweep, and the in-switch reduce path of the fused GEMM+RS reuses
// the same instruction wrappers (ptx/ldst_sys.cuh).
//
// The reference has no multicast path (no multimem anywhere in it).
#include <cuda_runtime.h>

#include <cstdint>

#include "../ptx/ldst_sys.cuh"
#include "../ptx/mbarrier.cuh"

namespace {
using namespace tcl::ptx;

__global__ void nvls_bcast_kernel(uint4* mc_dst, const uint4* __restrict__ src, size_t nvec) {
  const size_t st = (size_t)gridDim.x * blockDim.x;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nvec; i += st) multimem_st_v4(mc_dst + i, ld_v4_stream(src + i));
}
__global__ void nvls_ld_reduce_kernel(const uint4* mc_src, uint4* __restrict__ dst, size_t nvec) {
  const size_t st = (size_t)gridDim.x * blockDim.x;
  size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
  for (; i + 3 * st < nvec; i += 4 * st) {
    const uint4 a = multimem_ld_reduce_bf16x8(mc_src + i), b = multimem_ld_reduce_bf16x8(mc_src + i + st);
    const uint4 c = multimem_ld_reduce_bf16x8(mc_src + i + 2 * st), d = multimem_ld_reduce_bf16x8(mc_src + i + 3 * st);
    st_v4(dst + i, a); st_v4(dst + i + st, b); st_v4(dst + i + 2 * st, c); st_v4(dst + i + 3 * st, d);
  }
  for (; i < nvec; i += st) st_v4(dst + i, multimem_ld_reduce_bf16x8(mc_src + i));
}
__global__ void nvls_red_kernel(uint4* mc_dst, const uint4* __restrict__ src, size_t nvec) {
  const size_t st = (size_t)gridDim.x * blockDim.x;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nvec; i += st) multimem_red_bf16x8(mc_dst + i, ld_v4_stream(src + i));
}
__global__ void p2p_copy_kernel(uint4* dst, const uint4* __restrict__ src, size_t nvec) {
  const size_t st = (size_t)gridDim.x * blockDim.x;
  size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
  for (; i + 3 * st < nvec; i += 4 * st) {
    const uint4 a = ld_v4_stream(src + i), b = ld_v4_stream(src + i + st), c = ld_v4_stream(src + i + 2 * st), d = ld_v4_stream(src + i + 3 * st);
    st_v4(dst + i, a); st_v4(dst + i + st, b); st_v4(dst + i + 2 * st, c); st_v4(dst + i + 3 * st, d);
  }
  for (; i < nvec; i += st) st_v4(dst + i, ld_v4_stream(src + i));
}

// All-to-all store: slice p of `src` (slice_vec vectors) goes to slot `rank` of peer p's buffer; block b
// serves peer (b % peers), so every peer is written at the same time, as in the epilogue of the fused
// GEMM + reduce-scatter.  The own slice is skipped.
struct ScatterArgs {
  uint4* dst[8];
};
__global__ void p2p_scatter_kernel(ScatterArgs a, const uint4* __restrict__ src, size_t slice_vec, int world, int rank) {
  const int peers = world - 1;
  const int which = blockIdx.x % peers;
  const int peer = (rank + 1 + which) % world;
  const size_t lane_blocks = gridDim.x / peers;          // blocks that serve this peer (the host makes it >= 1)
  const size_t b = blockIdx.x / peers;
  if (b >= lane_blocks) return;
  const uint4* s = src + static_cast<size_t>(peer) * slice_vec;
  uint4* d = a.dst[peer] + static_cast<size_t>(rank) * slice_vec;
  const size_t st = lane_blocks * blockDim.x;
  size_t i = b * blockDim.x + threadIdx.x;
  for (; i + 3 * st < slice_vec; i += 4 * st) {
    const uint4 v0 = ld_v4_stream(s + i), v1 = ld_v4_stream(s + i + st), v2 = ld_v4_stream(s + i + 2 * st), v3 = ld_v4_stream(s + i + 3 * st);
    st_v4(d + i, v0); st_v4(d + i + st, v1); st_v4(d + i + 2 * st, v2); st_v4(d + i + 3 * st, v3);
  }
  for (; i < slice_vec; i += st) st_v4(d + i, ld_v4_stream(s + i));
}

// All-ranks barrier with ONE store per rank: the switch adds 1 to the counter's copy on every GPU.
// The counter is an epoch counter (never reset): a rank leaves when its own copy reached epoch*world.
// status = {code, rank, wanted, seen}; code 1 is the same "start barrier timed out" as the peer-store barrier.
__global__ void barrier_all_mc_kernel(int* mc_counter, const int* local_counter, int world, int rank, int epoch, int* status,
                                      unsigned long long timeout_ns) {
  if (threadIdx.x != 0) return;
  multimem_red_release_add(mc_counter, 1);
  const unsigned long long deadline = globaltimer_ns() + timeout_ns;
  int seen = 0;
  const int target = static_cast<int>(static_cast<unsigned>(epoch) * static_cast<unsigned>(world));  // may wrap
  if (!wait_ge<true>(local_counter, target, nullptr, deadline, &seen)) {
    if (atomicCAS(status, 0, 1) == 0) {
      status[1] = rank;
      status[2] = target;
      status[3] = seen;
    }
  }
}

// Flag ping-pong between two ranks (one thread each).  The signal goes out as
//   mode 0  st.release.sys of the round number to the peer's flag
//   mode 1  red.release.sys.add of 1 on the peer's flag
//   mode 2  multimem.red.release.add of 1 on the flag's multicast address; this lands on every copy, the
//           sender's own included, so a copy shows the sum of both sides' signals
// `base` is the value the flags hold when the call starts (counters are never reset).  The initiator
// writes the mean round-trip time; a wait that runs out sets status = {2, round, wanted, seen}.
__global__ void signal_pingpong_kernel(const int* local_flag, int* remote_flag, int mode, int initiator, int base, int rounds,
                                       float* ns_per_rtt, int* status, unsigned long long timeout_ns) {
  if (threadIdx.x != 0) return;
  const unsigned long long t0 = globaltimer_ns();
  const unsigned long long deadline = t0 + timeout_ns;
  auto send = [&](int k) {
    if (mode == 0) st_release_sys(remote_flag, base + k + 1);
    else if (mode == 1) red_release_sys_add(remote_flag, 1);
    else multimem_red_release_add(remote_flag, 1);
  };
  for (int k = 0; k < rounds; ++k) {
    const int want = mode == 2 ? base + 2 * k + (initiator ? 2 : 1) : base + k + 1;
    int seen = 0;
    if (initiator) send(k);
    if (!wait_ge<true>(local_flag, want, nullptr, deadline, &seen, 0)) {
      if (atomicCAS(status, 0, 2) == 0) {
        status[1] = k;
        status[2] = want;
        status[3] = seen;
      }
      return;
    }
    if (!initiator) send(k);
  }
  if (initiator) *ns_per_rtt = static_cast<float>(globaltimer_ns() - t0) / static_cast<float>(rounds);
}

int grid_for(size_t nvec, int blocks) {
  if (blocks > 0) return blocks;
  size_t b = (nvec + 1023) / 1024;
  return static_cast<int>(b < 1 ? 1 : (b > 148 * 4 ? 148 * 4 : b));
}
}  // namespace

extern "C" {
int tcl_nvls_bcast(void* mc_dst, const void* src, size_t bytes, int blocks, void* stream) {
  nvls_bcast_kernel<<<grid_for(bytes / 16, blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<uint4*>(mc_dst), static_cast<const uint4*>(src), bytes / 16);
  return static_cast<int>(cudaGetLastError());
}
int tcl_nvls_ld_reduce(const void* mc_src, void* dst, size_t bytes, int blocks, void* stream) {
  nvls_ld_reduce_kernel<<<grid_for(bytes / 16, blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const uint4*>(mc_src), static_cast<uint4*>(dst), bytes / 16);
  return static_cast<int>(cudaGetLastError());
}
int tcl_nvls_red(void* mc_dst, const void* src, size_t bytes, int blocks, void* stream) {
  nvls_red_kernel<<<grid_for(bytes / 16, blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<uint4*>(mc_dst), static_cast<const uint4*>(src), bytes / 16);
  return static_cast<int>(cudaGetLastError());
}
int tcl_p2p_copy(void* dst, const void* src, size_t bytes, int blocks, void* stream) {
  p2p_copy_kernel<<<grid_for(bytes / 16, blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<uint4*>(dst), static_cast<const uint4*>(src), bytes / 16);
  return static_cast<int>(cudaGetLastError());
}
int tcl_barrier_all_mc(int32_t* mc_counter, const int32_t* local_counter, int world, int rank, int epoch, int32_t* status,
                       uint64_t timeout_ns, void* stream) {
  if (!mc_counter || !local_counter || world < 1 || rank < 0 || rank >= world) return static_cast<int>(cudaErrorInvalidValue);
  barrier_all_mc_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(mc_counter, local_counter, world, rank, epoch, status,
                                                                      timeout_ns ? timeout_ns : 4000000000ull);
  return static_cast<int>(cudaGetLastError());
}
int tcl_signal_pingpong(const int32_t* local_flag, int32_t* remote_flag, int mode, int initiator, int base, int rounds,
                        float* ns_per_rtt, int32_t* status, uint64_t timeout_ns, void* stream) {
  if (!local_flag || !remote_flag || mode < 0 || mode > 2 || rounds < 1) return static_cast<int>(cudaErrorInvalidValue);
  signal_pingpong_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(local_flag, remote_flag, mode, initiator, base, rounds, ns_per_rtt,
                                                                       status, timeout_ns ? timeout_ns : 2000000000ull);
  return static_cast<int>(cudaGetLastError());
}
int tcl_p2p_scatter(void* const* dst, const void* src, size_t slice_bytes, int world, int rank, int blocks, void* stream) {
  if (world < 2 || world > 8 || rank < 0 || rank >= world || slice_bytes % 16 != 0) return static_cast<int>(cudaErrorInvalidValue);
  ScatterArgs a = {};
  for (int i = 0; i < world; ++i) a.dst[i] = static_cast<uint4*>(dst[i]);
  const int peers = world - 1;
  int per_peer = (blocks > 0 ? blocks : 148 * 4) / peers;
  if (per_peer < 1) per_peer = 1;
  p2p_scatter_kernel<<<per_peer * peers, 256, 0, static_cast<cudaStream_t>(stream)>>>(a, static_cast<const uint4*>(src), slice_bytes / 16, world, rank);
  return static_cast<int>(cudaGetLastError());
}
}
