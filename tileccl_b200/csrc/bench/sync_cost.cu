// sync_cost: what the synchronisation primitives of the fused kernels cost.
//   1. flag ping-pong between two GPUs (st.release.sys / ld.acquire.sys): round trip, one-way = RTT/2
//   2. producer sequence: S bytes of stores to the peer, then (a) nothing, (b) st.release.sys flag,
//      (c) __threadfence_system() + plain flag, (d) red.release.sys.add: time per sequence
//   3. dependent remote atomic chain (atom.add.sys on peer memory): time per operation
//   4. local shared-memory mbarrier arrive + wait, and tcgen05.commit -> mbarrier: cycles per round
// Every spin is bounded; a wait that runs out sets an error flag and the section reports FAIL.
//
// Reference parity: tests/sync_cost.cu (kernels :82-160, sections :316-395); its tables have no CSV,
// --csv here writes section,variant,payload_bytes,value,unit.
#include <string>
#include <vector>

#include "../common/host_common.hpp"
#include "../ptx/ldst_sys.cuh"
#include "../ptx/mbarrier.cuh"
#include "../ptx/tcgen05.cuh"

using namespace tcl::host;
using namespace tcl::ptx;

__device__ __forceinline__ bool spin_until(const int* p, int want, unsigned long long deadline) {
  for (unsigned it = 0;; ++it) {
    if (ld_acquire_sys(p) - want >= 0) return true;
    if ((it & 255u) == 255u && globaltimer_ns() > deadline) return false;
  }
}

// role 0 starts each round; role 1 answers.  my_flag is local, peer_flag lives on the other GPU.
__global__ void pingpong_kernel(int* my_flag, int* peer_flag, int rounds, int role, unsigned long long* ns_out, int* err,
                                unsigned long long timeout_ns) {
  if (threadIdx.x != 0) return;
  const unsigned long long deadline = globaltimer_ns() + timeout_ns;
  unsigned long long t0 = 0;
  for (int r = 1; r <= rounds; ++r) {
    if (role == 0) {
      if (r == 2) t0 = globaltimer_ns();  // the first round trip absorbs the launch skew
      st_release_sys(peer_flag, r);
      if (!spin_until(my_flag, r, deadline)) { *err = 1; return; }
    } else {
      if (!spin_until(my_flag, r, deadline)) { *err = 1; return; }
      st_release_sys(peer_flag, r);
    }
  }
  if (role == 0) *ns_out = globaltimer_ns() - t0;
}

// variant: 0 stores only, 1 + st.release.sys flag, 2 + fence.sys + plain flag, 3 + red.release.sys.add
__global__ void signal_seq_kernel(uint4* payload, int* flag, size_t bytes, int reps, int variant, unsigned long long* ns_out) {
  const int lane = threadIdx.x;
  const size_t nvec = bytes / 16;
  __syncwarp();
  const unsigned long long t0 = globaltimer_ns();
  for (int r = 1; r <= reps; ++r) {
    const uint4 v = make_uint4(r, r, r, r);
    for (size_t i = lane; i < nvec; i += 32) st_v4(payload + i, v);
    __syncwarp();
    if (lane == 0) {
      if (variant == 1) st_release_sys(flag, r);
      else if (variant == 2) { __threadfence_system(); st_relaxed_sys(flag, r); }
      else if (variant == 3) red_release_sys_add(flag, 1);
    }
    __syncwarp();
  }
  // Close with one fence so that every variant has finished its traffic inside the window.
  if (lane == 0) { __threadfence_system(); *ns_out = globaltimer_ns() - t0; }
}

__global__ void atomic_rtt_kernel(int* remote, int n, unsigned long long* ns_out, int* sink) {
  if (threadIdx.x != 0) return;
  int v = 0;
  const unsigned long long t0 = globaltimer_ns();
  for (int i = 0; i < n; ++i) v = atom_add_acq_rel_sys(remote, v & 1) + 1;  // each op depends on the last
  *ns_out = globaltimer_ns() - t0;
  *sink = v;
}

__global__ void mbarrier_cycle_kernel(int rounds, long long* cycles_plain, long long* cycles_commit, int* err) {
  __shared__ __align__(8) unsigned long long bar[2];
  __shared__ uint32_t tmem_slot;
  const int lane = threadIdx.x;
  if (lane == 0) { mbar_init(smem_u32(&bar[0]), 1); mbar_init(smem_u32(&bar[1]), 1); fence_mbar_init(); }
  __syncwarp();
  int abort_flag = 0;
  const unsigned long long deadline = globaltimer_ns() + 2000000000ull;
  if (lane == 0) {
    long long c0 = clock64();
    for (int r = 0; r < rounds; ++r) {
      mbar_arrive(smem_u32(&bar[0]));
      if (!mbar_wait(smem_u32(&bar[0]), r & 1, &abort_flag, deadline)) { *err = 1; break; }
    }
    *cycles_plain = (clock64() - c0) / rounds;
  }
  __syncwarp();
  // tcgen05.commit with nothing outstanding arrives as soon as the tensor pipe sees it.
  tmem_alloc<1>(smem_u32(&tmem_slot), 32);
  tmem_relinquish<1>();
  tc_fence_before_sync();
  __syncwarp();
  tc_fence_after_sync();
  if (lane == 0) {
    long long c0 = clock64();
    for (int r = 0; r < rounds; ++r) {
      tc_commit_1cta(smem_u32(&bar[1]));
      if (!mbar_wait(smem_u32(&bar[1]), r & 1, &abort_flag, deadline)) { *err = 1; break; }
    }
    *cycles_commit = (clock64() - c0) / rounds;
  }
  __syncwarp();
  tmem_dealloc<1>(tmem_slot, 32);
}

int main(int argc, char** argv) {
  int rounds = 2000, iters = 200, src = 0, dst = 1;
  std::vector<size_t> sizes;
  std::string csv_path;
  Args a(argc, argv);
  while (a.more()) {
    std::string f = a.flag(), v;
    if (f == "--rounds" && a.value(&v)) rounds = std::atoi(v.c_str());
    else if (f == "--sizes" && a.value(&v)) parse_size_list(v, &sizes);
    else if (f == "--iters" && a.value(&v)) iters = std::atoi(v.c_str());
    else if (f == "--src" && a.value(&v)) src = std::atoi(v.c_str());
    else if (f == "--dst" && a.value(&v)) dst = std::atoi(v.c_str());
    else if (f == "--csv" && a.value(&v)) csv_path = v;
    else {
      std::printf("usage: %s [--rounds N] [--sizes LIST] [--iters N] [--src N] [--dst N] [--csv FILE]\n", argv[0]);
      return f == "-h" || f == "--help" ? 0 : 1;
    }
  }
  if (sizes.empty()) parse_size_list("0,512,2K,8K,32K,128K", &sizes);
  const int ndev = device_count();
  if (src >= ndev || dst >= ndev) { std::fprintf(stderr, "need GPUs %d and %d, have %d\n", src, dst, ndev); return 1; }
  const bool two = src != dst;
  if (two && !enable_peer_all(std::max(src, dst) + 1)) return 1;
  Csv csv;
  if (!csv.open(csv_path, "section,variant,payload_bytes,value,unit")) return 1;
  print_device_line(src);

  // Buffers: flags + payload on both GPUs.
  int *flag_s, *flag_d, *err_s, *err_d, *sink;
  unsigned long long *ns_s;
  uint4* payload_d;
  const size_t max_bytes = 1 << 20;
  TCL_CUDA_CHECK(cudaSetDevice(dst));
  TCL_CUDA_CHECK(cudaMalloc(&flag_d, 256)); TCL_CUDA_CHECK(cudaMemset(flag_d, 0, 256));
  TCL_CUDA_CHECK(cudaMalloc(&err_d, 4)); TCL_CUDA_CHECK(cudaMemset(err_d, 0, 4));
  TCL_CUDA_CHECK(cudaMalloc(&payload_d, max_bytes));
  TCL_CUDA_CHECK(cudaSetDevice(src));
  TCL_CUDA_CHECK(cudaMalloc(&flag_s, 256)); TCL_CUDA_CHECK(cudaMemset(flag_s, 0, 256));
  TCL_CUDA_CHECK(cudaMalloc(&err_s, 4)); TCL_CUDA_CHECK(cudaMemset(err_s, 0, 4));
  TCL_CUDA_CHECK(cudaMalloc(&ns_s, 64)); TCL_CUDA_CHECK(cudaMalloc(&sink, 4));
  auto read_ns = [&]() { unsigned long long h = 0; TCL_CUDA_CHECK(cudaMemcpy(&h, ns_s, 8, cudaMemcpyDeviceToHost)); return h; };
  auto read_err = [&](int* p, int dev) { int h = 0; TCL_CUDA_CHECK(cudaSetDevice(dev)); TCL_CUDA_CHECK(cudaMemcpy(&h, p, 4, cudaMemcpyDeviceToHost)); TCL_CUDA_CHECK(cudaSetDevice(src)); return h; };

  // 1. ping-pong (two kernels that wait on one another: only across two GPUs)
  std::printf("\n## 1. flag ping-pong (st.release.sys / ld.acquire.sys), %d rounds\n", rounds);
  if (two) {
    cudaStream_t s0, s1;
    TCL_CUDA_CHECK(cudaStreamCreate(&s0));
    TCL_CUDA_CHECK(cudaSetDevice(dst));
    TCL_CUDA_CHECK(cudaStreamCreate(&s1));
    pingpong_kernel<<<1, 32, 0, s1>>>(flag_d, flag_s, rounds, 1, nullptr, err_d, 4000000000ull);
    TCL_CUDA_CHECK(cudaSetDevice(src));
    pingpong_kernel<<<1, 32, 0, s0>>>(flag_s, flag_d, rounds, 0, ns_s, err_s, 4000000000ull);
    TCL_CUDA_CHECK(cudaStreamSynchronize(s0));
    TCL_CUDA_CHECK(cudaSetDevice(dst));
    TCL_CUDA_CHECK(cudaStreamSynchronize(s1));
    TCL_CUDA_CHECK(cudaSetDevice(src));
    if (read_err(err_s, src) || read_err(err_d, dst)) std::printf("ping-pong: FAIL (a wait ran out)\n");
    else {
      const double rtt = read_ns() / 1000.0 / (rounds - 1);
      std::printf("round trip %.2f us   one-way %.2f us\n", rtt, rtt / 2);
      csv.row("pingpong,rtt,0,%.3f,us", rtt);
      csv.row("pingpong,one_way,0,%.3f,us", rtt / 2);
    }
  } else {
    std::printf("skipped: needs two GPUs (two kernels that wait on one another never share a GPU)\n");
  }

  // 2. producer sequences
  std::printf("\n## 2. producer sequence, one warp, us per sequence (%d repetitions)\n", iters);
  std::printf("%10s %12s %14s %18s %16s\n", "bytes", "stores", "+release flag", "+fence+plain flag", "+red.release");
  uint4* payload = payload_d;
  int* flag = two ? flag_d : flag_s;
  const char* vname[4] = {"stores", "release_flag", "fence_flag", "red_release"};
  for (size_t s : sizes) {
    if (s > max_bytes) continue;
    std::printf("%10zu", s);
    for (int variant = 0; variant < 4; ++variant) {
      signal_seq_kernel<<<1, 32>>>(payload, flag + 8, s, iters, variant, ns_s);
      TCL_CUDA_CHECK(cudaDeviceSynchronize());
      const double us = read_ns() / 1000.0 / iters;
      std::printf(" %*.3f", variant == 0 ? 12 : variant == 1 ? 14 : variant == 2 ? 18 : 16, us);
      csv.row("signal_seq,%s,%zu,%.4f,us", vname[variant], s, us);
    }
    std::printf("\n");
  }

  // 3. dependent remote atomics
  std::printf("\n## 3. dependent atom.add.acq_rel.sys chain on %s memory\n", two ? "peer" : "local");
  atomic_rtt_kernel<<<1, 32>>>(flag + 16, rounds, ns_s, sink);
  TCL_CUDA_CHECK(cudaDeviceSynchronize());
  const double aus = read_ns() / 1000.0 / rounds;
  std::printf("%.3f us per operation\n", aus);
  csv.row("atomic_rtt,%s,4,%.4f,us", two ? "peer" : "local", aus);

  // 4. mbarrier
  std::printf("\n## 4. shared-memory mbarrier, cycles per arrive+wait round\n");
  long long *cyc;
  TCL_CUDA_CHECK(cudaMalloc(&cyc, 16));
  mbarrier_cycle_kernel<<<1, 32>>>(100000, cyc, cyc + 1, err_s);
  TCL_CUDA_CHECK(cudaDeviceSynchronize());
  long long h[2];
  TCL_CUDA_CHECK(cudaMemcpy(h, cyc, 16, cudaMemcpyDeviceToHost));
  if (read_err(err_s, src)) std::printf("mbarrier: FAIL (a wait ran out)\n");
  else {
    std::printf("mbarrier.arrive + try_wait: %lld cycles    tcgen05.commit -> mbarrier: %lld cycles\n", h[0], h[1]);
    csv.row("mbarrier,arrive_wait,0,%lld,cycles", h[0]);
    csv.row("mbarrier,tcgen05_commit,0,%lld,cycles", h[1]);
  }
  return 0;
}
