// signal_fanin: latency of "F producers tell one consumer they are done", push versus pull.
//   signal      producer: st.release.sys flag                      (no payload)
//   post        payload delivered and confirmed ahead of the timed window (producer: payload stores, st.release.sys
//               on a "pre" flag, then waits for a second go); timed: second go -> st.release.sys flag.  What a
//               signal costs when the data is already there, per payload size.
//   push        producer: payload stores, then st.release.sys flag
//   push_fence  producer: payload stores, __threadfence_system(), plain flag
//   pull        consumer GPU: F CTAs load their slot from the producers' memory
// F logical producers are CTAs dealt round-robin over the source GPUs (so F may exceed the number
// of GPUs).  A control kernel on the target releases a "go" flag per producer each round, polls the
// producers' completion flags, and times the round with clock64 (calibrated against CUDA events).
// Payload slots and an epoch stamp are verified after the last round.  Every spin is bounded.
//
// Producers and the consumer wait on one another, so they must run on different GPUs: the program
// needs a target and at least one other GPU.
//
// Reference parity: signalling/signal_fanin.cu (kernels :122-260, calibration :485-515, launch
// :626-673, verify :685-703, CSV header :557).
#include <string>
#include <vector>

#include "../common/host_common.hpp"
#include "../ptx/ldst_sys.cuh"
#include "../ptx/mbarrier.cuh"

using namespace tcl::host;
using namespace tcl::ptx;

enum Mode { kSignal, kPost, kPush, kPushFence, kPull };
static const char* kModeNames[] = {"signal", "post", "push", "push_fence", "pull"};

__device__ __forceinline__ bool spin_ge(const int* p, int want, unsigned long long deadline) {
  for (unsigned it = 0;; ++it) {
    if (ld_acquire_sys(p) - want >= 0) return true;
    if ((it & 127u) == 127u && globaltimer_ns() > deadline) return false;
  }
}

// One CTA per logical producer.  go[] and go2[] are local to the source GPU; sig[], pre[] and slots live on the target.
__global__ void source_kernel(const int* go, const int* go2, int* sig, int* pre, uint4* slots, const int* ids, size_t slot_vec, int rounds,
                              int mode, int* err, unsigned long long timeout_ns) {
  const int id = ids[blockIdx.x];
  const unsigned long long deadline = globaltimer_ns() + timeout_ns;
  __shared__ int ok;
  uint4* slot = slots + static_cast<size_t>(id) * slot_vec;
  for (int r = 1; r <= rounds; ++r) {
    if (threadIdx.x == 0) ok = spin_ge(go + id, r, deadline) ? 1 : 0;
    __syncthreads();
    if (!ok) { if (threadIdx.x == 0) atomicExch(err, 1); return; }
    if (mode == kPush || mode == kPushFence || mode == kPost) {
      const uint4 v = make_uint4(static_cast<unsigned>(r), static_cast<unsigned>(id), 0x5eed0000u + id, static_cast<unsigned>(r));
      for (size_t i = threadIdx.x; i < slot_vec; i += blockDim.x) st_v4(slot + i, v);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      if (mode == kSignal || mode == kPush) st_release_sys(sig + id, r);
      else if (mode == kPushFence) { __threadfence_system(); st_relaxed_sys(sig + id, r); }
      else {
        // post: confirm the delivery (untimed on the target), wait for the second go, then signal
        st_release_sys(pre + id, r);
        ok = spin_ge(go2 + id, r, deadline) ? 1 : 0;
        if (ok) st_release_sys(sig + id, r);
      }
    }
    __syncthreads();
    if (!ok) { if (threadIdx.x == 0) atomicExch(err, 1); return; }
  }
}

// Target control: thread i owns producer i.  cycles[r] = clock64 window of round r.  In post mode the window
// opens only after every producer has confirmed its payload.
__global__ void target_ctrl_kernel(int* const* go_ptrs, int* const* go2_ptrs, const int* sig, const int* pre, int fanin, int rounds, int mode,
                                   long long* cycles, int* err, unsigned long long timeout_ns) {
  const int i = threadIdx.x;
  const unsigned long long deadline = globaltimer_ns() + timeout_ns;
  __shared__ int bad;
  if (i == 0) bad = 0;
  __syncthreads();
  for (int r = 1; r <= rounds; ++r) {
    if (mode == kPost && i < fanin) {
      st_release_sys(go_ptrs[i], r);
      if (!spin_ge(pre + i, r, deadline)) bad = 1;
    }
    __syncthreads();
    if (bad) { if (i == 0) atomicExch(err, 1); return; }
    const long long c0 = clock64();
    if (i < fanin) {
      st_release_sys(mode == kPost ? go2_ptrs[i] : go_ptrs[i], r);
      if (!spin_ge(sig + i, r, deadline)) bad = 1;
    }
    __syncthreads();
    if (i == 0) cycles[r - 1] = clock64() - c0;
    if (bad) { if (i == 0) atomicExch(err, 1); return; }
  }
}

// Pull: one CTA per producer slot, all on the target.  Rounds are separated by a grid barrier on a
// global counter (cooperative launch keeps all CTAs resident).
__global__ void pull_kernel(const uint4* const* src_slots, uint4* dst_slots, size_t slot_vec, int rounds, int* counter,
                            long long* cycles, int* err, unsigned long long timeout_ns) {
  const unsigned long long deadline = globaltimer_ns() + timeout_ns;
  const int F = gridDim.x;
  __shared__ int ok;
  const uint4* src = src_slots[blockIdx.x];
  uint4* dst = dst_slots + static_cast<size_t>(blockIdx.x) * slot_vec;
  auto grid_barrier = [&](int phase) -> bool {
    __syncthreads();
    if (threadIdx.x == 0) {
      red_release_gpu_add(counter, 1);
      ok = wait_ge<false>(counter, phase * F, nullptr, deadline, nullptr, 0) ? 1 : 0;
    }
    __syncthreads();
    return ok != 0;
  };
  int phase = 0;
  for (int r = 0; r < rounds; ++r) {
    if (!grid_barrier(++phase)) { if (threadIdx.x == 0) atomicExch(err, 1); return; }
    const long long c0 = clock64();
    uint4 acc = make_uint4(0, 0, 0, 0);
    for (size_t i = threadIdx.x; i < slot_vec; i += blockDim.x) {
      const uint4 v = ld_v4_relaxed_sys(src + i);
      dst[i] = v;
      acc.x ^= v.x;
    }
    if (!grid_barrier(++phase)) { if (threadIdx.x == 0) atomicExch(err, 1); return; }
    if (blockIdx.x == 0 && threadIdx.x == 0) cycles[r] = clock64() - c0;
    if (acc.x == 0xdeadbeefu && r < 0) dst[0] = acc;  // keeps the loads alive
  }
}

__global__ void calib_kernel(long long spin_cycles, long long* out) {
  const long long c0 = clock64();
  while (clock64() - c0 < spin_cycles) {}
  if (threadIdx.x == 0) *out = clock64() - c0;
}

struct Config {
  std::vector<int> modes = {kSignal, kPost, kPush, kPushFence, kPull};
  std::vector<size_t> sizes;
  std::vector<int> fanins;
  std::vector<int> sources;
  int target = 0, threads = 256, rounds = 200, warmup = 20;
  bool check = true;
  std::string csv;
};

int main(int argc, char** argv) {
  Config c;
  Args a(argc, argv);
  while (a.more()) {
    std::string f = a.flag(), v;
    auto need = [&]() { if (!a.value(&v)) std::exit(1); return v; };
    if (f == "--modes") {
      c.modes.clear();
      for (auto& m : split_csv(need())) {
        int id = -1;
        for (int k = 0; k < 5; ++k) if (m == kModeNames[k]) id = k;
        if (id < 0) { std::fprintf(stderr, "unknown mode %s\n", m.c_str()); return 1; }
        c.modes.push_back(id);
      }
    } else if (f == "--sizes") parse_size_list(need(), &c.sizes);
    else if (f == "--fanin") parse_int_list(need(), &c.fanins);
    else if (f == "--sources") parse_int_list(need(), &c.sources);
    else if (f == "--target") c.target = std::atoi(need().c_str());
    else if (f == "--threads") c.threads = std::atoi(need().c_str());
    else if (f == "--rounds") c.rounds = std::atoi(need().c_str());
    else if (f == "--warmup") c.warmup = std::atoi(need().c_str());
    else if (f == "--no-check") c.check = false;
    else if (f == "--csv") c.csv = need();
    else {
      std::printf("usage: %s [--modes LIST] [--sizes LIST] [--fanin LIST] [--sources LIST] [--target N] [--threads N]\n"
                  "          [--rounds N] [--warmup N] [--no-check] [--csv FILE]\nmodes: signal post push push_fence pull\n", argv[0]);
      return f == "-h" || f == "--help" ? 0 : 1;
    }
  }
  const int ndev = device_count();
  if (c.sources.empty()) for (int d = 0; d < ndev; ++d) if (d != c.target) c.sources.push_back(d);
  if (c.sources.empty() || c.target >= ndev) {
    std::fprintf(stderr, "signal_fanin needs a target GPU and at least one other GPU (have %d)\n", ndev);
    return 1;
  }
  for (int s : c.sources) if (s == c.target || s >= ndev) { std::fprintf(stderr, "bad source %d\n", s); return 1; }
  if (c.sizes.empty()) parse_size_list("4K,32K,128K", &c.sizes);
  if (c.fanins.empty()) { for (int f = 1; f <= 7; ++f) c.fanins.push_back(f); c.fanins.push_back(16); c.fanins.push_back(32); }
  if (!enable_peer_all(ndev)) return 1;
  const int nsrc = static_cast<int>(c.sources.size());
  int max_f = 0;
  for (int f : c.fanins) max_f = std::max(max_f, f);
  size_t max_size = 16;
  for (size_t s : c.sizes) max_size = std::max(max_size, s);
  const int total_rounds = c.rounds + c.warmup;

  // Target-side buffers: sig flags, payload slots (push destination / pull destination), cycle log.
  TCL_CUDA_CHECK(cudaSetDevice(c.target));
  print_device_line(c.target);
  int *sig, *pre, *err_t, *counter;
  uint4* slots_t;
  long long *cycles, *calib;
  int** go_ptrs_d;
  int** go2_ptrs_d;
  const uint4** pull_src_d;
  TCL_CUDA_CHECK(cudaMalloc(&sig, max_f * 4));
  TCL_CUDA_CHECK(cudaMalloc(&pre, max_f * 4));
  TCL_CUDA_CHECK(cudaMalloc(&err_t, 4));
  TCL_CUDA_CHECK(cudaMalloc(&counter, 4));
  TCL_CUDA_CHECK(cudaMalloc(&slots_t, max_f * max_size));
  TCL_CUDA_CHECK(cudaMalloc(&cycles, total_rounds * 8));
  TCL_CUDA_CHECK(cudaMalloc(&calib, 8));
  TCL_CUDA_CHECK(cudaMalloc(&go_ptrs_d, max_f * sizeof(int*)));
  TCL_CUDA_CHECK(cudaMalloc(&go2_ptrs_d, max_f * sizeof(int*)));
  TCL_CUDA_CHECK(cudaMalloc(&pull_src_d, max_f * sizeof(uint4*)));
  cudaStream_t st_t;
  TCL_CUDA_CHECK(cudaStreamCreateWithFlags(&st_t, cudaStreamNonBlocking));
  cudaEvent_t e0, e1;
  TCL_CUDA_CHECK(cudaEventCreate(&e0));
  TCL_CUDA_CHECK(cudaEventCreate(&e1));
  // clock64 calibration on the target: median of three.
  double cyc_per_us = 0;
  {
    std::vector<double> r;
    for (int k = 0; k < 3; ++k) {
      TCL_CUDA_CHECK(cudaEventRecord(e0, st_t));
      calib_kernel<<<1, 32, 0, st_t>>>(20000000, calib);
      TCL_CUDA_CHECK(cudaEventRecord(e1, st_t));
      TCL_CUDA_CHECK(cudaStreamSynchronize(st_t));
      long long cyc;
      TCL_CUDA_CHECK(cudaMemcpy(&cyc, calib, 8, cudaMemcpyDeviceToHost));
      r.push_back(cyc / elapsed_us(e0, e1));
    }
    std::sort(r.begin(), r.end());
    cyc_per_us = r[1];
  }
  std::printf("# signal_fanin target=%d sources=%d GPUs rounds=%d warmup=%d  clock64: %.1f cycles/us\n", c.target, nsrc, c.rounds,
              c.warmup, cyc_per_us);

  // Source-side buffers.
  std::vector<int*> go(nsrc), go2(nsrc), ids_d(nsrc), err_s(nsrc);
  std::vector<uint4*> slots_s(nsrc);
  std::vector<cudaStream_t> st_s(nsrc);
  for (int g = 0; g < nsrc; ++g) {
    TCL_CUDA_CHECK(cudaSetDevice(c.sources[g]));
    TCL_CUDA_CHECK(cudaMalloc(&go[g], max_f * 4));
    TCL_CUDA_CHECK(cudaMalloc(&go2[g], max_f * 4));
    TCL_CUDA_CHECK(cudaMalloc(&ids_d[g], max_f * 4));
    TCL_CUDA_CHECK(cudaMalloc(&err_s[g], 4));
    TCL_CUDA_CHECK(cudaMalloc(&slots_s[g], max_f * max_size));
    TCL_CUDA_CHECK(cudaStreamCreateWithFlags(&st_s[g], cudaStreamNonBlocking));
  }
  Csv csv;
  if (!csv.open(c.csv, "mode,fanin,bytes,min_us,p50_us,p95_us,p99_us,verify")) return 1;
  std::printf("%-11s %6s %9s | %8s %8s %8s %8s | %s\n", "mode", "fanin", "bytes", "min_us", "p50_us", "p95_us", "p99_us", "verify");

  for (int mode : c.modes) {
    for (int F : c.fanins) {
      std::vector<size_t> sizes = (mode == kSignal) ? std::vector<size_t>{0} : c.sizes;
      for (size_t bytes : sizes) {
        const size_t slot_vec = bytes / 16;
        // Deal producers to source GPUs.
        std::vector<std::vector<int>> ids(nsrc);
        std::vector<int*> go_ptrs(F), go2_ptrs(F);
        std::vector<const uint4*> pull_src(F);
        for (int i = 0; i < F; ++i) {
          const int g = i % nsrc;
          ids[g].push_back(i);
          go_ptrs[i] = go[g] + i;
          go2_ptrs[i] = go2[g] + i;
          pull_src[i] = slots_s[g] + static_cast<size_t>(i) * slot_vec;
        }
        TCL_CUDA_CHECK(cudaSetDevice(c.target));
        TCL_CUDA_CHECK(cudaMemset(sig, 0, max_f * 4));
        TCL_CUDA_CHECK(cudaMemset(pre, 0, max_f * 4));
        TCL_CUDA_CHECK(cudaMemset(err_t, 0, 4));
        TCL_CUDA_CHECK(cudaMemset(counter, 0, 4));
        TCL_CUDA_CHECK(cudaMemset(slots_t, 0, max_f * max_size));
        TCL_CUDA_CHECK(cudaMemcpy(go_ptrs_d, go_ptrs.data(), F * sizeof(int*), cudaMemcpyHostToDevice));
        TCL_CUDA_CHECK(cudaMemcpy(go2_ptrs_d, go2_ptrs.data(), F * sizeof(int*), cudaMemcpyHostToDevice));
        TCL_CUDA_CHECK(cudaMemcpy(pull_src_d, pull_src.data(), F * sizeof(uint4*), cudaMemcpyHostToDevice));
        for (int g = 0; g < nsrc; ++g) {
          TCL_CUDA_CHECK(cudaSetDevice(c.sources[g]));
          TCL_CUDA_CHECK(cudaMemset(go[g], 0, max_f * 4));
          TCL_CUDA_CHECK(cudaMemset(go2[g], 0, max_f * 4));
          TCL_CUDA_CHECK(cudaMemset(err_s[g], 0, 4));
          TCL_CUDA_CHECK(cudaMemset(slots_s[g], 0x5a, max_f * max_size));
          if (!ids[g].empty()) TCL_CUDA_CHECK(cudaMemcpy(ids_d[g], ids[g].data(), ids[g].size() * 4, cudaMemcpyHostToDevice));
          TCL_CUDA_CHECK(cudaDeviceSynchronize());
        }
        TCL_CUDA_CHECK(cudaSetDevice(c.target));
        TCL_CUDA_CHECK(cudaDeviceSynchronize());
        bool launched = true;
        if (mode == kPull) {
          int max_blocks = 0, sms = 0;
          TCL_CUDA_CHECK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&max_blocks, pull_kernel, c.threads, 0));
          TCL_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, c.target));
          if (F > max_blocks * sms) { std::printf("%-11s %6d %9zu | skipped: more CTAs than can be co-resident\n", kModeNames[mode], F, bytes); continue; }
          const uint4* const* a0 = pull_src_d;
          uint4* a1 = slots_t;
          size_t a2 = slot_vec;
          int a3 = total_rounds;
          int* a4 = counter;
          long long* a5 = cycles;
          int* a6 = err_t;
          unsigned long long a7 = 4000000000ull;
          void* args[] = {&a0, &a1, &a2, &a3, &a4, &a5, &a6, &a7};
          TCL_CUDA_CHECK(cudaLaunchCooperativeKernel(reinterpret_cast<void*>(pull_kernel), dim3(F), dim3(c.threads), args, 0, st_t));
        } else {
          for (int g = 0; g < nsrc; ++g) {
            if (ids[g].empty()) continue;
            TCL_CUDA_CHECK(cudaSetDevice(c.sources[g]));
            source_kernel<<<static_cast<unsigned>(ids[g].size()), c.threads, 0, st_s[g]>>>(go[g], go2[g], sig, pre, slots_t, ids_d[g], slot_vec,
                                                                                         total_rounds, mode, err_s[g], 4000000000ull);
            TCL_CUDA_CHECK(cudaGetLastError());
          }
          TCL_CUDA_CHECK(cudaSetDevice(c.target));
          const int thr = std::max(64, (F + 31) / 32 * 32);
          target_ctrl_kernel<<<1, thr, 0, st_t>>>(go_ptrs_d, go2_ptrs_d, sig, pre, F, total_rounds, mode, cycles, err_t, 4000000000ull);
          TCL_CUDA_CHECK(cudaGetLastError());
        }
        if (!launched) continue;
        TCL_CUDA_CHECK(cudaSetDevice(c.target));
        TCL_CUDA_CHECK(cudaStreamSynchronize(st_t));
        int bad = 0, h = 0;
        TCL_CUDA_CHECK(cudaMemcpy(&h, err_t, 4, cudaMemcpyDeviceToHost));
        bad |= h;
        for (int g = 0; g < nsrc; ++g) {
          TCL_CUDA_CHECK(cudaSetDevice(c.sources[g]));
          TCL_CUDA_CHECK(cudaStreamSynchronize(st_s[g]));
          TCL_CUDA_CHECK(cudaMemcpy(&h, err_s[g], 4, cudaMemcpyDeviceToHost));
          bad |= h;
        }
        TCL_CUDA_CHECK(cudaSetDevice(c.target));
        std::vector<long long> cyc(total_rounds);
        TCL_CUDA_CHECK(cudaMemcpy(cyc.data(), cycles, total_rounds * 8, cudaMemcpyDeviceToHost));
        std::vector<double> us;
        for (int r = c.warmup; r < total_rounds; ++r) us.push_back(cyc[r] / cyc_per_us);
        Stats s = make_stats(us);
        // Verify payload (push: epoch stamp of the last round + producer id; pull: the 0x5a fill).
        const char* ver = "-";
        if (bad) ver = "TIMEOUT";
        else if (c.check && slot_vec > 0) {
          std::vector<uint32_t> hbuf(F * slot_vec * 4);
          TCL_CUDA_CHECK(cudaMemcpy(hbuf.data(), slots_t, hbuf.size() * 4, cudaMemcpyDeviceToHost));
          bool good = true;
          for (int i = 0; i < F && good; ++i)
            for (size_t k = 0; k < slot_vec && good; ++k) {
              const uint32_t* w = &hbuf[(static_cast<size_t>(i) * slot_vec + k) * 4];
              if (mode == kPull) good = w[0] == 0x5a5a5a5au && w[3] == 0x5a5a5a5au;
              else good = w[0] == static_cast<uint32_t>(total_rounds) && w[1] == static_cast<uint32_t>(i) && w[3] == static_cast<uint32_t>(total_rounds);
            }
          ver = good ? "ok" : "FAIL";
        }
        std::printf("%-11s %6d %9zu | %8.2f %8.2f %8.2f %8.2f | %s\n", kModeNames[mode], F, bytes, s.min, s.p50, s.p95, s.p99, ver);
        csv.row("%s,%d,%zu,%.3f,%.3f,%.3f,%.3f,%s", kModeNames[mode], F, bytes, s.min, s.p50, s.p95, s.p99, ver);
        if (bad) { std::fprintf(stderr, "a bounded wait ran out; stopping\n"); return 3; }
      }
    }
  }
  return 0;
}
