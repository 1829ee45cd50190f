// peer_l2_probe: is a peer GPU's memory cached in the *requesting* GPU's L2?
//
// Instruments
//   bw    stream a working set that wraps around (sizes across the L2 capacity) and time it:
//         against local memory the bandwidth has a knee at the L2 size; if peer memory were cached
//         by the reader's L2 the peer curve would show the same knee
//   lat   pointer chase over a random cycle of 128-byte lines (one thread): ns per hop
//   wire  bracket the same streaming with the NVLink byte counters of `nvidia-smi nvlink -gt d`:
//         bytes on the wire / bytes asked for ~ 1 means nothing was served from a local cache
//   once  one launch of the bw kernel, for a profiler
// Axes: --via ldst | tma (cp.async.bulk through shared memory), --dir read | write,
//       --cache ca | cg | na (L1 policy of the ldst loads, written in the instruction; the reference
//       builds the program twice, with and without -dlcm=cg), targets local (control) and peer.
//
// Reference parity: l2_peer_cache/peer_l2_probe.cu (kernels :197-534, NVLink counters :550-591,
// sizes :761-786, knee :909-929, bw :931-1001, chase :1003-1086, wire :1088-1224, CSV :1365-1375).
#include <algorithm>
#include <numeric>
#include <random>
#include <string>
#include <vector>

#include "../common/host_common.hpp"
#include "movers.cuh"

using namespace tcl::host;
using namespace tcl::bench;
namespace ptx = tcl::ptx;

enum Cache { kCa = 0, kCg = 1, kNa = 2 };

template <int kCache>
__device__ __forceinline__ uint4 load16(const uint4* p) {
  if (kCache == kCa) return ptx::ld_v4_ca(p);
  if (kCache == kCg) return ptx::ld_v4_cg(p);
  return ptx::ld_v4_stream(p);
}

// Thread t starts at vector t % n_vec and advances by stride_vec (wrapping) `iters` times.
template <int kCache>
__global__ void __launch_bounds__(1024) stream_read_kernel(const uint4* p, size_t n_vec, size_t stride_vec, unsigned long long iters,
                                                            uint32_t* sink) {
  size_t i = (blockIdx.x * (size_t)blockDim.x + threadIdx.x) % n_vec;
  uint4 acc = make_uint4(0, 0, 0, 0);
#pragma unroll 4
  for (unsigned long long k = 0; k < iters; ++k) {
    const uint4 v = load16<kCache>(p + i);
    acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    i += stride_vec;
    if (i >= n_vec) i -= n_vec;
  }
  uint32_t s = acc.x + acc.y + acc.z + acc.w;
  for (int o = 16; o; o >>= 1) s += __shfl_down_sync(0xffffffffu, s, o);
  if ((threadIdx.x & 31) == 0) atomicAdd(sink + (blockIdx.x & 255), s);
}

__global__ void __launch_bounds__(1024) stream_write_kernel(uint4* p, size_t n_vec, size_t stride_vec, unsigned long long iters, uint4 val) {
  size_t i = (blockIdx.x * (size_t)blockDim.x + threadIdx.x) % n_vec;
#pragma unroll 4
  for (unsigned long long k = 0; k < iters; ++k) {
    ptx::st_v4(p + i, val);
    i += stride_vec;
    if (i >= n_vec) i -= n_vec;
  }
  __threadfence_system();
}

__global__ void count_not_equal_kernel(const uint32_t* p, size_t n, uint32_t val, unsigned long long* bad) {
  unsigned long long c = 0;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) c += p[i] != val;
  if (c) atomicAdd(bad, c);
}

__global__ void sum_kernel(const uint32_t* p, size_t n, unsigned long long* out) {
  unsigned long long c = 0;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) c += p[i];
  atomicAdd(out, c);
}

// next[] holds, in the first word of every 128-byte line, the index of the next line.
__global__ void scatter_chain_kernel(uint32_t* base, const uint32_t* next, size_t lines) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < lines; i += (size_t)gridDim.x * blockDim.x) base[i * 32] = next[i];
}
template <int kCache>
__global__ void chase_kernel(const uint32_t* base, int hops, long long* cycles, uint32_t* sink) {
  uint32_t i = 0;
  const long long c0 = clock64();
  for (int h = 0; h < hops; ++h) {
    uint32_t v;
    if (kCache == kCa) asm volatile("ld.global.ca.u32 %0, [%1];" : "=r"(v) : "l"(base + (size_t)i * 32) : "memory");
    else asm volatile("ld.global.cg.u32 %0, [%1];" : "=r"(v) : "l"(base + (size_t)i * 32) : "memory");
    i = v;
  }
  *cycles = clock64() - c0;
  *sink = i;
}

struct Config {
  int reader = 0, owner = 1;
  std::vector<std::string> modes = {"bw", "lat", "wire"};
  std::vector<std::string> targets = {"local", "peer"};
  std::string via = "ldst", dir = "read", cache = "ca", csv;
  size_t tma_tile = 8192, total = size_t(4) << 30, wire_total = size_t(64) << 30;
  std::vector<size_t> sizes, wire_sizes;
  int reps = 5, blocks = 0, threads = 256, hops = 20000, wire_launches = 8, idle_ms = 500;
  bool counters = true, verify = true;
};

struct Buffers {
  char* local = nullptr;
  char* peer = nullptr;
  size_t bytes = 0;
  uint32_t* sink = nullptr;
  int* err = nullptr;
};

struct Ctx {
  Config c;
  Buffers b;
  int sms = 0, l2 = 0;
  cudaEvent_t e0, e1;
};

static int cache_id(const std::string& s) { return s == "cg" ? kCg : s == "na" ? kNa : kCa; }

// One timed pass over a working set of `bytes` moving `total` logical bytes.  Returns milliseconds.
static double time_op(Ctx& x, char* base, size_t bytes, size_t total, size_t* logical, unsigned long long* iters_out) {
  const Config& c = x.c;
  const int blocks = c.blocks > 0 ? c.blocks : 4 * x.sms;
  const size_t n_vec = bytes / 16;
  const size_t threads_total = static_cast<size_t>(blocks) * c.threads;
  if (c.via == "tma") {
    // The bulk mover walks `total` bytes; wrap the working set by launching over [base, base+bytes) repeatedly.
    const size_t passes = std::max<size_t>(1, total / bytes);
    *logical = passes * bytes;
    *iters_out = passes;
    TCL_CUDA_CHECK(cudaEventRecord(x.e0));
    for (size_t p = 0; p < passes; ++p)
      TCL_CUDA_CHECK(launch_bulk_pipe(4, std::min<int>(blocks, std::max<size_t>(1, bytes / c.tma_tile)), 0, base, base, bytes,
                                      static_cast<uint32_t>(std::min(c.tma_tile, bytes)),
                                      c.dir == "read" ? kBulkLoadOnly : kBulkStoreOnly, x.b.err, 2000000000ull));
    TCL_CUDA_CHECK(cudaEventRecord(x.e1));
  } else {
    unsigned long long iters = std::max<size_t>(1, total / 16 / threads_total);
    *logical = iters * threads_total * 16;
    *iters_out = iters;
    const size_t stride = threads_total % n_vec;
    TCL_CUDA_CHECK(cudaEventRecord(x.e0));
    if (c.dir == "write") {
      stream_write_kernel<<<blocks, c.threads>>>(reinterpret_cast<uint4*>(base), n_vec, stride, iters, make_uint4(0xabcd1234u, 0xabcd1234u, 0xabcd1234u, 0xabcd1234u));
    } else {
      switch (cache_id(c.cache)) {
        case kCg: stream_read_kernel<kCg><<<blocks, c.threads>>>(reinterpret_cast<const uint4*>(base), n_vec, stride, iters, x.b.sink); break;
        case kNa: stream_read_kernel<kNa><<<blocks, c.threads>>>(reinterpret_cast<const uint4*>(base), n_vec, stride, iters, x.b.sink); break;
        default: stream_read_kernel<kCa><<<blocks, c.threads>>>(reinterpret_cast<const uint4*>(base), n_vec, stride, iters, x.b.sink); break;
      }
    }
    TCL_CUDA_CHECK(cudaGetLastError());
    TCL_CUDA_CHECK(cudaEventRecord(x.e1));
  }
  TCL_CUDA_CHECK(cudaEventSynchronize(x.e1));
  return elapsed_us(x.e0, x.e1) / 1000.0;
}

// Largest ratio between the bandwidth of consecutive sizes around the L2 capacity.
static double find_knee(const std::vector<size_t>& sizes, const std::vector<double>& gbps, size_t l2) {
  double in_l2 = 0, out_l2 = 1e30;
  for (size_t i = 0; i < sizes.size(); ++i) {
    if (sizes[i] <= l2 / 4) in_l2 = std::max(in_l2, gbps[i]);
    if (sizes[i] >= 2 * l2) out_l2 = std::min(out_l2, gbps[i]);
  }
  return (in_l2 > 0 && out_l2 < 1e29 && out_l2 > 0) ? in_l2 / out_l2 : 0.0;
}

// NVLink data counters of one GPU, summed over links, in KiB (rx, tx).  false if unavailable.
static bool read_nvlink_kib(int dev, double* rx, double* tx) {
  char cmd[128];
  std::snprintf(cmd, sizeof(cmd), "nvidia-smi nvlink -gt d -i %d 2>/dev/null", dev);
  FILE* p = popen(cmd, "r");
  if (!p) return false;
  char line[256];
  double r = 0, t = 0;
  int found = 0;
  while (std::fgets(line, sizeof(line), p)) {
    double v;
    const char* q;
    if ((q = std::strstr(line, "Data Rx:")) && std::sscanf(q + 8, "%lf", &v) == 1) { r += v; ++found; }
    if ((q = std::strstr(line, "Data Tx:")) && std::sscanf(q + 8, "%lf", &v) == 1) { t += v; ++found; }
  }
  pclose(p);
  *rx = r; *tx = t;
  return found > 0;
}

int main(int argc, char** argv) {
  Config c;
  Args a(argc, argv);
  while (a.more()) {
    std::string f = a.flag(), v;
    auto need = [&]() { if (!a.value(&v)) std::exit(1); return v; };
    if (f == "--reader") c.reader = std::atoi(need().c_str());
    else if (f == "--owner") c.owner = std::atoi(need().c_str());
    else if (f == "--modes") c.modes = split_csv(need());
    else if (f == "--targets") c.targets = split_csv(need());
    else if (f == "--via") c.via = need();
    else if (f == "--dir") c.dir = need();
    else if (f == "--cache") c.cache = need();
    else if (f == "--tma-tile") parse_bytes(need(), &c.tma_tile);
    else if (f == "--sizes") parse_size_list(need(), &c.sizes);
    else if (f == "--total") parse_bytes(need(), &c.total);
    else if (f == "--reps") c.reps = std::atoi(need().c_str());
    else if (f == "--blocks") c.blocks = std::atoi(need().c_str());
    else if (f == "--threads") c.threads = std::atoi(need().c_str());
    else if (f == "--hops") c.hops = std::atoi(need().c_str());
    else if (f == "--wire-sizes") parse_size_list(need(), &c.wire_sizes);
    else if (f == "--wire-total") parse_bytes(need(), &c.wire_total);
    else if (f == "--wire-launches") c.wire_launches = std::atoi(need().c_str());
    else if (f == "--idle-ms") c.idle_ms = std::atoi(need().c_str());
    else if (f == "--no-counters") c.counters = false;
    else if (f == "--no-verify") c.verify = false;
    else if (f == "--csv") c.csv = need();
    else {
      std::printf("usage: %s [--reader N] [--owner N] [--modes bw,lat,wire,once] [--targets local,peer] [--via ldst|tma]\n"
                  "          [--dir read|write] [--cache ca|cg|na] [--tma-tile B] [--sizes LIST] [--total B] [--reps N] [--blocks N]\n"
                  "          [--threads N] [--hops N] [--wire-sizes LIST] [--wire-total B] [--wire-launches N] [--idle-ms N]\n"
                  "          [--no-counters] [--no-verify] [--csv PREFIX]\n", argv[0]);
      return f == "-h" || f == "--help" ? 0 : 1;
    }
  }
  const int ndev = device_count();
  const bool have_peer = c.owner != c.reader && c.owner < ndev;
  if (c.reader >= ndev) { std::fprintf(stderr, "no GPU %d\n", c.reader); return 1; }
  if (!have_peer) {
    c.targets = {"local"};
    std::printf("# only one GPU usable: running the local control only\n");
  } else if (!enable_peer_all(std::max(c.reader, c.owner) + 1)) return 1;

  Ctx x;
  x.c = c;
  TCL_CUDA_CHECK(cudaSetDevice(c.reader));
  TCL_CUDA_CHECK(cudaDeviceGetAttribute(&x.sms, cudaDevAttrMultiProcessorCount, c.reader));
  TCL_CUDA_CHECK(cudaDeviceGetAttribute(&x.l2, cudaDevAttrL2CacheSize, c.reader));
  print_device_line(c.reader);
  const size_t l2 = static_cast<size_t>(x.l2);
  if (c.sizes.empty()) {
    for (size_t s : {size_t(128) << 10, size_t(256) << 10, size_t(512) << 10}) c.sizes.push_back(s);
    for (int sh = 6; sh >= -3; --sh) c.sizes.push_back(sh >= 0 ? l2 >> sh : l2 << -sh);
    for (auto& s : c.sizes) s = s / 4096 * 4096;
    x.c.sizes = c.sizes;
  }
  if (c.wire_sizes.empty()) { parse_size_list("1M,8M,64M", &c.wire_sizes); x.c.wire_sizes = c.wire_sizes; }
  size_t max_bytes = 0;
  for (size_t s : c.sizes) max_bytes = std::max(max_bytes, s);
  for (size_t s : c.wire_sizes) max_bytes = std::max(max_bytes, s);
  Buffers& b = x.b;
  b.bytes = max_bytes;
  TCL_CUDA_CHECK(cudaMalloc(&b.local, max_bytes));
  TCL_CUDA_CHECK(cudaMalloc(&b.sink, 256 * 4));
  TCL_CUDA_CHECK(cudaMemset(b.sink, 0, 256 * 4));
  TCL_CUDA_CHECK(cudaMalloc(&b.err, 4));
  TCL_CUDA_CHECK(cudaMemset(b.err, 0, 4));
  TCL_CUDA_CHECK(cudaEventCreate(&x.e0));
  TCL_CUDA_CHECK(cudaEventCreate(&x.e1));
  fill_pattern_kernel<<<1024, 256>>>(reinterpret_cast<uint32_t*>(b.local), max_bytes / 4, 7u);
  if (have_peer) {
    TCL_CUDA_CHECK(cudaSetDevice(c.owner));
    TCL_CUDA_CHECK(cudaMalloc(&b.peer, max_bytes));
    fill_pattern_kernel<<<1024, 256>>>(reinterpret_cast<uint32_t*>(b.peer), max_bytes / 4, 7u);
    TCL_CUDA_CHECK(cudaDeviceSynchronize());
    TCL_CUDA_CHECK(cudaSetDevice(c.reader));
    // The peer pointer must really belong to the owner GPU.
    cudaPointerAttributes at;
    TCL_CUDA_CHECK(cudaPointerGetAttributes(&at, b.peer));
    if (at.device != c.owner) { std::fprintf(stderr, "peer buffer is on device %d, expected %d\n", at.device, c.owner); return 1; }
  }
  TCL_CUDA_CHECK(cudaDeviceSynchronize());
  if (c.verify && have_peer) {
    // Checksums: owner's own view, reader's view of the peer buffer, reader's local copy: all equal.
    unsigned long long* d;
    TCL_CUDA_CHECK(cudaMalloc(&d, 24));
    TCL_CUDA_CHECK(cudaMemset(d, 0, 24));
    sum_kernel<<<256, 256>>>(reinterpret_cast<uint32_t*>(b.local), max_bytes / 4, d);
    sum_kernel<<<256, 256>>>(reinterpret_cast<uint32_t*>(b.peer), max_bytes / 4, d + 1);
    TCL_CUDA_CHECK(cudaDeviceSynchronize());
    unsigned long long h[3];
    TCL_CUDA_CHECK(cudaMemcpy(h, d, 24, cudaMemcpyDeviceToHost));
    std::printf("# checksum local %llx, peer-as-seen-by-reader %llx: %s\n", h[0], h[1], h[0] == h[1] ? "match" : "MISMATCH");
    if (h[0] != h[1]) return 1;
  }
  Csv csv_bw, csv_lat, csv_wire;
  if (!c.csv.empty()) {
    if (!csv_bw.open(c.csv + "_bw.csv", "build,target,bytes,frac_l2,iters_per_thread,blocks,threads,logical_bytes,ms_med,ms_min,gbps,via,dir,tma_tile_bytes")) return 1;
    if (!csv_lat.open(c.csv + "_lat.csv", "build,target,bytes,frac_l2,lines,hops,ms,ns_per_hop")) return 1;
    if (!csv_wire.open(c.csv + "_wire.csv", "build,target,bytes,launches,iters_per_thread,asked_bytes,ms,gbps,wire_rx_bytes,wire_tx_bytes,rx_over_asked,tx_over_asked,idle_rx_bps,idle_tx_bps,counters_ok,via,dir,tma_tile_bytes")) return 1;
  }
  const int blocks = c.blocks > 0 ? c.blocks : 4 * x.sms;
  auto has = [&](const char* m) { return std::find(c.modes.begin(), c.modes.end(), m) != c.modes.end(); };
  auto base_of = [&](const std::string& t) { return t == "peer" ? b.peer : b.local; };

  if (has("once")) {
    for (auto& t : c.targets) {
      size_t logical; unsigned long long iters;
      const double ms = time_op(x, base_of(t), c.sizes.back(), c.total, &logical, &iters);
      std::printf("once %s: %zu bytes working set, %.3f ms, %.1f GB/s\n", t.c_str(), c.sizes.back(), ms, logical / ms / 1e6);
    }
  }
  if (has("bw")) {
    std::printf("\n## bw  via=%s dir=%s cache=%s  (L2 = %.1f MiB)\n%12s %8s", c.via.c_str(), c.dir.c_str(), c.cache.c_str(), l2 / 1048576.0, "bytes", "x L2");
    for (auto& t : c.targets) std::printf(" %12s GB/s", t.c_str());
    std::printf("\n");
    std::vector<std::vector<double>> curves(c.targets.size());
    for (size_t s : c.sizes) {
      std::printf("%12zu %8.3f", s, static_cast<double>(s) / l2);
      for (size_t ti = 0; ti < c.targets.size(); ++ti) {
        size_t logical = 0; unsigned long long iters = 0;
        time_op(x, base_of(c.targets[ti]), s, c.total / 8, &logical, &iters);  // warm
        std::vector<double> ms;
        for (int r = 0; r < c.reps; ++r) ms.push_back(time_op(x, base_of(c.targets[ti]), s, c.total, &logical, &iters));
        Stats st = make_stats(ms);
        const double gbps = logical / st.p50 / 1e6;
        curves[ti].push_back(gbps);
        std::printf(" %17.1f", gbps);
        csv_bw.row("%s,%s,%zu,%.4f,%llu,%d,%d,%zu,%.4f,%.4f,%.2f,%s,%s,%zu", c.cache.c_str(), c.targets[ti].c_str(), s,
                   static_cast<double>(s) / l2, iters, blocks, c.threads, logical, st.p50, st.min, gbps, c.via.c_str(), c.dir.c_str(), c.tma_tile);
      }
      std::printf("\n");
    }
    for (size_t ti = 0; ti < c.targets.size(); ++ti) {
      const double knee = find_knee(c.sizes, curves[ti], l2);
      std::printf("knee(%s) = %.2fx (bandwidth inside L2/4 over bandwidth beyond 2 x L2)\n", c.targets[ti].c_str(), knee);
    }
    if (c.dir == "write" && c.verify) {
      for (auto& t : c.targets) {
        unsigned long long* bad;
        TCL_CUDA_CHECK(cudaMalloc(&bad, 8));
        TCL_CUDA_CHECK(cudaMemset(bad, 0, 8));
        if (t == "peer") TCL_CUDA_CHECK(cudaSetDevice(c.owner));
        count_not_equal_kernel<<<256, 256>>>(reinterpret_cast<uint32_t*>(base_of(t)), c.sizes.front() / 4, 0xabcd1234u, bad);
        TCL_CUDA_CHECK(cudaDeviceSynchronize());
        unsigned long long h;
        TCL_CUDA_CHECK(cudaMemcpy(&h, bad, 8, cudaMemcpyDeviceToHost));
        TCL_CUDA_CHECK(cudaSetDevice(c.reader));
        std::printf("write landing check on the owner of %s: %s\n", t.c_str(), h == 0 ? "ok" : "FAIL");
      }
    }
  }
  if (has("lat") && c.dir == "read") {
    std::printf("\n## lat  (one thread, %d hops over a random cycle of 128-byte lines, cache=%s)\n%12s %8s", c.hops, c.cache.c_str(), "bytes", "x L2");
    for (auto& t : c.targets) std::printf(" %10s ns/hop", t.c_str());
    std::printf("\n");
    int clk_khz = 0;
    TCL_CUDA_CHECK(cudaDeviceGetAttribute(&clk_khz, cudaDevAttrClockRate, c.reader));
    long long* cyc;
    uint32_t* nxt;
    TCL_CUDA_CHECK(cudaMalloc(&cyc, 8));
    for (size_t s : c.sizes) {
      const size_t lines = s / 128;
      if (lines < 2) continue;
      // Sattolo's algorithm: one cycle through all lines.
      std::vector<uint32_t> perm(lines);
      std::iota(perm.begin(), perm.end(), 0u);
      std::mt19937_64 rng(lines);
      for (size_t i = lines - 1; i > 0; --i) std::swap(perm[i], perm[rng() % i]);
      TCL_CUDA_CHECK(cudaMalloc(&nxt, lines * 4));
      TCL_CUDA_CHECK(cudaMemcpy(nxt, perm.data(), lines * 4, cudaMemcpyHostToDevice));
      std::printf("%12zu %8.3f", s, static_cast<double>(s) / l2);
      for (auto& t : c.targets) {
        scatter_chain_kernel<<<256, 256>>>(reinterpret_cast<uint32_t*>(base_of(t)), nxt, lines);
        TCL_CUDA_CHECK(cudaDeviceSynchronize());
        TCL_CUDA_CHECK(cudaEventRecord(x.e0));
        if (cache_id(c.cache) == kCa) chase_kernel<kCa><<<1, 1>>>(reinterpret_cast<uint32_t*>(base_of(t)), c.hops, cyc, b.sink);
        else chase_kernel<kCg><<<1, 1>>>(reinterpret_cast<uint32_t*>(base_of(t)), c.hops, cyc, b.sink);
        TCL_CUDA_CHECK(cudaEventRecord(x.e1));
        TCL_CUDA_CHECK(cudaEventSynchronize(x.e1));
        const double ms = elapsed_us(x.e0, x.e1) / 1000.0;
        const double ns = ms * 1e6 / c.hops;
        std::printf(" %17.1f", ns);
        csv_lat.row("%s,%s,%zu,%.4f,%zu,%d,%.4f,%.2f", c.cache.c_str(), t.c_str(), s, static_cast<double>(s) / l2, lines, c.hops, ms, ns);
      }
      std::printf("\n");
      TCL_CUDA_CHECK(cudaFree(nxt));
      // restore the data pattern for the later instruments
      fill_pattern_kernel<<<1024, 256>>>(reinterpret_cast<uint32_t*>(b.local), s / 4, 7u);
      if (have_peer) fill_pattern_kernel<<<1024, 256>>>(reinterpret_cast<uint32_t*>(b.peer), s / 4, 7u);
      TCL_CUDA_CHECK(cudaDeviceSynchronize());
    }
  }
  if (has("wire") && have_peer) {
    std::printf("\n## wire  (NVLink counters of the reader GPU around %d launches)\n", c.wire_launches);
    double rx0, tx0, rx1, tx1;
    bool ok = c.counters && read_nvlink_kib(c.reader, &rx0, &tx0);
    double idle_rx = 0, idle_tx = 0;
    if (ok) {
      const double t0 = now_ms();
      while (now_ms() - t0 < c.idle_ms) {}
      ok = read_nvlink_kib(c.reader, &rx1, &tx1);
      idle_rx = (rx1 - rx0) * 1024.0 / (c.idle_ms / 1000.0);
      idle_tx = (tx1 - tx0) * 1024.0 / (c.idle_ms / 1000.0);
    }
    if (!ok) std::printf("NVLink counters unavailable (nvidia-smi nvlink -gt d gave nothing): reporting bandwidth only\n");
    std::printf("%12s %10s %12s %14s %12s %12s\n", "bytes", "ms", "GB/s", "asked_bytes", "rx/asked", "tx/asked");
    for (size_t s : c.wire_sizes) {
      size_t logical = 0, asked = 0; unsigned long long iters = 0;
      if (ok) read_nvlink_kib(c.reader, &rx0, &tx0);
      const double w0 = now_ms();
      double ms = 0;
      for (int l = 0; l < c.wire_launches; ++l) { ms += time_op(x, b.peer, s, c.wire_total / c.wire_launches, &logical, &iters); asked += logical; }
      const double wall = (now_ms() - w0) / 1000.0;
      double rxo = 0, txo = 0, rxb = 0, txb = 0;
      if (ok && read_nvlink_kib(c.reader, &rx1, &tx1)) {
        rxb = (rx1 - rx0) * 1024.0 - idle_rx * wall;
        txb = (tx1 - tx0) * 1024.0 - idle_tx * wall;
        rxo = rxb / asked; txo = txb / asked;
      }
      std::printf("%12zu %10.2f %12.1f %14zu %12.3f %12.3f\n", s, ms, asked / ms / 1e6, asked, rxo, txo);
      csv_wire.row("%s,peer,%zu,%d,%llu,%zu,%.3f,%.2f,%.0f,%.0f,%.4f,%.4f,%.0f,%.0f,%d,%s,%s,%zu", c.cache.c_str(), s, c.wire_launches, iters, asked, ms,
                   asked / ms / 1e6, rxb, txb, rxo, txo, idle_rx, idle_tx, ok ? 1 : 0, c.via.c_str(), c.dir.c_str(), c.tma_tile);
    }
  }
  int herr = 0;
  TCL_CUDA_CHECK(cudaMemcpy(&herr, b.err, 4, cudaMemcpyDeviceToHost));
  if (herr) { std::fprintf(stderr, "a bounded wait in a bulk mover ran out\n"); return 3; }
  return 0;
}
