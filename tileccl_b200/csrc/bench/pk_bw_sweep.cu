// pk_bw_sweep: peer-to-peer push bandwidth of three movers
//   ce   copy engine, one cudaMemcpyPeerAsync per message
//   tma  bulk copies through shared memory (cp.async.bulk), multi-stage ring
//   reg  16-byte ld/st through registers
//   reg256  32-byte ld/st through registers (ld/st.global.v8.b32; not in the default list: --methods ce,tma,reg,reg256)
// (a) against message size at full SM count, (b) against the number of SMs at
// a fixed message size.  The destination is verified on the device.
//
// Reference parity: tests/pk_bw_sweep.cu (flags :375-394, planner :485-530,
// Fig.2 loop :746-778, Fig.3 loop :782-829).  The reference prints tables only;
// --csv is added here (columns: figure,mover,msg_bytes,sms,total_bytes,us,gbps,verify).
#include <string>
#include <vector>

#include "../common/host_common.hpp"
#include "movers.cuh"

using namespace tcl::host;
using namespace tcl::bench;

struct Config {
  std::string mode = "both";
  size_t total = size_t(1) << 30;
  std::vector<size_t> sizes;
  std::vector<int> sms;
  std::vector<std::string> methods = {"ce", "tma", "reg"};
  int blocks = 0;
  size_t msg_tma = 0, msg_reg = 16384;
  int stages = 4, reg_threads = 1024, iters = 10, warmup = 3;
  size_t max_ce_msgs = 16384;
  int src = 0, dst = 1;
  bool check = true;
  std::string csv;
};

static void usage(const char* p) {
  std::printf(
      "usage: %s [--mode size|sms|both] [--total BYTES] [--sizes LIST] [--sms LIST] [--methods ce,tma,reg,reg256]\n"
      "          [--blocks N] [--msg-tma BYTES] [--msg-reg BYTES] [--stages 3|4|6|8] [--reg-threads N]\n"
      "          [--iters N] [--warmup N] [--max-ce-msgs N] [--src N] [--dst N] [--no-check] [--csv FILE]\n"
      "  --src and --dst may be the same GPU (loop-back: measures the movers against local memory)\n", p);
}

struct Ctx {
  Config c;
  char *s = nullptr, *d = nullptr;
  int* err = nullptr;
  unsigned long long* mism = nullptr;
  cudaStream_t st;
  cudaEvent_t e0, e1;
  int sm_count = 0;
  size_t smem_max = 0;
};

static bool verify(Ctx& x, size_t bytes, uint32_t seed) {
  TCL_CUDA_CHECK(cudaSetDevice(x.c.dst));
  unsigned long long* m;
  TCL_CUDA_CHECK(cudaMalloc(&m, 8));
  TCL_CUDA_CHECK(cudaMemset(m, 0, 8));
  verify_pattern_kernel<<<1024, 256>>>(reinterpret_cast<uint32_t*>(x.d), bytes / 4, seed, m);
  unsigned long long h = 0;
  TCL_CUDA_CHECK(cudaMemcpy(&h, m, 8, cudaMemcpyDeviceToHost));
  TCL_CUDA_CHECK(cudaFree(m));
  TCL_CUDA_CHECK(cudaSetDevice(x.c.src));
  return h == 0;
}

// One measurement: returns average microseconds per iteration, or < 0 on error.
static double run_point(Ctx& x, const std::string& method, size_t msg, size_t total, int blocks, bool* ok) {
  const Config& c = x.c;
  total = total / msg * msg;
  if (total == 0) { total = msg; }
  size_t n_msgs = total / msg;
  if (method == "ce" && n_msgs > c.max_ce_msgs) { n_msgs = c.max_ce_msgs; total = n_msgs * msg; }
  TCL_CUDA_CHECK(cudaSetDevice(c.dst));
  TCL_CUDA_CHECK(cudaMemset(x.d, 0, total));
  TCL_CUDA_CHECK(cudaDeviceSynchronize());
  TCL_CUDA_CHECK(cudaSetDevice(c.src));
  TCL_CUDA_CHECK(cudaMemset(x.err, 0, 4));
  auto once = [&]() {
    if (method == "ce") {
      for (size_t m = 0; m < n_msgs; ++m)
        TCL_CUDA_CHECK(cudaMemcpyPeerAsync(x.d + m * msg, c.dst, x.s + m * msg, c.src, msg, x.st));
    } else if (method == "reg") {
      reg_copy_kernel<<<blocks, c.reg_threads, 0, x.st>>>(reinterpret_cast<const uint4*>(x.s), reinterpret_cast<uint4*>(x.d),
                                                            n_msgs, msg / 16);
    } else if (method == "reg256") {
      reg256_copy_kernel<<<blocks, c.reg_threads, 0, x.st>>>(reinterpret_cast<const tcl::ptx::Vec8*>(x.s), reinterpret_cast<tcl::ptx::Vec8*>(x.d),
                                                               n_msgs, msg / 32);
    } else {
      // A message larger than a slot is moved as several tiles.
      const size_t budget = (x.smem_max - 8 * c.stages) / c.stages / 128 * 128;
      const uint32_t tile = static_cast<uint32_t>(msg < budget ? msg : budget);
      TCL_CUDA_CHECK(launch_bulk_pipe(c.stages, blocks, x.st, x.s, x.d, total, tile, kBulkCopy, x.err, 2000000000ull));
    }
  };
  for (int i = 0; i < c.warmup; ++i) once();
  TCL_CUDA_CHECK(cudaStreamSynchronize(x.st));
  TCL_CUDA_CHECK(cudaEventRecord(x.e0, x.st));
  for (int i = 0; i < c.iters; ++i) once();
  TCL_CUDA_CHECK(cudaEventRecord(x.e1, x.st));
  TCL_CUDA_CHECK(cudaStreamSynchronize(x.st));
  int herr = 0;
  TCL_CUDA_CHECK(cudaMemcpy(&herr, x.err, 4, cudaMemcpyDeviceToHost));
  *ok = herr == 0;
  if (c.check && *ok) *ok = verify(x, total, 0x1234u);
  return elapsed_us(x.e0, x.e1) / c.iters * (herr ? -1.0 : 1.0);
}

int main(int argc, char** argv) {
  Config c;
  Args a(argc, argv);
  while (a.more()) {
    std::string f = a.flag(), v;
    auto need = [&]() { if (!a.value(&v)) { usage(argv[0]); std::exit(1); } return v; };
    if (f == "--mode") c.mode = need();
    else if (f == "--total") { if (!parse_bytes(need(), &c.total)) { usage(argv[0]); return 1; } }
    else if (f == "--sizes") { if (!parse_size_list(need(), &c.sizes)) { usage(argv[0]); return 1; } }
    else if (f == "--sms") parse_int_list(need(), &c.sms);
    else if (f == "--methods") c.methods = split_csv(need());
    else if (f == "--blocks") c.blocks = std::atoi(need().c_str());
    else if (f == "--msg-tma") parse_bytes(need(), &c.msg_tma);
    else if (f == "--msg-reg") parse_bytes(need(), &c.msg_reg);
    else if (f == "--stages") c.stages = std::atoi(need().c_str());
    else if (f == "--reg-threads") c.reg_threads = std::atoi(need().c_str());
    else if (f == "--iters") c.iters = std::atoi(need().c_str());
    else if (f == "--warmup") c.warmup = std::atoi(need().c_str());
    else if (f == "--max-ce-msgs") c.max_ce_msgs = std::strtoull(need().c_str(), nullptr, 10);
    else if (f == "--src") c.src = std::atoi(need().c_str());
    else if (f == "--dst") c.dst = std::atoi(need().c_str());
    else if (f == "--no-check") c.check = false;
    else if (f == "--csv") c.csv = need();
    else { usage(argv[0]); return f == "-h" || f == "--help" ? 0 : 1; }
  }
  if (c.stages != 3 && c.stages != 4 && c.stages != 6 && c.stages != 8) c.stages = 4;
  if (c.sizes.empty()) parse_size_list("128,512,2K,8K,32K,64K,128K,512K,2M,8M,32M,128M,512M,1G", &c.sizes);
  const int ndev = device_count();
  if (c.src >= ndev || c.dst >= ndev) { std::fprintf(stderr, "need GPUs %d and %d, have %d\n", c.src, c.dst, ndev); return 1; }
  if (c.src != c.dst && !enable_peer_all(std::max(c.src, c.dst) + 1)) return 1;

  Ctx x;
  x.c = c;
  TCL_CUDA_CHECK(cudaSetDevice(c.dst));
  TCL_CUDA_CHECK(cudaMalloc(&x.d, c.total));
  TCL_CUDA_CHECK(cudaSetDevice(c.src));
  TCL_CUDA_CHECK(cudaMalloc(&x.s, c.total));
  TCL_CUDA_CHECK(cudaMalloc(&x.err, 4));
  TCL_CUDA_CHECK(cudaStreamCreateWithFlags(&x.st, cudaStreamNonBlocking));
  TCL_CUDA_CHECK(cudaEventCreate(&x.e0));
  TCL_CUDA_CHECK(cudaEventCreate(&x.e1));
  cudaDeviceProp prop;
  TCL_CUDA_CHECK(cudaGetDeviceProperties(&prop, c.src));
  x.sm_count = prop.multiProcessorCount;
  x.smem_max = prop.sharedMemPerBlockOptin;
  fill_pattern_kernel<<<1024, 256>>>(reinterpret_cast<uint32_t*>(x.s), c.total / 4, 0x1234u);
  TCL_CUDA_CHECK(cudaDeviceSynchronize());
  print_device_line(c.src);
  std::printf("# pk_bw_sweep src=%d dst=%d total=%zu iters=%d stages=%d%s\n", c.src, c.dst, c.total, c.iters, c.stages,
              c.src == c.dst ? " (loop-back)" : "");
  Csv csv;
  if (!csv.open(c.csv, "figure,mover,msg_bytes,sms,total_bytes,us,gbps,verify")) return 1;
  const int full_blocks = c.blocks > 0 ? c.blocks : x.sm_count;

  if (c.mode == "size" || c.mode == "both") {
    std::printf("\n## bandwidth vs message size (%d CTAs)\n%12s", full_blocks, "msg_bytes");
    for (auto& m : c.methods) std::printf(" %10s GB/s", m.c_str());
    std::printf("\n");
    for (size_t msg : c.sizes) {
      if (msg > c.total || msg % 16) continue;
      std::printf("%12zu", msg);
      for (auto& m : c.methods) {
        bool ok = true;
        size_t total = c.total;
        if (m == "reg256" && msg % 32) { std::printf(" %14s ", "-"); continue; }
        if (m == "ce" && total / msg > c.max_ce_msgs) total = c.max_ce_msgs * msg;
        const double us = run_point(x, m, msg, total, full_blocks, &ok);
        const double gbps = us > 0 ? (total / msg * msg) / us / 1e3 : 0.0;
        std::printf(" %14.1f%s", gbps, ok ? " " : "!");
        csv.row("size,%s,%zu,%d,%zu,%.2f,%.2f,%s", m.c_str(), msg, full_blocks, total, us, gbps, ok ? "ok" : "FAIL");
      }
      std::printf("\n");
    }
  }
  if (c.mode == "sms" || c.mode == "both") {
    std::vector<int> sms = c.sms;
    if (sms.empty()) for (int s : {1, 2, 4, 8, 12, 16, 24, 32, 48, 64, 96, 128, x.sm_count}) if (s <= x.sm_count) sms.push_back(s);
    const size_t msg_tma = c.msg_tma ? c.msg_tma : 32768;
    std::printf("\n## bandwidth vs SM count (tma msg %zu B, reg msg %zu B)\n%6s", msg_tma, c.msg_reg, "sms");
    for (auto& m : c.methods) if (m != "ce") std::printf(" %10s GB/s", m.c_str());
    std::printf("\n");
    for (int s : sms) {
      std::printf("%6d", s);
      for (auto& m : c.methods) {
        if (m == "ce") continue;
        bool ok = true;
        const size_t msg = m == "tma" ? msg_tma : c.msg_reg;
        const double us = run_point(x, m, msg, c.total, s, &ok);
        const double gbps = us > 0 ? (c.total / msg * msg) / us / 1e3 : 0.0;
        std::printf(" %14.1f%s", gbps, ok ? " " : "!");
        csv.row("sms,%s,%zu,%d,%zu,%.2f,%.2f,%s", m.c_str(), msg, s, c.total, us, gbps, ok ? "ok" : "FAIL");
      }
      std::printf("\n");
    }
  }
  TCL_CUDA_CHECK(cudaFree(x.s));
  TCL_CUDA_CHECK(cudaFree(x.err));
  TCL_CUDA_CHECK(cudaSetDevice(c.dst));
  TCL_CUDA_CHECK(cudaFree(x.d));
  return 0;
}
