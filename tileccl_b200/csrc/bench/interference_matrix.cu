// interference_matrix: (probe x mover) matrix of mutual slow-downs between a compute probe and a
// peer-to-peer transfer that run at the same time on different SMs of one GPU.
//   S_c = probe rate alone / probe rate while the mover runs      (compute slow-down)
//   S_m = mover bandwidth alone / mover bandwidth under the probe (communication slow-down)
// Probes: tcgen05, mma (legacy mma.sync), ffma, hbm, l2, smem.  Movers: ce, tma (bulk copies), reg.
// The probe runs on --probe-dev (the source or the destination GPU of the transfer) on all SMs but
// --comm-sms, which are left to the mover (--probe-sms sets the probe's CTA count directly).  --hbm-buf sizes
// the hbm probe's buffer.  The mover's bandwidth alone is measured once per mover and reused for every probe
// unless --no-alone-cache asks for a fresh figure beside each pair.  --mode starve fills every SM with a
// squatter kernel and shows what each mover does when it gets no SM (the squatter leaves after --starve-ms,
// one second by default, at the latest).  --mode once launches every probe once, alone, for --window-ms: the
// form a profiler can capture.
//
// Reference parity: tests/interference_matrix.cu (movers :174-254, probes :282-377, probe context
// :558-670, matrix :846-946, starve :950-1029, CSV header :839-841).
#include <string>
#include <thread>
#include <vector>

#include "../common/host_common.hpp"
#include "movers.cuh"
#include "probes.cuh"

using namespace tcl::host;
using namespace tcl::bench;

struct ProbeCtx {
  int dev = 0, sms = 0;
  volatile int* stop_h = nullptr;
  int* stop_d = nullptr;
  unsigned long long* cnt_h = nullptr;
  unsigned long long* cnt_d = nullptr;
  uint4* buf = nullptr;
  size_t buf_bytes = 0;
  float* sink = nullptr;
  int* err = nullptr;
  cudaStream_t st, snap;
  int blocks = 0, threads = 256;
  size_t buf_vec = 0;
  size_t pin_smem = 122880;

  void init(int device, size_t hbm_bytes) {
    dev = device;
    TCL_CUDA_CHECK(cudaSetDevice(dev));
    TCL_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    TCL_CUDA_CHECK(cudaHostAlloc(const_cast<int**>(&stop_h), 4, cudaHostAllocDefault));
    TCL_CUDA_CHECK(cudaMalloc(&stop_d, 4));
    // Counters live in device memory (a probe writing host memory every iteration would load
    // PCIe and slow the host's own submissions); the host snapshots them with an async copy on
    // its own stream while the probe runs.
    TCL_CUDA_CHECK(cudaHostAlloc(&cnt_h, 1024 * 8, cudaHostAllocDefault));
    TCL_CUDA_CHECK(cudaMalloc(&cnt_d, 1024 * 8));
    TCL_CUDA_CHECK(cudaStreamCreateWithFlags(&snap, cudaStreamNonBlocking));
    buf_bytes = hbm_bytes;
    TCL_CUDA_CHECK(cudaMalloc(&buf, buf_bytes));
    TCL_CUDA_CHECK(cudaMemset(buf, 1, buf_bytes));
    TCL_CUDA_CHECK(cudaMalloc(&sink, 64));
    TCL_CUDA_CHECK(cudaMalloc(&err, 4));
    TCL_CUDA_CHECK(cudaMemset(err, 0, 4));
    TCL_CUDA_CHECK(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking));
    // 120 KiB of dynamic shared memory per probe CTA: at most one probe CTA fits on an SM, so the
    // probe really leaves `comm_sms` SMs to the mover (the squatter of --mode starve passes 0).
    TCL_CUDA_CHECK(cudaFuncSetAttribute(probe_tc5_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 122880));
    TCL_CUDA_CHECK(cudaFuncSetAttribute(probe_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 122880));
    TCL_CUDA_CHECK(cudaFuncSetAttribute(probe_ffma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 122880));
    TCL_CUDA_CHECK(cudaFuncSetAttribute(probe_hbm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 122880));
    TCL_CUDA_CHECK(cudaFuncSetAttribute(probe_l2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 122880));
    TCL_CUDA_CHECK(cudaFuncSetAttribute(probe_smem_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 122880));
  }

  // Starts the probe; it ends when stop() is called or after max_ms at the latest.
  void launch(int kind, int nblocks, double max_ms, int l2_bytes) {
    TCL_CUDA_CHECK(cudaSetDevice(dev));
    blocks = std::min(nblocks, 1024);
    TCL_CUDA_CHECK(cudaMemsetAsync(stop_d, 0, 4, st));
    TCL_CUDA_CHECK(cudaMemsetAsync(cnt_d, 0, 1024 * 8, st));
    // The host clock cannot be compared with %globaltimer: pass a relative budget, which
    // launch_kernel turns into an absolute device-clock deadline.
    ProbeArgs a;
    a.stop = stop_d;
    a.counters = cnt_d;
    a.buf = buf;
    a.sink = sink;
    a.deadline_ns = static_cast<unsigned long long>(max_ms * 1e6);  // relative; made absolute on the device
    threads = 256;
    if (kind == kProbeHbm) buf_vec = buf_bytes / 16 / blocks;
    else if (kind == kProbeL2) buf_vec = static_cast<size_t>(l2_bytes) / 2 / 16;
    else buf_vec = 0;
    a.buf_vec = buf_vec;
    launch_kernel(kind, a);
  }
  void launch_kernel(int kind, ProbeArgs a);
  void stop() {
    *stop_h = 1;
    TCL_CUDA_CHECK(cudaSetDevice(dev));
    TCL_CUDA_CHECK(cudaMemcpyAsync(stop_d, const_cast<int*>(stop_h), 4, cudaMemcpyHostToDevice, snap));
    TCL_CUDA_CHECK(cudaStreamSynchronize(snap));
    TCL_CUDA_CHECK(cudaStreamSynchronize(st));
  }
  unsigned long long total() {
    int prev = 0;
    TCL_CUDA_CHECK(cudaGetDevice(&prev));
    TCL_CUDA_CHECK(cudaSetDevice(dev));
    TCL_CUDA_CHECK(cudaMemcpyAsync(cnt_h, cnt_d, blocks * 8, cudaMemcpyDeviceToHost, snap));
    TCL_CUDA_CHECK(cudaStreamSynchronize(snap));
    TCL_CUDA_CHECK(cudaSetDevice(prev));  // the caller may be driving the mover's device
    unsigned long long t = 0;
    for (int i = 0; i < blocks; ++i) t += cnt_h[i];
    return t;
  }
  // Probe rate over `ms` of wall clock, in probe_unit (1e9 units per second).
  double rate(int kind, double ms) {
    const unsigned long long c0 = total();
    const double t0 = now_ms();
    std::this_thread::sleep_for(std::chrono::microseconds(static_cast<long>(ms * 1000)));
    const unsigned long long c1 = total();
    const double dt = (now_ms() - t0) / 1000.0;
    return (c1 - c0) * probe_work_per_iter(kind, threads, buf_vec, blocks) / dt / 1e9;
  }
};

// The probes take a relative time budget and turn it into an absolute %globaltimer deadline here.
__global__ void arm_deadline_kernel(unsigned long long* out, unsigned long long budget_ns) { *out = tcl::ptx::globaltimer_ns() + budget_ns; }

void ProbeCtx::launch_kernel(int kind, ProbeArgs a) {
  unsigned long long* d;
  TCL_CUDA_CHECK(cudaMalloc(&d, 8));
  arm_deadline_kernel<<<1, 1, 0, st>>>(d, a.deadline_ns);
  unsigned long long h = 0;
  TCL_CUDA_CHECK(cudaMemcpyAsync(&h, d, 8, cudaMemcpyDeviceToHost, st));
  TCL_CUDA_CHECK(cudaStreamSynchronize(st));
  TCL_CUDA_CHECK(cudaFree(d));
  a.deadline_ns = h;
  switch (kind) {
    case kProbeTc5: probe_tc5_kernel<<<blocks, 32, pin_smem, st>>>(a, err); break;
    case kProbeMma: probe_mma_kernel<<<blocks, threads, pin_smem, st>>>(a); break;
    case kProbeFfma: probe_ffma_kernel<<<blocks, threads, pin_smem, st>>>(a); break;
    case kProbeHbm: probe_hbm_kernel<<<blocks, threads, pin_smem, st>>>(a); break;
    case kProbeL2: probe_l2_kernel<<<blocks, threads, pin_smem, st>>>(a); break;
    default: probe_smem_kernel<<<blocks, threads, pin_smem, st>>>(a); break;
  }
  TCL_CUDA_CHECK(cudaGetLastError());
  if (kind == kProbeTc5) threads = 32;
}

struct Mover {
  int src, dst, blocks;
  char *s, *d;
  size_t total, msg;
  int reg_threads = 1024, stages = 4;
  int* err;
  cudaStream_t st;
  cudaEvent_t e0, e1;
  void once(const std::string& m) {
    if (m == "ce") {
      const size_t chunk = std::max(msg, size_t(1) << 20);
      for (size_t off = 0; off < total; off += chunk)
        TCL_CUDA_CHECK(cudaMemcpyPeerAsync(d + off, dst, s + off, src, std::min(chunk, total - off), st));
    } else if (m == "reg") {
      reg_copy_kernel<<<blocks, reg_threads, 0, st>>>(reinterpret_cast<const uint4*>(s), reinterpret_cast<uint4*>(d), total / msg, msg / 16);
    } else {
      TCL_CUDA_CHECK(launch_bulk_pipe(stages, blocks, st, s, d, total, static_cast<uint32_t>(std::min<size_t>(msg, 32768)), kBulkCopy, err, 3000000000ull));
    }
  }
  // GB/s over `iters` back-to-back transfers.
  double gbps(const std::string& m, int iters) {
    TCL_CUDA_CHECK(cudaSetDevice(src));
    once(m);
    TCL_CUDA_CHECK(cudaStreamSynchronize(st));
    TCL_CUDA_CHECK(cudaEventRecord(e0, st));
    for (int i = 0; i < iters; ++i) once(m);
    TCL_CUDA_CHECK(cudaEventRecord(e1, st));
    TCL_CUDA_CHECK(cudaStreamSynchronize(st));
    return static_cast<double>(total) * iters / elapsed_us(e0, e1) / 1e3;
  }
};

int main(int argc, char** argv) {
  std::string mode = "matrix", probe_dev = "src", csv_path;
  std::vector<std::string> probes = {"tcgen05", "mma", "ffma", "hbm", "l2", "smem"}, comms = {"ce", "tma", "reg"};
  int src = 0, dst = 1, comm_sms = 16, probe_sms = 0, iters = 20, window_ms = 200, reg_threads = 1024, stages = 4;
  double starve_ms = 1000.0;
  bool alone_cache = true;
  size_t total = size_t(256) << 20, msg = 16384, hbm_bytes = size_t(256) << 20;
  Args a(argc, argv);
  while (a.more()) {
    std::string f = a.flag(), v;
    auto need = [&]() { if (!a.value(&v)) std::exit(1); return v; };
    if (f == "--mode") mode = need();
    else if (f == "--probes") probes = split_csv(need());
    else if (f == "--comm" || f == "--comms") comms = split_csv(need());
    else if (f == "--probe-sms") probe_sms = std::atoi(need().c_str());
    else if (f == "--hbm-buf") parse_bytes(need(), &hbm_bytes);
    else if (f == "--starve-ms") starve_ms = std::atof(need().c_str());
    else if (f == "--no-alone-cache") alone_cache = false;
    else if (f == "--reg-threads") reg_threads = std::atoi(need().c_str());
    else if (f == "--stages") stages = std::atoi(need().c_str());
    else if (f == "--probe-dev") probe_dev = need();
    else if (f == "--comm-sms") comm_sms = std::atoi(need().c_str());
    else if (f == "--msg") parse_bytes(need(), &msg);
    else if (f == "--total") parse_bytes(need(), &total);
    else if (f == "--iters") iters = std::atoi(need().c_str());
    else if (f == "--window-ms") window_ms = std::atoi(need().c_str());
    else if (f == "--src") src = std::atoi(need().c_str());
    else if (f == "--dst") dst = std::atoi(need().c_str());
    else if (f == "--csv") csv_path = need();
    else {
      std::printf("usage: %s [--mode matrix|starve|once] [--probes LIST] [--comms ce,tma,reg] [--probe-dev src|dst] [--comm-sms N] [--probe-sms N]\n"
                  "          [--msg B] [--total B] [--hbm-buf B] [--iters N] [--window-ms N] [--starve-ms MS] [--no-alone-cache] [--reg-threads N]\n"
                  "          [--stages 3|4|6|8] [--src N] [--dst N] [--csv FILE]\n", argv[0]);
      return f == "-h" || f == "--help" ? 0 : 1;
    }
  }
  if (reg_threads < 32 || reg_threads > 1024 || reg_threads % 32) { std::fprintf(stderr, "--reg-threads must be a multiple of 32 in [32, 1024]\n"); return 1; }
  if (stages != 3 && stages != 4 && stages != 6 && stages != 8) { std::fprintf(stderr, "--stages must be 3, 4, 6 or 8\n"); return 1; }
  if (starve_ms <= 0 || starve_ms > 5000) { std::fprintf(stderr, "--starve-ms must lie in (0, 5000]\n"); return 1; }
  if (hbm_bytes < (size_t(1) << 20)) { std::fprintf(stderr, "--hbm-buf must be at least 1 MiB\n"); return 1; }
  const int ndev = device_count();
  if (src >= ndev || dst >= ndev) { std::fprintf(stderr, "need GPUs %d and %d, have %d\n", src, dst, ndev); return 1; }
  if (src != dst && !enable_peer_all(std::max(src, dst) + 1)) return 1;
  total = total / msg * msg;
  Mover mv;
  mv.src = src; mv.dst = dst; mv.total = total; mv.msg = msg; mv.blocks = comm_sms; mv.reg_threads = reg_threads; mv.stages = stages;
  TCL_CUDA_CHECK(cudaSetDevice(dst));
  TCL_CUDA_CHECK(cudaMalloc(&mv.d, total));
  TCL_CUDA_CHECK(cudaSetDevice(src));
  TCL_CUDA_CHECK(cudaMalloc(&mv.s, total));
  TCL_CUDA_CHECK(cudaMalloc(&mv.err, 4));
  TCL_CUDA_CHECK(cudaMemset(mv.err, 0, 4));
  TCL_CUDA_CHECK(cudaStreamCreateWithFlags(&mv.st, cudaStreamNonBlocking));
  TCL_CUDA_CHECK(cudaEventCreate(&mv.e0));
  TCL_CUDA_CHECK(cudaEventCreate(&mv.e1));
  fill_pattern_kernel<<<1024, 256>>>(reinterpret_cast<uint32_t*>(mv.s), total / 4, 5u);
  TCL_CUDA_CHECK(cudaDeviceSynchronize());
  ProbeCtx pc;
  const int pdev = probe_dev == "dst" ? dst : src;
  pc.init(pdev, hbm_bytes);
  int l2 = 0;
  TCL_CUDA_CHECK(cudaDeviceGetAttribute(&l2, cudaDevAttrL2CacheSize, pdev));
  print_device_line(pdev);
  Csv csv;
  if (!csv.open(csv_path, "mode,probe,comm,probe_dev,probe_sms,comm_sms,msg_bytes,comm_alone_gbps,comm_ovl_gbps,S_m,probe_alone,probe_ovl,unit,S_c")) return 1;
  auto kind_of = [&](const std::string& p) { for (int k = 0; k < kProbeCount; ++k) if (p == probe_name(k)) return k; return -1; };

  if (mode == "once") {
    // For a profiler: every probe is launched once, alone, for --window-ms, and ends on its own deadline; nothing is
    // measured and the host does not touch the kernel while it runs.
    const int nb = probe_sms > 0 ? std::min(probe_sms, pc.sms) : pc.sms;
    for (auto& p : probes) {
      const int k = kind_of(p);
      if (k < 0) { std::fprintf(stderr, "unknown probe %s\n", p.c_str()); return 1; }
      pc.launch(k, nb, static_cast<double>(window_ms), l2);
      TCL_CUDA_CHECK(cudaStreamSynchronize(pc.st));
      std::printf("once: %s probe, %d CTAs, %d ms\n", p.c_str(), nb, window_ms);
    }
    return 0;
  }
  if (mode == "starve") {
    // Squatter: as many FFMA CTAs as the GPU can hold, for at most one second.
    int per_sm = 0;
    TCL_CUDA_CHECK(cudaSetDevice(pdev));
    TCL_CUDA_CHECK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, probe_ffma_kernel, 256, 0));
    std::printf("# starve: %d squatter CTAs on GPU %d, deadline %.0f ms\n%-6s %14s %14s\n", per_sm * pc.sms, pdev, starve_ms, "mover", "alone_us", "starved_us");
    for (auto& m : comms) {
      const double alone = static_cast<double>(total) / mv.gbps(m, 3) / 1e3;
      pc.pin_smem = 0;
      pc.launch(kProbeFfma, std::min(1024, per_sm * pc.sms), starve_ms, l2);
      pc.rate(kProbeFfma, 20);
      TCL_CUDA_CHECK(cudaSetDevice(src));
      TCL_CUDA_CHECK(cudaEventRecord(mv.e0, mv.st));
      mv.once(m);
      TCL_CUDA_CHECK(cudaEventRecord(mv.e1, mv.st));
      TCL_CUDA_CHECK(cudaStreamSynchronize(mv.st));   // returns when the squatter's deadline frees the SMs at the latest
      const double starved = elapsed_us(mv.e0, mv.e1);
      pc.stop();
      std::printf("%-6s %14.1f %14.1f\n", m.c_str(), alone, starved);
      csv.row("starve,ffma,%s,%s,%d,%d,%zu,%.2f,%.2f,%.3f,0,0,us,0", m.c_str(), probe_dev.c_str(), pc.sms, comm_sms, msg, alone, starved, starved / alone);
    }
    return 0;
  }

  const int probe_blocks = probe_sms > 0 ? std::min(probe_sms, pc.sms) : pc.sms - (pdev == src ? comm_sms : 0);
  std::vector<double> alone_cached(comms.size(), -1.0);
  std::printf("# interference matrix: probe on %s GPU (%d CTAs), mover on %d SMs of GPU %d, msg %zu B, window %d ms\n", probe_dev.c_str(), probe_blocks,
              comm_sms, src, msg, window_ms);
  std::printf("%-8s %-5s | %12s %12s %6s | %12s %12s %-8s %6s\n", "probe", "comm", "comm_alone", "comm_ovl", "S_m", "probe_alone", "probe_ovl", "unit", "S_c");
  for (auto& p : probes) {
    const int k = kind_of(p);
    if (k < 0) { std::fprintf(stderr, "unknown probe %s\n", p.c_str()); return 1; }
    pc.launch(k, probe_blocks, 20000.0, l2);
    pc.rate(k, 30);
    const double alone = pc.rate(k, window_ms);
    pc.stop();
    if (alone <= 0) { std::printf("%-8s [!] probe made NO progress\n", p.c_str()); continue; }
    for (size_t mi = 0; mi < comms.size(); ++mi) {
      const std::string& m = comms[mi];
      if (!alone_cache || alone_cached[mi] < 0) alone_cached[mi] = mv.gbps(m, iters);
      const double comm_alone = alone_cached[mi];
      pc.launch(k, probe_blocks, 20000.0, l2);
      pc.rate(k, 30);
      // Mover and probe together: the host thread measures the probe while the mover runs.
      double probe_ovl = 0;
      TCL_CUDA_CHECK(cudaSetDevice(src));
      TCL_CUDA_CHECK(cudaEventRecord(mv.e0, mv.st));
      int n = 0;
      const double t0 = now_ms();
      const unsigned long long c0 = pc.total();
      while (now_ms() - t0 < window_ms) { mv.once(m); ++n; TCL_CUDA_CHECK(cudaStreamSynchronize(mv.st)); }
      const unsigned long long c1 = pc.total();
      const double dt = (now_ms() - t0) / 1000.0;
      TCL_CUDA_CHECK(cudaEventRecord(mv.e1, mv.st));
      TCL_CUDA_CHECK(cudaStreamSynchronize(mv.st));
      probe_ovl = (c1 - c0) * probe_work_per_iter(k, pc.threads, pc.buf_vec, pc.blocks) / dt / 1e9;
      const double comm_ovl = static_cast<double>(total) * n / (dt * 1e9);
      pc.stop();
      const double sm = comm_ovl > 0 ? comm_alone / comm_ovl : 0, sc = probe_ovl > 0 ? alone / probe_ovl : 0;
      std::printf("%-8s %-5s | %12.1f %12.1f %6.2f | %12.2f %12.2f %-8s %6.2f\n", p.c_str(), m.c_str(), comm_alone, comm_ovl, sm, alone, probe_ovl, probe_unit(k), sc);
      csv.row("matrix,%s,%s,%s,%d,%d,%zu,%.2f,%.2f,%.3f,%.3f,%.3f,%s,%.3f", p.c_str(), m.c_str(), probe_dev.c_str(), probe_blocks, comm_sms, msg, comm_alone, comm_ovl, sm,
              alone, probe_ovl, probe_unit(k), sc);
    }
  }
  int herr = 0;
  TCL_CUDA_CHECK(cudaSetDevice(pdev));
  TCL_CUDA_CHECK(cudaMemcpy(&herr, pc.err, 4, cudaMemcpyDeviceToHost));
  if (herr) { std::fprintf(stderr, "the tcgen05 probe's bounded wait ran out\n"); return 3; }
  return 0;
}
