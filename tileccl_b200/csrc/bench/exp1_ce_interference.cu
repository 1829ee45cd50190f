// exp1: does copy-engine traffic that has nothing to do with a GEMM slow that GEMM down?
// The library's tcgen05 GEMM runs on --gemm-dev while copy-engine "legs" move unrelated buffers:
//   pull         every other GPU -> the GEMM GPU         push       the GEMM GPU -> every other GPU
//   allgather    every GPU -> every other GPU            bystander  only between GPUs that are not the GEMM GPU
//   engine-only  host -> GEMM GPU (no NVLink)            local      device-to-device copy inside the GEMM GPU
// A host "pump" keeps a ring of bursts queued on every leg and re-enqueues a burst as soon as its
// event completes; a leg found idle is counted as a gap.  Every pattern is preceded by its own
// GEMM-alone baseline (paired), and the baseline is re-checked at the end for drift.
//   S_c = GEMM time under traffic / GEMM time alone
//
// Reference parity: comm_comp/exp1_ce_interference.cu (legs :127-255, pump :270-320, calibrate
// :330-370, loop :500-615, CSV :492-494).
#include <string>
#include <vector>

#include "../common/host_common.hpp"
#include "../ops/tileccl_ops.h"

using namespace tcl::host;

struct Leg {
  int src_dev, dst_dev;        // -1 = host
  char *src, *dst;
  cudaStream_t st;
  std::vector<cudaEvent_t> ring;
  size_t head = 0;
};

struct Pump {
  std::vector<Leg>* legs;
  size_t msg;
  int per_burst;
  long gaps = 0;
  unsigned long long bytes = 0;
  void enqueue(Leg& l, cudaEvent_t ev) {
    for (int i = 0; i < per_burst; ++i) {
      if (l.src_dev < 0 || l.dst_dev < 0 || l.src_dev == l.dst_dev) TCL_CUDA_CHECK(cudaMemcpyAsync(l.dst, l.src, msg, cudaMemcpyDefault, l.st));
      else TCL_CUDA_CHECK(cudaMemcpyPeerAsync(l.dst, l.dst_dev, l.src, l.src_dev, msg, l.st));
    }
    TCL_CUDA_CHECK(cudaEventRecord(ev, l.st));
    bytes += msg * per_burst;
  }
  void start() { for (auto& l : *legs) { l.head = 0; for (auto ev : l.ring) enqueue(l, ev); } }
  void poll() {
    for (auto& l : *legs) {
      if (cudaStreamQuery(l.st) == cudaSuccess) ++gaps; else cudaGetLastError();
      while (cudaEventQuery(l.ring[l.head]) == cudaSuccess) {
        enqueue(l, l.ring[l.head]);
        l.head = (l.head + 1) % l.ring.size();
      }
      cudaGetLastError();
    }
  }
  void drain() { for (auto& l : *legs) TCL_CUDA_CHECK(cudaStreamSynchronize(l.st)); }
};

struct GemmRunner {
  void* plan = nullptr;
  void *A, *B, *D;
  int* status;
  cudaStream_t st;
  cudaEvent_t e0, e1;
  int dev, epoch = 0;
  Shape3 sh;
  bool init(int device, Shape3 s, int cta_group) {
    dev = device; sh = s;
    TCL_CUDA_CHECK(cudaSetDevice(dev));
    TCL_CUDA_CHECK(cudaMalloc(&A, size_t(2) * s.m * s.k));
    TCL_CUDA_CHECK(cudaMalloc(&B, size_t(2) * s.n * s.k));
    TCL_CUDA_CHECK(cudaMalloc(&D, size_t(2) * s.m * s.n));
    TCL_CUDA_CHECK(cudaMalloc(&status, 16));
    TCL_CUDA_CHECK(cudaMemset(status, 0, 16));
    TCL_CUDA_CHECK(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking));
    TCL_CUDA_CHECK(cudaEventCreate(&e0));
    TCL_CUDA_CHECK(cudaEventCreate(&e1));
    tcl_fill_normal_bf16(A, int64_t(s.m) * s.k, 1, 0.f, 1.f, st);
    tcl_fill_normal_bf16(B, int64_t(s.n) * s.k, 2, 0.f, 1.f, st);
    tcl_gemm_desc d;
    std::memset(&d, 0, sizeof(d));
    d.mode = TCL_MODE_PLAIN; d.cta_group = cta_group;
    d.M = s.m; d.N = s.n; d.K = s.k; d.lda = s.k; d.ldb = s.k; d.ldc = s.n;
    d.A = A; d.B = B; d.world = 1; d.rank = 0; d.seg_rows = s.m; d.dst_base[0] = D; d.status = status;
    char err[256];
    plan = tcl_gemm_plan_create(&d, err, sizeof(err));
    if (!plan) { std::fprintf(stderr, "GEMM plan rejected: %s\n", err); return false; }
    return true;
  }
  // Times `iters` GEMMs one by one; `tick` runs on the host while each is in flight.
  template <class F>
  Stats timed(int warm, int iters, F tick) {
    TCL_CUDA_CHECK(cudaSetDevice(dev));
    std::vector<double> us;
    for (int i = 0; i < warm + iters; ++i) {
      TCL_CUDA_CHECK(cudaEventRecord(e0, st));
      if (tcl_gemm_plan_run(plan, ++epoch, st) != 0) { std::fprintf(stderr, "GEMM launch failed\n"); std::exit(2); }
      TCL_CUDA_CHECK(cudaEventRecord(e1, st));
      while (cudaEventQuery(e1) == cudaErrorNotReady) tick();
      cudaGetLastError();
      if (i >= warm) us.push_back(elapsed_us(e0, e1));
    }
    return make_stats(us);
  }
  void destroy() {
    tcl_gemm_plan_destroy(plan);
    TCL_CUDA_CHECK(cudaSetDevice(dev));
    cudaFree(A); cudaFree(B); cudaFree(D);
  }
};

int main(int argc, char** argv) {
  std::vector<std::string> shapes = {"2048", "4096", "8192"}, patterns = {"pull", "push", "allgather", "bystander", "engine-only", "local"};
  std::vector<size_t> msgs;
  int gemm_dev = 0, ndev = 0, iters = 30, warm = 3, cta_group = 2;
  std::string csv_path;
  Args a(argc, argv);
  while (a.more()) {
    std::string f = a.flag(), v;
    auto need = [&]() { if (!a.value(&v)) std::exit(1); return v; };
    if (f == "--sizes") shapes = split_csv(need());
    else if (f == "--patterns") patterns = split_csv(need());
    else if (f == "--msgs") parse_size_list(need(), &msgs);
    else if (f == "--gemm-dev") gemm_dev = std::atoi(need().c_str());
    else if (f == "--ndev") ndev = std::atoi(need().c_str());
    else if (f == "--iters") iters = std::atoi(need().c_str());
    else if (f == "--warmup") warm = std::atoi(need().c_str());
    else if (f == "--cta-group") cta_group = std::atoi(need().c_str());
    else if (f == "--csv") csv_path = need();
    else {
      std::printf("usage: %s [--sizes LIST] [--patterns pull,push,allgather,bystander,engine-only,local] [--msgs LIST] [--gemm-dev N] [--ndev N]\n"
                  "          [--iters N] [--warmup N] [--cta-group 1|2] [--csv FILE]\n", argv[0]);
      return f == "-h" || f == "--help" ? 0 : 1;
    }
  }
  if (msgs.empty()) parse_size_list("64M", &msgs);
  const int have = device_count();
  if (ndev <= 0 || ndev > have) ndev = have;
  if (gemm_dev >= ndev) { std::fprintf(stderr, "no GPU %d among %d\n", gemm_dev, ndev); return 1; }
  if (ndev > 1 && !enable_peer_all(ndev)) return 1;
  size_t max_msg = 0;
  for (size_t m : msgs) max_msg = std::max(max_msg, m);
  print_device_line(gemm_dev);
  std::printf("# exp1 CE interference: GEMM on GPU %d, %d GPUs, cta_group %d\n", gemm_dev, ndev, cta_group);
  // One send and one receive buffer per (device, peer) pair keeps the legs independent.
  std::vector<std::vector<char*>> sendb(ndev, std::vector<char*>(ndev + 1)), recvb(ndev, std::vector<char*>(ndev + 1));
  for (int d = 0; d < ndev; ++d) {
    TCL_CUDA_CHECK(cudaSetDevice(d));
    for (int p = 0; p <= ndev; ++p) { TCL_CUDA_CHECK(cudaMalloc(&sendb[d][p], max_msg)); TCL_CUDA_CHECK(cudaMalloc(&recvb[d][p], max_msg)); }
  }
  char* host;
  TCL_CUDA_CHECK(cudaHostAlloc(&host, max_msg, cudaHostAllocDefault));
  Csv csv;
  if (!csv.open(csv_path, "pattern,m,n,k,msg_bytes,legs,alone_us,ovl_us,alone_p95,ovl_p95,S_c,tflops_alone,tflops_ovl,comm_alone_gbps,comm_ovl_gbps,gaps")) return 1;
  std::printf("%-12s %-14s %10s %4s | %10s %10s %6s | %10s %10s | %s\n", "pattern", "shape", "msg", "legs", "alone_us", "ovl_us", "S_c", "comm_alone", "comm_ovl", "gaps");

  for (auto& ss : shapes) {
    Shape3 sh;
    if (!parse_shape(ss, &sh)) { std::fprintf(stderr, "bad shape %s\n", ss.c_str()); return 1; }
    GemmRunner g;
    if (!g.init(gemm_dev, sh, cta_group)) return 1;
    const double flop = 2.0 * sh.m * sh.n * sh.k;
    const Stats first = g.timed(warm, iters, [] {});
    for (auto& pat : patterns) {
      for (size_t msg : msgs) {
        std::vector<Leg> legs;
        auto add = [&](int s, int d) {
          Leg l;
          l.src_dev = s; l.dst_dev = d;
          const int owner = d >= 0 ? d : s;
          l.src = s < 0 ? host : sendb[s][d < 0 ? ndev : d];
          l.dst = d < 0 ? host : recvb[d][s < 0 ? ndev : s];
          TCL_CUDA_CHECK(cudaSetDevice(owner));
          TCL_CUDA_CHECK(cudaStreamCreateWithFlags(&l.st, cudaStreamNonBlocking));
          l.ring.resize(4);
          for (auto& e : l.ring) TCL_CUDA_CHECK(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
          legs.push_back(l);
        };
        if (pat == "pull") { for (int p = 0; p < ndev; ++p) if (p != gemm_dev) add(p, gemm_dev); }
        else if (pat == "push") { for (int p = 0; p < ndev; ++p) if (p != gemm_dev) add(gemm_dev, p); }
        else if (pat == "allgather") { for (int s = 0; s < ndev; ++s) for (int d = 0; d < ndev; ++d) if (s != d) add(s, d); }
        else if (pat == "bystander") { for (int s = 0; s < ndev; ++s) for (int d = 0; d < ndev; ++d) if (s != d && s != gemm_dev && d != gemm_dev) add(s, d); }
        else if (pat == "engine-only") add(-1, gemm_dev);
        else if (pat == "local") { Leg l; l.src_dev = l.dst_dev = gemm_dev; l.src = sendb[gemm_dev][ndev]; l.dst = recvb[gemm_dev][ndev];
          TCL_CUDA_CHECK(cudaSetDevice(gemm_dev)); TCL_CUDA_CHECK(cudaStreamCreateWithFlags(&l.st, cudaStreamNonBlocking)); l.ring.resize(4);
          for (auto& e : l.ring) TCL_CUDA_CHECK(cudaEventCreateWithFlags(&e, cudaEventDisableTiming)); legs.push_back(l); }
        if (legs.empty()) { std::printf("%-12s %-14s %10zu    0 | skipped: needs more GPUs\n", pat.c_str(), ss.c_str(), msg); continue; }
        Pump pump{&legs, msg, std::max<int>(1, static_cast<int>((size_t(256) << 20) / msg / 4))};
        // Transfer bandwidth alone.
        pump.bytes = 0;
        const double t0 = now_ms();
        pump.start();
        pump.drain();
        const double comm_alone = pump.bytes / ((now_ms() - t0) * 1e6);
        // Paired GEMM-alone baseline, then the overlapped run.
        const Stats alone = g.timed(warm, iters, [] {});
        pump.bytes = 0; pump.gaps = 0;
        pump.start();
        const double t1 = now_ms();
        const Stats ovl = g.timed(warm, iters, [&] { pump.poll(); });
        const double comm_ovl = pump.bytes / ((now_ms() - t1) * 1e6);
        pump.drain();
        const double sc = alone.mean > 0 ? ovl.mean / alone.mean : 0;
        std::printf("%-12s %-14s %10zu %4zu | %10.1f %10.1f %6.3f | %10.1f %10.1f | %ld\n", pat.c_str(), ss.c_str(), msg, legs.size(), alone.mean, ovl.mean, sc,
                    comm_alone, comm_ovl, pump.gaps);
        csv.row("%s,%d,%d,%d,%zu,%zu,%.2f,%.2f,%.2f,%.2f,%.4f,%.1f,%.1f,%.2f,%.2f,%ld", pat.c_str(), sh.m, sh.n, sh.k, msg, legs.size(), alone.mean, ovl.mean, alone.p95,
                ovl.p95, sc, flop / alone.mean / 1e6, flop / ovl.mean / 1e6, comm_alone, comm_ovl, pump.gaps);
        for (auto& l : legs) { cudaStreamDestroy(l.st); for (auto e : l.ring) cudaEventDestroy(e); }
      }
    }
    const Stats last = g.timed(warm, iters, [] {});
    const double drift = first.mean > 0 ? last.mean / first.mean : 0;
    std::printf("# baseline recheck %s: first %.1f us, last %.1f us, drift %.3f%s\n", ss.c_str(), first.mean, last.mean, drift, (drift > 1.05 || drift < 0.95) ? "  [!]" : "");
    int st[4];
    TCL_CUDA_CHECK(cudaSetDevice(gemm_dev));
    TCL_CUDA_CHECK(cudaMemcpy(st, g.status, 16, cudaMemcpyDeviceToHost));
    if (st[0]) { std::fprintf(stderr, "GEMM gave up: %s\n", tcl_status_string(st[0])); return 3; }
    g.destroy();
  }
  return 0;
}
