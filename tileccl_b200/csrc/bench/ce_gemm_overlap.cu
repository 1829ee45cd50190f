// ce_gemm_overlap: copy engine against a real library GEMM (cuBLAS), both directions of interference.
//   phase A  GEMM timed while a host "pump" keeps the copy engines saturated   -> S_c
//   phase B  a burst of copies timed while a pump keeps GEMMs queued            -> S_m
// Transfers: p2p push / pull / bidir between two GPUs, d2d on the GEMM's GPU, h2d, d2h (pinned).
// The GEMM is cublasGemmEx in bf16 / fp16 / tf32 / fp32.  cuBLAS here is the baseline library, not a
// product path.
//
// Reference parity: tests/ce_gemm_overlap.cu (Gemm :288-380, Comm :386-474, pumps :533-620, loop
// :741-834, CSV :719-722).
#include <cublas_v2.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <string>
#include <vector>

#include "../common/host_common.hpp"

using namespace tcl::host;

#define CUBLAS_CHECK(x) do { cublasStatus_t s__ = (x); if (s__ != CUBLAS_STATUS_SUCCESS) { std::fprintf(stderr, "cuBLAS error %d at %s:%d\n", (int)s__, __FILE__, __LINE__); std::exit(2);} } while (0)

struct Gemm {
  cublasHandle_t h;
  cudaStream_t st;
  void *A, *B, *C;
  int m, n, k;
  cudaDataType_t ab, c;
  cublasComputeType_t comp;
  cudaEvent_t e0, e1;
  void init(int dev, Shape3 s, const std::string& dtype) {
    TCL_CUDA_CHECK(cudaSetDevice(dev));
    m = s.m; n = s.n; k = s.k;
    size_t es = 2;
    if (dtype == "fp32") { ab = c = CUDA_R_32F; comp = CUBLAS_COMPUTE_32F; es = 4; }
    else if (dtype == "tf32") { ab = c = CUDA_R_32F; comp = CUBLAS_COMPUTE_32F_FAST_TF32; es = 4; }
    else if (dtype == "fp16") { ab = c = CUDA_R_16F; comp = CUBLAS_COMPUTE_32F; }
    else { ab = c = CUDA_R_16BF; comp = CUBLAS_COMPUTE_32F; }
    TCL_CUDA_CHECK(cudaMalloc(&A, es * m * k));
    TCL_CUDA_CHECK(cudaMalloc(&B, es * k * n));
    TCL_CUDA_CHECK(cudaMalloc(&C, es * m * n));
    TCL_CUDA_CHECK(cudaMemset(A, 0, es * m * k));
    TCL_CUDA_CHECK(cudaMemset(B, 0, es * k * n));
    TCL_CUDA_CHECK(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking));
    CUBLAS_CHECK(cublasCreate(&h));
    CUBLAS_CHECK(cublasSetStream(h, st));
    TCL_CUDA_CHECK(cudaEventCreate(&e0));
    TCL_CUDA_CHECK(cudaEventCreate(&e1));
  }
  void run() {
    const float alpha = 1.f, beta = 0.f;
    CUBLAS_CHECK(cublasGemmEx(h, CUBLAS_OP_N, CUBLAS_OP_N, m, n, k, &alpha, A, ab, m, B, ab, k, &beta, C, c, m, comp, CUBLAS_GEMM_DEFAULT));
  }
  Stats time(int iters) {
    std::vector<double> us;
    for (int i = 0; i < iters; ++i) {
      TCL_CUDA_CHECK(cudaEventRecord(e0, st));
      run();
      TCL_CUDA_CHECK(cudaEventRecord(e1, st));
      TCL_CUDA_CHECK(cudaEventSynchronize(e1));
      us.push_back(elapsed_us(e0, e1));
    }
    return make_stats(us);
  }
};

struct Leg { void* dst; int dst_dev; const void* src; int src_dev; cudaStream_t st; bool host; };

struct Comm {
  std::vector<Leg> legs;
  size_t msg = 0;
  void burst(int reps) {
    for (int r = 0; r < reps; ++r)
      for (auto& l : legs) {
        if (l.host) TCL_CUDA_CHECK(cudaMemcpyAsync(l.dst, l.src, msg, cudaMemcpyDefault, l.st));
        else TCL_CUDA_CHECK(cudaMemcpyPeerAsync(l.dst, l.dst_dev, l.src, l.src_dev, msg, l.st));
      }
  }
  void sync() { for (auto& l : legs) TCL_CUDA_CHECK(cudaStreamSynchronize(l.st)); }
  bool idle() { for (auto& l : legs) if (cudaStreamQuery(l.st) != cudaSuccess) { cudaGetLastError(); return false; } return true; }
  // GB/s of `reps` bursts, wall clock.
  double gbps(int reps) {
    sync();
    const double t0 = now_ms();
    burst(reps);
    sync();
    return static_cast<double>(msg) * legs.size() * reps / ((now_ms() - t0) * 1e6);
  }
};

int main(int argc, char** argv) {
  std::vector<std::string> shapes = {"4096", "8192"}, dtypes = {"bf16"}, comms = {"p2p_push", "p2p_pull", "p2p_bidir", "d2d", "h2d", "d2h"};
  std::vector<size_t> msgs;
  int gemm_dev = 0, peer = 1, iters = 20;
  std::string csv_path;
  Args a(argc, argv);
  while (a.more()) {
    std::string f = a.flag(), v;
    auto need = [&]() { if (!a.value(&v)) std::exit(1); return v; };
    if (f == "--sizes") shapes = split_csv(need());
    else if (f == "--dtypes") dtypes = split_csv(need());
    else if (f == "--comm") comms = split_csv(need());
    else if (f == "--msgs") parse_size_list(need(), &msgs);
    else if (f == "--gemm-dev") gemm_dev = std::atoi(need().c_str());
    else if (f == "--peer") peer = std::atoi(need().c_str());
    else if (f == "--iters") iters = std::atoi(need().c_str());
    else if (f == "--csv") csv_path = need();
    else {
      std::printf("usage: %s [--sizes LIST(N|MxNxK)] [--dtypes bf16,fp16,tf32,fp32] [--comm p2p_push,p2p_pull,p2p_bidir,d2d,h2d,d2h]\n"
                  "          [--msgs LIST] [--gemm-dev N] [--peer N] [--iters N] [--csv FILE]\n", argv[0]);
      return f == "-h" || f == "--help" ? 0 : 1;
    }
  }
  if (msgs.empty()) parse_size_list("64M", &msgs);
  const int ndev = device_count();
  const bool two = peer != gemm_dev && peer < ndev;
  if (gemm_dev >= ndev) { std::fprintf(stderr, "no GPU %d\n", gemm_dev); return 1; }
  if (two && !enable_peer_all(std::max(gemm_dev, peer) + 1)) return 1;
  size_t max_msg = 0;
  for (size_t m : msgs) max_msg = std::max(max_msg, m);
  print_device_line(gemm_dev);
  char *loc_a, *loc_b, *rem = nullptr, *host;
  TCL_CUDA_CHECK(cudaSetDevice(gemm_dev));
  TCL_CUDA_CHECK(cudaMalloc(&loc_a, max_msg));
  TCL_CUDA_CHECK(cudaMalloc(&loc_b, max_msg));
  TCL_CUDA_CHECK(cudaHostAlloc(&host, max_msg, cudaHostAllocDefault));
  cudaStream_t cs[2];
  TCL_CUDA_CHECK(cudaStreamCreateWithFlags(&cs[0], cudaStreamNonBlocking));
  TCL_CUDA_CHECK(cudaStreamCreateWithFlags(&cs[1], cudaStreamNonBlocking));
  if (two) { TCL_CUDA_CHECK(cudaSetDevice(peer)); TCL_CUDA_CHECK(cudaMalloc(&rem, max_msg)); TCL_CUDA_CHECK(cudaSetDevice(gemm_dev)); }
  Csv csv;
  if (!csv.open(csv_path, "m,n,k,dtype,comm,dir,msg_bytes,gemm_alone_us,gemm_ovl_us,gemm_alone_p95,gemm_ovl_p95,S_c,tflops_alone,tflops_ovl,comm_alone_gbps,comm_ovl_gbps_approx,comm_ovl_gbps,S_m,gaps")) return 1;
  std::printf("%-14s %-5s %-10s %10s | %10s %10s %6s | %10s %10s %6s | %s\n", "shape", "dtype", "comm", "msg", "gemm_alone", "gemm_ovl", "S_c", "comm_alone", "comm_ovl", "S_m", "gaps");
  for (auto& ss : shapes) {
    Shape3 sh;
    if (!parse_shape(ss, &sh)) { std::fprintf(stderr, "bad shape %s\n", ss.c_str()); return 1; }
    for (auto& dt : dtypes) {
      Gemm g;
      g.init(gemm_dev, sh, dt);
      for (int i = 0; i < 3; ++i) g.run();
      TCL_CUDA_CHECK(cudaStreamSynchronize(g.st));
      const double flop = 2.0 * sh.m * sh.n * sh.k;
      for (auto& cn : comms) {
        if (!two && cn.rfind("p2p", 0) == 0) continue;
        for (size_t msg : msgs) {
          Comm c;
          c.msg = msg;
          if (cn == "p2p_push") c.legs.push_back({rem, peer, loc_a, gemm_dev, cs[0], false});
          else if (cn == "p2p_pull") c.legs.push_back({loc_a, gemm_dev, rem, peer, cs[0], false});
          else if (cn == "p2p_bidir") { c.legs.push_back({rem, peer, loc_a, gemm_dev, cs[0], false}); c.legs.push_back({loc_b, gemm_dev, rem, peer, cs[1], false}); }
          else if (cn == "d2d") c.legs.push_back({loc_b, gemm_dev, loc_a, gemm_dev, cs[0], true});
          else if (cn == "h2d") c.legs.push_back({loc_a, gemm_dev, host, -1, cs[0], true});
          else if (cn == "d2h") c.legs.push_back({host, -1, loc_a, gemm_dev, cs[0], true});
          else continue;
          // Paired alone baselines, taken right before the overlapped run.
          const Stats ga = g.time(iters);
          const double ca = c.gbps(4);
          // Phase A: GEMM timed, copies pumped (re-enqueued whenever the copy streams drain).
          int gaps = 0;
          std::vector<double> us;
          c.burst(4);
          for (int i = 0; i < iters; ++i) {
            TCL_CUDA_CHECK(cudaEventRecord(g.e0, g.st));
            g.run();
            TCL_CUDA_CHECK(cudaEventRecord(g.e1, g.st));
            while (cudaEventQuery(g.e1) == cudaErrorNotReady) {
              if (c.idle()) { ++gaps; c.burst(4); }
            }
            cudaGetLastError();
            us.push_back(elapsed_us(g.e0, g.e1));
          }
          c.sync();
          const Stats go = make_stats(us);
          // Phase B: a burst of copies timed (wall clock) while GEMMs are kept queued.
          for (int i = 0; i < 4; ++i) g.run();
          const double t0 = now_ms();
          c.burst(4);
          while (!c.idle()) { if (cudaStreamQuery(g.st) == cudaSuccess) for (int i = 0; i < 2; ++i) g.run(); else cudaGetLastError(); }
          const double co = static_cast<double>(msg) * c.legs.size() * 4 / ((now_ms() - t0) * 1e6);
          TCL_CUDA_CHECK(cudaStreamSynchronize(g.st));
          const double sc = ga.mean > 0 ? go.mean / ga.mean : 0, sm = co > 0 ? ca / co : 0;
          std::printf("%-14s %-5s %-10s %10zu | %10.1f %10.1f %6.3f | %10.1f %10.1f %6.3f | %d\n", ss.c_str(), dt.c_str(), cn.c_str(), msg, ga.mean, go.mean, sc, ca, co, sm, gaps);
          csv.row("%d,%d,%d,%s,%s,%s,%zu,%.2f,%.2f,%.2f,%.2f,%.4f,%.1f,%.1f,%.2f,%.2f,%.2f,%.4f,%d", sh.m, sh.n, sh.k, dt.c_str(), cn.c_str(),
                  cn == "p2p_pull" || cn == "h2d" ? "in" : cn == "p2p_bidir" ? "both" : "out", msg, ga.mean, go.mean, ga.p95, go.p95, sc, flop / ga.mean / 1e6,
                  flop / go.mean / 1e6, ca, co, co, sm, gaps);
        }
      }
      TCL_CUDA_CHECK(cudaFree(g.A)); TCL_CUDA_CHECK(cudaFree(g.B)); TCL_CUDA_CHECK(cudaFree(g.C));
      cublasDestroy(g.h);
    }
  }
  return 0;
}
