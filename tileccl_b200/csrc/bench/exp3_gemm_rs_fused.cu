// exp3_gemm_rs_fused (native driver): the fused GEMM + reduce-scatter with no Python and no
// torch.distributed - ranks are forked by the native launcher, buffers are exchanged as cudaIpc
// handles through its shared blob, and the kernels are driven through the C interface of the library.
// Same three variants per rank as the Python driver (bench/exp3_gemm_rs_fused.py):
//   base  plain tcgen05 GEMM      ctrl  fused kernel, communication off      fused  the real thing
// one iteration of each in turn, a device barrier before every timed iteration, per-iteration CUDA
// events; fp32 verification against the sum of every rank's base result; the reference's 27 CSV
// columns (NCCL columns stay empty here: this program links no NCCL).  --order picks the variants and their
// order inside an iteration, --dump-iters writes every rank's per-iteration times, --warmup-ms adds a
// wall-clock warm-up whose iteration count rank 0 derives from its own pace and shares with the others
// through the launcher's shared blob (every rank must make the same number of fused launches).
//
// Reference parity: comm_comp/exp3_gemm_rs_fused.cu (main :337-691) on top of
// comm_comp/ipc_multiproc.cuh; --k is K per rank as there, --k-global shards a global K.
#include <unistd.h>

#include <chrono>
#include <string>
#include <vector>

#include <cuda_bf16.h>

#include "../common/host_common.hpp"
#include "../ops/tileccl_ops.h"
#include "../runtime/launcher.hpp"

using namespace tcl::host;
using tcl::rt::Launcher;

// ref[i] = sum over ranks of D_r[seg_off + i] in fp32.
struct PeerD { const __nv_bfloat16* d[TCL_MAX_WORLD]; };
__global__ void sum_partials_kernel(PeerD p, int world, size_t seg_off, size_t n, float* ref) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    float s = 0.f;
    for (int r = 0; r < world; ++r) s += __bfloat162float(p.d[r][seg_off + i]);
    ref[i] = s;
  }
}
__global__ void max_abs_diff_kernel(const __nv_bfloat16* got, const float* ref, size_t n, float* out) {
  float m = 0.f;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    float e = fabsf(__bfloat162float(got[i]) - ref[i]);
    if (!(e == e)) e = 3.4e38f;
    m = fmaxf(m, e);
  }
  atomicMax(reinterpret_cast<int*>(out), __float_as_int(m));   // non-negative floats order like ints
}

struct Buf { void* local = nullptr; void* peer[TCL_MAX_WORLD] = {}; };

static bool share(Launcher& L, int slot, Buf& b) {
  cudaIpcMemHandle_t mine, all[TCL_MAX_WORLD];
  if (cudaIpcGetMemHandle(&mine, b.local) != cudaSuccess) { L.fail("cudaIpcGetMemHandle"); return false; }
  if (!L.exchange(slot, &mine, sizeof(mine), all)) return false;
  for (int r = 0; r < L.world(); ++r) {
    if (r == L.rank()) { b.peer[r] = b.local; continue; }
    if (cudaIpcOpenMemHandle(&b.peer[r], all[r], cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) { L.fail("cudaIpcOpenMemHandle"); return false; }
  }
  return L.barrier();
}

int main(int argc, char** argv) {
  int M = 8192, N = 8192, K = 0, k_global = 8192, ndev = 0, iters = 50, warm = 5, cta_group = 2;
  bool verify = false;
  double warmup_ms = 0;
  std::string csv_path, order_arg = "base,ctrl,fused", dump_prefix;
  Args a(argc, argv);
  while (a.more()) {
    std::string f = a.flag(), v;
    auto need = [&]() { if (!a.value(&v)) std::exit(1); return v; };
    if (f == "--m") M = std::atoi(need().c_str());
    else if (f == "--n") N = std::atoi(need().c_str());
    else if (f == "--k") K = std::atoi(need().c_str());
    else if (f == "--k-global") k_global = std::atoi(need().c_str());
    else if (f == "--ndev") ndev = std::atoi(need().c_str());
    else if (f == "--iters") iters = std::atoi(need().c_str());
    else if (f == "--warmup") warm = std::atoi(need().c_str());
    else if (f == "--cta-group") cta_group = std::atoi(need().c_str());
    else if (f == "--verify") verify = true;
    else if (f == "--csv") csv_path = need();
    else if (f == "--order") order_arg = need();
    else if (f == "--dump-iters") dump_prefix = need();
    else if (f == "--warmup-ms") warmup_ms = std::atof(need().c_str());
    else {
      std::printf("usage: %s [--m M] [--n N] [--k K_per_rank | --k-global K] [--ndev W] [--iters I] [--warmup W] [--warmup-ms MS]\n"
                  "          [--order base,ctrl,fused] [--dump-iters PREFIX] [--cta-group 1|2] [--verify] [--csv FILE]\n", argv[0]);
      return f == "-h" || f == "--help" ? 0 : 1;
    }
  }
  static const char* kVariantNames[3] = {"base", "ctrl", "fused"};
  std::vector<int> order;
  for (auto& name : split_csv(order_arg)) {
    int id = -1;
    for (int v = 0; v < 3; ++v) if (name == kVariantNames[v]) id = v;
    if (id < 0) { std::fprintf(stderr, "--order: unknown variant %s (base, ctrl, fused)\n", name.c_str()); return 1; }
    order.push_back(id);
  }
  if (order.empty()) { std::fprintf(stderr, "--order is empty\n"); return 1; }
  const int have = Launcher::probe_device_count();     // in a child: this process stays CUDA-free until after fork
  const int world = ndev > 0 ? ndev : have;
  if (world < 1 || world > have || world > TCL_MAX_WORLD) { std::fprintf(stderr, "need %d GPUs, have %d\n", world, have); return 1; }
  if (K <= 0) K = k_global / world;
  const int seg = M / world;
  if (M % (world * 128 * cta_group) || N % 256 || K % 8) { std::fprintf(stderr, "shape not supported: M %% (world*128*cta_group), N %% 256, K %% 8 must be 0\n"); return 1; }

  Launcher L;
  const int rank = L.init(world);
  if (rank < 0) return 2;
  auto die = [&](const char* why) { L.fail(why); std::fprintf(stderr, "rank %d: %s\n", rank, why); if (rank) _exit(3); L.wait_children(10); std::exit(3); };
  if (cudaSetDevice(rank) != cudaSuccess) die("cudaSetDevice");

  const size_t mn = size_t(M) * N, segn = size_t(seg) * N;
  void *A, *B, *D;
  Buf stage, cnt, bar_fused, bar_dev, out, dbuf;
  int* status;
  float *ref, *maxd;
  TCL_CUDA_CHECK(cudaMalloc(&A, size_t(M) * K * 2));
  TCL_CUDA_CHECK(cudaMalloc(&B, size_t(N) * K * 2));
  TCL_CUDA_CHECK(cudaMalloc(&D, mn * 2));
  TCL_CUDA_CHECK(cudaMalloc(&stage.local, mn * 2));
  TCL_CUDA_CHECK(cudaMalloc(&out.local, segn * 2));
  const size_t ncnt = size_t(seg / 128) * (N / 256);
  TCL_CUDA_CHECK(cudaMalloc(&cnt.local, ncnt * 4));
  TCL_CUDA_CHECK(cudaMemset(cnt.local, 0, ncnt * 4));
  TCL_CUDA_CHECK(cudaMalloc(&bar_fused.local, 128));
  TCL_CUDA_CHECK(cudaMemset(bar_fused.local, 0, 128));
  TCL_CUDA_CHECK(cudaMalloc(&bar_dev.local, 128));
  TCL_CUDA_CHECK(cudaMemset(bar_dev.local, 0, 128));
  TCL_CUDA_CHECK(cudaMalloc(&status, 64));
  TCL_CUDA_CHECK(cudaMemset(status, 0, 64));
  TCL_CUDA_CHECK(cudaMalloc(&ref, segn * 4));
  TCL_CUDA_CHECK(cudaMalloc(&maxd, 4));
  dbuf.local = D;
  cudaStream_t st;
  TCL_CUDA_CHECK(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking));
  tcl_fill_normal_bf16(A, int64_t(M) * K, 1000 + rank, 0.f, 1.f, st);
  tcl_fill_normal_bf16(B, int64_t(N) * K, 2000 + rank, 0.f, 1.f, st);
  TCL_CUDA_CHECK(cudaStreamSynchronize(st));
  if (world > 1) {
    if (!share(L, 0, stage) || !share(L, 1, cnt) || !share(L, 2, bar_fused) || !share(L, 3, bar_dev) || !share(L, 4, dbuf)) die("handle exchange failed");
  } else {
    stage.peer[0] = stage.local; cnt.peer[0] = cnt.local; bar_fused.peer[0] = bar_fused.local; bar_dev.peer[0] = bar_dev.local; dbuf.peer[0] = D;
  }

  char err[256];
  auto make = [&](int mode, int comm) -> void* {
    tcl_gemm_desc d;
    std::memset(&d, 0, sizeof(d));
    d.mode = mode; d.cta_group = cta_group; d.M = M; d.N = N; d.K = K; d.lda = K; d.ldb = K; d.ldc = N; d.A = A; d.B = B;
    d.status = status;
    if (mode == TCL_MODE_PLAIN) { d.world = 1; d.rank = 0; d.seg_rows = M; d.dst_base[0] = D; }
    else {
      d.world = world; d.rank = rank; d.seg_rows = seg; d.comm_enabled = comm;
      for (int s = 0; s < world; ++s) {
        d.dst_base[s] = comm ? stage.peer[s] : stage.local;
        d.dst_row_off[s] = comm ? int64_t(rank) * seg : int64_t(s) * seg;
        d.rs_tile_cnt[s] = static_cast<int32_t*>(cnt.peer[s]);
        d.barrier[s] = static_cast<int32_t*>(bar_fused.peer[s]);
      }
      d.rs_stage = stage.local; d.rs_out = out.local; d.ld_out = N;
    }
    void* p = tcl_gemm_plan_create(&d, err, sizeof(err));
    if (!p) { std::fprintf(stderr, "rank %d: plan rejected: %s\n", rank, err); die("plan"); }
    return p;
  };
  void* plans[3] = {make(TCL_MODE_PLAIN, 0), make(TCL_MODE_GEMM_RS, 0), make(TCL_MODE_GEMM_RS, 1)};
  int epochs[3] = {0, 0, 0}, bar_epoch = 0;
  int32_t* bar_ptrs[TCL_MAX_WORLD];
  for (int s = 0; s < world; ++s) bar_ptrs[s] = static_cast<int32_t*>(bar_dev.peer[s]);
  cudaEvent_t e0, e1;
  TCL_CUDA_CHECK(cudaEventCreate(&e0));
  TCL_CUDA_CHECK(cudaEventCreate(&e1));
  std::vector<double> us[3];
  if (!L.barrier()) die("a rank failed before timing");
  auto one_iteration = [&](bool record) {
    if (L.failed()) die("a peer failed during timing");   // learnt on the host, before the next launch
    for (int v : order) {
      tcl_barrier_all(bar_ptrs, world, rank, ++bar_epoch, status + 8, 0, st);
      TCL_CUDA_CHECK(cudaEventRecord(e0, st));
      if (tcl_gemm_plan_run(plans[v], ++epochs[v], st) != 0) die("launch failed");
      TCL_CUDA_CHECK(cudaEventRecord(e1, st));
      TCL_CUDA_CHECK(cudaEventSynchronize(e1));
      if (record) us[v].push_back(elapsed_us(e0, e1));
    }
    L.beat();
  };
  const auto w0 = std::chrono::steady_clock::now();
  for (int it = 0; it < warm; ++it) one_iteration(false);
  if (warmup_ms > 0) {
    // Rank 0 turns the wall-clock budget into an iteration count from its own pace; all ranks run that many.
    const double spent_ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - w0).count();
    if (rank == 0) {
      const double per_iter = warm > 0 ? spent_ms / warm : 1.0;
      const double extra = (warmup_ms - spent_ms) / (per_iter > 1e-3 ? per_iter : 1e-3);
      L.shm()->results[0][15] = extra > 0 ? std::ceil(std::min(extra, 1e6)) : 0.0;
    }
    if (!L.barrier()) die("a rank failed during warm-up");
    const int extra_iters = static_cast<int>(L.shm()->results[0][15]);
    for (int it = 0; it < extra_iters; ++it) one_iteration(false);
    if (rank == 0) std::printf("# warm-up: %d + %d iterations (%.0f ms asked)\n", warm, extra_iters, warmup_ms);
  }
  for (int it = 0; it < iters; ++it) one_iteration(true);
  if (!dump_prefix.empty()) {
    Csv dump;
    if (dump.open(dump_prefix + ".rank" + std::to_string(rank) + ".csv", "m,n,k,world,rank,variant,iter,us"))
      for (int v : order)
        for (size_t i = 0; i < us[v].size(); ++i) dump.row("%d,%d,%d,%d,%d,%s,%zu,%.3f", M, N, K, world, rank, kVariantNames[v], i, us[v][i]);
  }
  int hst[16];
  TCL_CUDA_CHECK(cudaMemcpy(hst, status, 64, cudaMemcpyDeviceToHost));
  if (hst[0] || hst[8]) { std::fprintf(stderr, "rank %d: a device wait ran out: %s\n", rank, tcl_status_string(hst[0] ? hst[0] : hst[8])); die("device time-out"); }

  double max_abs = -1;
  if (verify) {
    // every rank's base result is in its D; the fused output must equal the fp32 sum of the peers' rows
    tcl_gemm_plan_run(plans[0], ++epochs[0], st);
    TCL_CUDA_CHECK(cudaStreamSynchronize(st));
    if (!L.barrier()) die("peer failed");
    tcl_barrier_all(bar_ptrs, world, rank, ++bar_epoch, status + 8, 0, st);
    tcl_gemm_plan_run(plans[2], ++epochs[2], st);
    PeerD pd;
    for (int r = 0; r < world; ++r) pd.d[r] = static_cast<const __nv_bfloat16*>(dbuf.peer[r]);
    sum_partials_kernel<<<1024, 256, 0, st>>>(pd, world, size_t(rank) * segn, segn, ref);
    TCL_CUDA_CHECK(cudaMemsetAsync(maxd, 0, 4, st));
    max_abs_diff_kernel<<<1024, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(out.local), ref, segn, maxd);
    float h = 0;
    TCL_CUDA_CHECK(cudaMemcpyAsync(&h, maxd, 4, cudaMemcpyDeviceToHost, st));
    TCL_CUDA_CHECK(cudaStreamSynchronize(st));
    max_abs = h;
    if (!L.barrier()) die("peer failed");
  }
  Stats s[3];
  for (int v = 0; v < 3; ++v) s[v] = make_stats(us[v]);
  double* res = L.shm()->results[rank];
  for (int v = 0; v < 3; ++v) { res[4 * v] = s[v].mean; res[4 * v + 1] = s[v].p95; res[4 * v + 2] = s[v].p50; res[4 * v + 3] = s[v].min; }
  res[12] = max_abs;
  if (!L.barrier()) die("peer failed");
  int rc = 0;
  if (rank == 0) {
    const double flop = 2.0 * M * N * K;
    const double scale = std::sqrt(double(K) * world);
    std::printf("# exp3 fused GEMM+RS (native launcher)  M=%d N=%d K/rank=%d world=%d cta_group=%d iters=%d\n", M, N, K, world, cta_group, iters);
    std::printf("rank |  base us   TF/s |  ctrl us | fused us   TF/s | struct   comm  total | push GB/s | verify\n");
    Csv csv;
    csv.open(csv_path, "m,n,k,world,rank,base_us,base_p95,ctrl_us,ctrl_p95,fused_us,fused_p95,struct_sd,comm_sd,total_sd,pull_gbps,max_rel_diff,"
                       "base_p50,ctrl_p50,fused_p50,base_min,ctrl_min,fused_min,comm_sd_p50,comm_sd_skew,comm_abs_us,order,iters,"
                       "max_over_ranks_us,nccl_cublas_us,speedup,roofline_us,pct_roofline,dtype");
    double ctrl_max = 0, fused_max = 0;
    auto ratio = [](double x, double y) { return y > 0 ? x / y : 0.0; };   // a variant left out of --order has no time
    std::string order_col;
    for (int v : order) order_col += (order_col.empty() ? "" : "|") + std::string(kVariantNames[v]);
    for (int r = 0; r < world; ++r) { ctrl_max = std::max(ctrl_max, L.shm()->results[r][4]); fused_max = std::max(fused_max, L.shm()->results[r][8]); }
    for (int r = 0; r < world; ++r) {
      const double* q = L.shm()->results[r];
      const double b = q[0], c = q[4], f = q[8];
      const double gb = f > 0 ? double(world - 1) / world * M * N * 2 / (f * 1e-6) / 1e9 : 0.0;
      const double rel = q[12] < 0 ? -1 : q[12] / scale;     // error on the scale of the partial sums
      char ver[48];
      if (q[12] < 0) std::snprintf(ver, sizeof(ver), "-");
      else { std::snprintf(ver, sizeof(ver), "%s (max|d|/sqrt(K*w) %.3g)", rel <= 0.05 ? "ok" : "FAIL", rel); if (rel > 0.05) rc = 4; }
      std::printf("%4d | %9.1f %6.0f | %8.1f | %8.1f %6.0f | %6.3f %6.3f %6.3f | %9.1f | %s\n", r, b, ratio(flop, b) / 1e6, c, f, ratio(flop, f) / 1e6, ratio(c, b), ratio(f, c),
                  ratio(f, b), gb, ver);
      csv.row("%d,%d,%d,%d,%d,%.2f,%.2f,%.2f,%.2f,%.2f,%.2f,%.4f,%.4f,%.4f,%.2f,%.4g,%.2f,%.2f,%.2f,%.2f,%.2f,%.2f,%.4f,%.4f,%.2f,%s,%d,%.2f,,,,,bf16", M, N, K, world, r, b,
              q[1], c, q[5], f, q[9], ratio(c, b), ratio(f, c), ratio(f, b), gb, rel, q[2], q[6], q[10], q[3], q[7], q[11], ratio(q[10], q[6]), ratio(f, ctrl_max), f - c,
              order_col.c_str(), iters, fused_max);
    }
    std::printf("max over ranks: fused %.1f us\n", fused_max);
  }
  for (int v = 0; v < 3; ++v) tcl_gemm_plan_destroy(plans[v]);
  TCL_CUDA_CHECK(cudaDeviceSynchronize());
  if (!L.barrier()) rc = rc ? rc : 5;      // nobody closes a mapping a peer may still use
  if (world > 1)
    for (Buf* b : {&stage, &cnt, &bar_fused, &bar_dev, &dbuf})
      for (int r = 0; r < world; ++r) if (r != rank) cudaIpcCloseMemHandle(b->peer[r]);
  L.barrier();
  if (rank != 0) _exit(rc);
  const int worst = L.wait_children(30.0);
  return rc ? rc : worst;
}
