// exp2_ag_gemm_granularity (native driver): all-gather -> GEMM at several gather granularities,
// ranks forked by the native launcher, buffers shared as cudaIpc handles, kernels through the C
// interface of the library.  Per granularity (rows per gather tile):
//   t_full  one plain GEMM on a pre-gathered A            t_seg  the fused kernel with communication off
//   t_ovl   the fused kernel pulling the peers' shards    seg_eff = t_full / t_seg, overlap_eff = t_seg / t_ovl
// Verification scrubs the peers' rows of the gathered buffer with 0x55, runs the fused kernel once and
// compares its output bit-wise with the pre-gathered run.  (The Python driver of the same name also has
// the copy-engine and NCCL modes.)
//
// Reference parity: comm_comp/exp2_ag_gemm_granularity.cu (pipeline :168-300, verify :511-533, CSV :446-448).
#include <string>

#include "native_common.cuh"

using namespace tcl::host;
using namespace tcl::native;
using tcl::rt::Launcher;

__global__ void count_diff_kernel(const uint4* a, const uint4* b, size_t nvec, unsigned long long* out) {
  unsigned long long c = 0;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nvec; i += (size_t)gridDim.x * blockDim.x) {
    const uint4 x = a[i], y = b[i];
    c += (x.x != y.x) + (x.y != y.y) + (x.z != y.z) + (x.w != y.w);
  }
  if (c) atomicAdd(out, c);
}

int main(int argc, char** argv) {
  int M = 32768, K = 8192, N = 0, n_global = 28672, ndev = 0, iters = 20, warm = 3, cta_group = 2;
  std::vector<int> grains;
  bool verify = false;
  std::string csv_path;
  Args a(argc, argv);
  while (a.more()) {
    std::string f = a.flag(), v;
    auto need = [&]() { if (!a.value(&v)) std::exit(1); return v; };
    if (f == "--m") M = std::atoi(need().c_str());
    else if (f == "--k") K = std::atoi(need().c_str());
    else if (f == "--n") N = std::atoi(need().c_str());
    else if (f == "--n-global") n_global = std::atoi(need().c_str());
    else if (f == "--gather-rows") parse_int_list(need(), &grains);
    else if (f == "--ndev") ndev = std::atoi(need().c_str());
    else if (f == "--iters") iters = std::atoi(need().c_str());
    else if (f == "--warmup") warm = std::atoi(need().c_str());
    else if (f == "--cta-group") cta_group = std::atoi(need().c_str());
    else if (f == "--verify") verify = true;
    else if (f == "--csv") csv_path = need();
    else {
      std::printf("usage: %s [--m M] [--k K] [--n N_local | --n-global N] [--gather-rows LIST] [--ndev W] [--iters I] [--warmup W] [--cta-group 1|2] [--verify] [--csv FILE]\n", argv[0]);
      return f == "-h" || f == "--help" ? 0 : 1;
    }
  }
  const int have = Launcher::probe_device_count();
  const int world = ndev > 0 ? ndev : have;
  if (world < 1 || world > have || world > TCL_MAX_WORLD) { std::fprintf(stderr, "need %d GPUs, have %d\n", world, have); return 1; }
  if (N <= 0) N = n_global / world;
  const int seg = M / world;
  if (M % (world * 128 * cta_group) || N % 256 || K % 8) { std::fprintf(stderr, "shape not supported\n"); return 1; }
  if (grains.empty()) grains = {128, 512, 2048, 4096};

  Launcher L;
  const int rank = L.init(world);
  if (rank < 0) return 2;
  if (cudaSetDevice(rank) != cudaSuccess) die(L, "cudaSetDevice");
  const size_t mk = size_t(M) * K, mn = size_t(M) * N;
  Buf afull, flags, done, bar_k, bar_d;
  void *B, *out, *out_ref, *gathered;
  int32_t* status;
  unsigned long long* diff;
  TCL_CUDA_CHECK(cudaMalloc(&afull.local, mk * 2));
  TCL_CUDA_CHECK(cudaMalloc(&gathered, mk * 2));
  TCL_CUDA_CHECK(cudaMalloc(&B, size_t(N) * K * 2));
  TCL_CUDA_CHECK(cudaMalloc(&out, mn * 2));
  TCL_CUDA_CHECK(cudaMalloc(&out_ref, mn * 2));
  TCL_CUDA_CHECK(cudaMalloc(&flags.local, (M / 128 + 32) * 4));
  TCL_CUDA_CHECK(cudaMalloc(&done.local, 128));
  TCL_CUDA_CHECK(cudaMalloc(&bar_k.local, 128));
  TCL_CUDA_CHECK(cudaMalloc(&bar_d.local, 128));
  TCL_CUDA_CHECK(cudaMalloc(&status, 64));
  TCL_CUDA_CHECK(cudaMalloc(&diff, 8));
  TCL_CUDA_CHECK(cudaMemset(done.local, 0, 128));
  TCL_CUDA_CHECK(cudaMemset(bar_k.local, 0, 128));
  TCL_CUDA_CHECK(cudaMemset(bar_d.local, 0, 128));
  TCL_CUDA_CHECK(cudaMemset(status, 0, 64));
  cudaStream_t st;
  TCL_CUDA_CHECK(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking));
  char* shard = static_cast<char*>(afull.local) + size_t(rank) * seg * K * 2;
  tcl_fill_normal_bf16(shard, int64_t(seg) * K, 600 + rank, 0.f, 1.f, st);
  tcl_fill_normal_bf16(B, int64_t(N) * K, 500 + rank, 0.f, 0.02f, st);
  TCL_CUDA_CHECK(cudaStreamSynchronize(st));
  if (!share(L, 0, afull) || !share(L, 1, flags) || !share(L, 2, done) || !share(L, 3, bar_k) || !share(L, 4, bar_d)) die(L, "handle exchange failed");
  // Pre-gathered copy for t_full and for the verification reference (plain peer copies).
  for (int r = 0; r < world; ++r)
    TCL_CUDA_CHECK(cudaMemcpyAsync(static_cast<char*>(gathered) + size_t(r) * seg * K * 2, static_cast<char*>(afull.peer[r]) + size_t(r) * seg * K * 2, size_t(seg) * K * 2, cudaMemcpyDefault, st));
  TCL_CUDA_CHECK(cudaStreamSynchronize(st));
  if (!L.barrier()) die(L, "peer failed");

  DeviceBarrier bar;
  bar.world = world; bar.rank = rank; bar.status = status + 8;
  for (int s = 0; s < world; ++s) bar.ptrs[s] = static_cast<int32_t*>(bar_d.peer[s]);
  cudaEvent_t e0, e1;
  TCL_CUDA_CHECK(cudaEventCreate(&e0));
  TCL_CUDA_CHECK(cudaEventCreate(&e1));
  char err[256];
  auto plain_plan = [&]() {
    tcl_gemm_desc d;
    std::memset(&d, 0, sizeof(d));
    d.mode = TCL_MODE_PLAIN; d.cta_group = cta_group; d.M = M; d.N = N; d.K = K; d.lda = K; d.ldb = K; d.ldc = N; d.A = gathered; d.B = B;
    d.world = 1; d.seg_rows = M; d.dst_base[0] = out_ref; d.status = status;
    void* p = tcl_gemm_plan_create(&d, err, sizeof(err));
    if (!p) die(L, err);
    return p;
  };
  auto ag_plan = [&](int gather_rows, int comm) {
    tcl_gemm_desc d;
    std::memset(&d, 0, sizeof(d));
    d.mode = TCL_MODE_AG_GEMM; d.cta_group = cta_group; d.M = M; d.N = N; d.K = K; d.lda = K; d.ldb = K; d.ldc = N;
    d.A = comm ? afull.local : gathered; d.B = B; d.world = world; d.rank = rank; d.seg_rows = seg; d.comm_enabled = comm;
    for (int s = 0; s < world; ++s) {
      d.dst_base[s] = out; d.dst_row_off[s] = int64_t(s) * seg;
      d.ag_src[s] = static_cast<char*>(afull.peer[s]) + size_t(s) * seg * K * 2;
      d.ag_read_done[s] = static_cast<int32_t*>(done.peer[s]) + 16;
      d.barrier[s] = static_cast<int32_t*>(bar_k.peer[s]);
    }
    d.ag_flags = static_cast<int32_t*>(flags.local); d.gather_rows = gather_rows; d.ag_item_rows = 1; d.ag_done = static_cast<int32_t*>(done.local);
    d.status = status;
    void* p = tcl_gemm_plan_create(&d, err, sizeof(err));
    if (!p) die(L, err);
    return p;
  };
  void* full = plain_plan();
  int ep_full = 0;
  if (rank == 0) {
    std::printf("# exp2 AG+GEMM (native launcher)  M=%d N/rank=%d K=%d world=%d cta_group=%d iters=%d\n", M, N, K, world, cta_group, iters);
    std::printf("    S chunk_rows |  t_full us   t_seg us   t_ovl us | seg_eff ovl_eff | e2e TF/s | verify\n");
  }
  Csv csv;
  if (rank == 0) csv.open(csv_path, "m,n,k,world,S,chunk_rows,chunk_mib,mode,streams,t_full_us,t_seg_us,t_comm_us,t_ovl_us,seg_eff,comm_gbps,overlap_eff,e2e_tflops,verify,"
                                    "max_over_ranks_us,nccl_cublas_us,speedup,roofline_us,pct_roofline,dtype");
  int rc = 0;
  for (int g : grains) {
    if (g > seg) g = seg;
    if (seg % g || g % 128) continue;
    // Counters restart for a plan with a different arrival count per epoch.
    TCL_CUDA_CHECK(cudaMemset(flags.local, 0, (M / 128 + 32) * 4));
    TCL_CUDA_CHECK(cudaMemset(done.local, 0, 128));
    TCL_CUDA_CHECK(cudaMemset(bar_k.local, 0, 128));
    TCL_CUDA_CHECK(cudaDeviceSynchronize());
    if (!L.barrier()) die(L, "peer failed");
    void* seg_plan = ag_plan(g, 0);
    void* ovl_plan = ag_plan(g, 1);
    int ep_seg = 0, ep_ovl = 0;
    const char* ver = "-";
    if (verify) {
      tcl_gemm_plan_run(full, ++ep_full, st);
      // scrub the peers' rows: a broken dependency would feed 0x55 bytes to the GEMM
      TCL_CUDA_CHECK(cudaMemsetAsync(afull.local, 0x55, size_t(rank) * seg * K * 2, st));
      TCL_CUDA_CHECK(cudaMemsetAsync(shard + size_t(seg) * K * 2, 0x55, size_t(world - 1 - rank) * seg * K * 2, st));
      TCL_CUDA_CHECK(cudaMemsetAsync(out, 0, mn * 2, st));
      TCL_CUDA_CHECK(cudaStreamSynchronize(st));
      if (!L.barrier()) die(L, "peer failed");
      bar.run(st);
      tcl_gemm_plan_run(ovl_plan, ++ep_ovl, st);
      TCL_CUDA_CHECK(cudaMemsetAsync(diff, 0, 8, st));
      count_diff_kernel<<<1024, 256, 0, st>>>(static_cast<const uint4*>(out), static_cast<const uint4*>(out_ref), mn * 2 / 16, diff);
      unsigned long long h = 1;
      TCL_CUDA_CHECK(cudaMemcpyAsync(&h, diff, 8, cudaMemcpyDeviceToHost, st));
      TCL_CUDA_CHECK(cudaStreamSynchronize(st));
      ver = h == 0 ? "ok" : "FAIL";
      if (h) rc = 4;
      if (!L.barrier()) die(L, "peer failed");
    }
    std::vector<double> tf, ts, to;
    for (int it = 0; it < warm + iters; ++it) {
      if (L.failed()) die(L, "a peer failed during timing");
      const double a0 = timed_run(full, &ep_full, bar, st, e0, e1);
      const double a1 = timed_run(seg_plan, &ep_seg, bar, st, e0, e1);
      const double a2 = timed_run(ovl_plan, &ep_ovl, bar, st, e0, e1);
      if (a0 < 0 || a1 < 0 || a2 < 0) die(L, "launch failed");
      if (it >= warm) { tf.push_back(a0); ts.push_back(a1); to.push_back(a2); }
      L.beat();
    }
    int hst[16];
    TCL_CUDA_CHECK(cudaMemcpy(hst, status, 64, cudaMemcpyDeviceToHost));
    if (hst[0] || hst[8]) { std::fprintf(stderr, "rank %d: %s\n", rank, tcl_status_string(hst[0] ? hst[0] : hst[8])); die(L, "a device wait ran out"); }
    double* res = L.shm()->results[rank];
    res[0] = make_stats(tf).mean; res[1] = make_stats(ts).mean; res[2] = make_stats(to).mean; res[3] = std::strcmp(ver, "FAIL") == 0;
    if (!L.barrier()) die(L, "peer failed");
    if (rank == 0) {
      double f = 0, s = 0, o = 0, bad = 0;
      for (int r = 0; r < world; ++r) { f = std::max(f, L.shm()->results[r][0]); s = std::max(s, L.shm()->results[r][1]); o = std::max(o, L.shm()->results[r][2]); bad += L.shm()->results[r][3]; }
      const double flop = 2.0 * M * N * K;
      if (bad) { ver = "FAIL"; rc = 4; }
      std::printf("%5d %10d | %10.1f %10.1f %10.1f | %7.3f %7.3f | %8.0f | %s\n", seg / g, g, f, s, o, f / s, s / o, flop / o / 1e6, ver);
      csv.row("%d,%d,%d,%d,%d,%d,%.2f,fused,1,%.2f,%.2f,0,%.2f,%.4f,0,%.4f,%.1f,%s,%.2f,,,,,bf16", M, N, K, world, seg / g, g, double(g) * K * 2 / 1048576.0, f, s, o, f / s, s / o,
              flop / o / 1e6, ver, o);
    }
    if (!L.barrier()) die(L, "peer failed");
    tcl_gemm_plan_destroy(seg_plan);
    tcl_gemm_plan_destroy(ovl_plan);
  }
  tcl_gemm_plan_destroy(full);
  TCL_CUDA_CHECK(cudaDeviceSynchronize());
  if (!L.barrier()) rc = rc ? rc : 5;
  for (Buf* b : {&afull, &flags, &done, &bar_k, &bar_d}) unshare(L, *b);
  L.barrier();
  if (rank != 0) _exit(rc);
  const int worst = L.wait_children(30.0);
  return rc ? rc : worst;
}
