// exp3_epilogue_remote (native driver): the cost of pointing the GEMM epilogue at a peer.  The same
// tcgen05 GEMM with only its output routing changed:
//   local  D in this GPU's memory      remote  all of D in the next rank's memory
//   scatter-local  D cut into `world` row segments, all local      scatter  segment s goes to rank s
// slowdown = time / time of `local`, one iteration of every mode in turn behind a device barrier.
// With --verify every rank uses the same inputs, so each destination's bits are known whoever wrote last.
// Ranks are forked by the native launcher; D buffers are shared as cudaIpc handles.
//
// Reference parity: comm_comp/exp3_epilogue_remote.cu (modes :147-156,311-328, timing :185-204, verify
// :366-395, CSV :255-257).  Its two epilogues (TMA store / direct stores) are one here: 16-byte st.global.
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
  std::vector<std::string> shapes = {"8192", "32768x8192x1024"};
  int ndev = 0, iters = 30, warm = 3, cta_group = 2;
  bool verify = false;
  std::string csv_path;
  Args a(argc, argv);
  while (a.more()) {
    std::string f = a.flag(), v;
    auto need = [&]() { if (!a.value(&v)) std::exit(1); return v; };
    if (f == "--sizes") shapes = split_csv(need());
    else if (f == "--ndev") ndev = std::atoi(need().c_str());
    else if (f == "--iters") iters = std::atoi(need().c_str());
    else if (f == "--warmup") warm = std::atoi(need().c_str());
    else if (f == "--cta-group") cta_group = std::atoi(need().c_str());
    else if (f == "--verify") verify = true;
    else if (f == "--csv") csv_path = need();
    else {
      std::printf("usage: %s [--sizes LIST(N|MxNxK)] [--ndev W] [--iters I] [--warmup W] [--cta-group 1|2] [--verify] [--csv FILE]\n", argv[0]);
      return f == "-h" || f == "--help" ? 0 : 1;
    }
  }
  const int have = Launcher::probe_device_count();
  const int world = ndev > 0 ? ndev : have;
  if (world < 1 || world > have || world > TCL_MAX_WORLD) { std::fprintf(stderr, "need %d GPUs, have %d\n", world, have); return 1; }
  std::vector<Shape3> shp;
  size_t max_mn = 0, max_mk = 0, max_nk = 0;
  for (auto& s : shapes) {
    Shape3 x;
    if (!parse_shape(s, &x) || x.m % (128 * cta_group) || x.n % 256 || x.k % 8) { std::fprintf(stderr, "bad shape %s\n", s.c_str()); return 1; }
    shp.push_back(x);
    max_mn = std::max(max_mn, size_t(x.m) * x.n); max_mk = std::max(max_mk, size_t(x.m) * x.k); max_nk = std::max(max_nk, size_t(x.n) * x.k);
  }
  Launcher L;
  const int rank = L.init(world);
  if (rank < 0) return 2;
  if (cudaSetDevice(rank) != cudaSuccess) die(L, "cudaSetDevice");
  Buf D, bar_d;
  void *A, *B, *ref;
  int32_t* status;
  unsigned long long* diff;
  TCL_CUDA_CHECK(cudaMalloc(&D.local, max_mn * 2));
  TCL_CUDA_CHECK(cudaMalloc(&ref, max_mn * 2));
  TCL_CUDA_CHECK(cudaMalloc(&A, max_mk * 2));
  TCL_CUDA_CHECK(cudaMalloc(&B, max_nk * 2));
  TCL_CUDA_CHECK(cudaMalloc(&bar_d.local, 128));
  TCL_CUDA_CHECK(cudaMemset(bar_d.local, 0, 128));
  TCL_CUDA_CHECK(cudaMalloc(&status, 64));
  TCL_CUDA_CHECK(cudaMemset(status, 0, 64));
  TCL_CUDA_CHECK(cudaMalloc(&diff, 8));
  cudaStream_t st;
  TCL_CUDA_CHECK(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking));
  if (!share(L, 0, D) || !share(L, 1, bar_d)) die(L, "handle exchange failed");
  DeviceBarrier bar;
  bar.world = world; bar.rank = rank; bar.status = status + 8;
  for (int s = 0; s < world; ++s) bar.ptrs[s] = static_cast<int32_t*>(bar_d.peer[s]);
  cudaEvent_t e0, e1;
  TCL_CUDA_CHECK(cudaEventCreate(&e0));
  TCL_CUDA_CHECK(cudaEventCreate(&e1));
  const int peer = (rank + 1) % world;
  Csv csv;
  if (rank == 0) {
    csv.open(csv_path, "m,n,k,epi,mode,peer,iter_us,iter_p95,slowdown,tflops,d_write_gbps,verify,max_over_ranks_us,nccl_cublas_us,speedup,roofline_us,pct_roofline,dtype");
    std::printf("# exp3 epilogue remote write (native launcher) world=%d cta_group=%d iters=%d\n", world, cta_group, iters);
    std::printf("          shape mode           |  iter us |  TF/s | slowdown | D write GB/s | verify\n");
  }
  int rc = 0;
  const char* mode_names[4] = {"local", "remote", "scatter-local", "scatter"};
  for (const Shape3& x : shp) {
    const int M = x.m, N = x.n, K = x.k;
    const int nseg = (world > 1 && M % (world * 128 * cta_group) == 0) ? world : 1;
    const int seg = M / nseg;
    tcl_fill_normal_bf16(A, int64_t(M) * K, 31 + (verify ? 0 : rank), 0.f, 1.f, st);
    tcl_fill_normal_bf16(B, int64_t(N) * K, 41 + (verify ? 0 : rank), 0.f, 1.f, st);
    TCL_CUDA_CHECK(cudaStreamSynchronize(st));
    char err[256];
    void* plans[4] = {};
    int epochs[4] = {};
    for (int m = 0; m < 4; ++m) {
      if ((m == 1 && world == 1) || (m >= 2 && nseg == 1)) continue;
      tcl_gemm_desc d;
      std::memset(&d, 0, sizeof(d));
      d.mode = TCL_MODE_PLAIN; d.cta_group = cta_group; d.M = M; d.N = N; d.K = K; d.lda = K; d.ldb = K; d.ldc = N; d.A = A; d.B = B;
      d.world = 1; d.status = status;
      if (m < 2) { d.seg_rows = M; d.dst_base[0] = m == 0 ? D.local : D.peer[peer]; }
      else {
        d.seg_rows = seg;
        for (int s = 0; s < nseg; ++s) d.dst_base[s] = static_cast<char*>(m == 2 ? D.local : D.peer[s]) + size_t(s) * seg * N * 2;
      }
      plans[m] = tcl_gemm_plan_create(&d, err, sizeof(err));
      if (!plans[m]) die(L, err);
    }
    std::vector<double> us[4];
    if (!L.barrier()) die(L, "peer failed");
    for (int it = 0; it < warm + iters; ++it) {
      if (L.failed()) die(L, "a peer failed during timing");
      for (int m = 0; m < 4; ++m) {
        if (!plans[m]) continue;
        const double t = timed_run(plans[m], &epochs[m], bar, st, e0, e1);
        if (t < 0) die(L, "launch failed");
        if (it >= warm) us[m].push_back(t);
      }
      L.beat();
    }
    // Verification: the local result is the reference; every other mode must leave the same bits where it wrote.
    bool ok[4] = {true, true, true, true};
    if (verify) {
      bar.run(st);
      tcl_gemm_plan_run(plans[0], ++epochs[0], st);
      TCL_CUDA_CHECK(cudaMemcpyAsync(ref, D.local, size_t(M) * N * 2, cudaMemcpyDeviceToDevice, st));
      for (int m = 1; m < 4; ++m) {
        if (!plans[m]) continue;
        TCL_CUDA_CHECK(cudaMemsetAsync(D.local, 0, size_t(M) * N * 2, st));
        TCL_CUDA_CHECK(cudaStreamSynchronize(st));
        if (!L.barrier()) die(L, "peer failed");
        tcl_gemm_plan_run(plans[m], ++epochs[m], st);
        TCL_CUDA_CHECK(cudaStreamSynchronize(st));
        if (!L.barrier()) die(L, "peer failed");
        // remote: the previous rank filled my whole D; scatter: every rank filled my segment; scatter-local: I did
        const size_t off = m == 3 ? size_t(rank) * seg * N * 2 : 0;
        const size_t bytes = m == 3 ? size_t(seg) * N * 2 : size_t(M) * N * 2;
        TCL_CUDA_CHECK(cudaMemsetAsync(diff, 0, 8, st));
        count_diff_kernel<<<1024, 256, 0, st>>>(reinterpret_cast<const uint4*>(static_cast<char*>(D.local) + off), reinterpret_cast<const uint4*>(static_cast<char*>(ref) + off), bytes / 16, diff);
        unsigned long long h = 1;
        TCL_CUDA_CHECK(cudaMemcpyAsync(&h, diff, 8, cudaMemcpyDeviceToHost, st));
        TCL_CUDA_CHECK(cudaStreamSynchronize(st));
        ok[m] = h == 0;
        if (!L.barrier()) die(L, "peer failed");
      }
    }
    int hst[16];
    TCL_CUDA_CHECK(cudaMemcpy(hst, status, 64, cudaMemcpyDeviceToHost));
    if (hst[0] || hst[8]) die(L, "a device wait ran out");
    double* res = L.shm()->results[rank];
    for (int m = 0; m < 4; ++m) { Stats s = make_stats(us[m]); res[3 * m] = s.mean; res[3 * m + 1] = s.p95; res[3 * m + 2] = ok[m] ? 0 : 1; }
    if (!L.barrier()) die(L, "peer failed");
    if (rank == 0) {
      const double flop = 2.0 * M * N * K;
      double base = 0;
      for (int r = 0; r < world; ++r) base = std::max(base, L.shm()->results[r][0]);
      for (int m = 0; m < 4; ++m) {
        if (!plans[m]) continue;
        double mean = 0, p95 = 0, bad = 0;
        for (int r = 0; r < world; ++r) { mean = std::max(mean, L.shm()->results[r][3 * m]); p95 = std::max(p95, L.shm()->results[r][3 * m + 1]); bad += L.shm()->results[r][3 * m + 2]; }
        const char* ver = !verify || m == 0 ? "-" : bad ? "FAIL" : "ok";
        if (bad) rc = 4;
        std::printf("%6dx%5dx%5d %-14s | %8.1f | %5.0f | %8.3f | %12.1f | %s\n", M, N, K, mode_names[m], mean, flop / mean / 1e6, mean / base, double(M) * N * 2 / mean / 1e3, ver);
        csv.row("%d,%d,%d,st16,%s,%d,%.2f,%.2f,%.4f,%.1f,%.2f,%s,%.2f,,,,,bf16", M, N, K, mode_names[m], peer, mean, p95, mean / base, flop / mean / 1e6, double(M) * N * 2 / mean / 1e3, ver, mean);
      }
    }
    if (!L.barrier()) die(L, "peer failed");
    for (int m = 0; m < 4; ++m) if (plans[m]) tcl_gemm_plan_destroy(plans[m]);
  }
  TCL_CUDA_CHECK(cudaDeviceSynchronize());
  if (!L.barrier()) rc = rc ? rc : 5;
  unshare(L, D);
  unshare(L, bar_d);
  L.barrier();
  if (rank != 0) _exit(rc);
  const int worst = L.wait_children(30.0);
  return rc ? rc : worst;
}
