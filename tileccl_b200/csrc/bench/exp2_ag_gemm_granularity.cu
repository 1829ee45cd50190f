// exp2_ag_gemm_granularity (native driver): all-gather -> GEMM at several gather granularities,
// ranks forked by the native launcher, buffers shared as cudaIpc handles, kernels through the C
// interface of the library.  Per granularity (rows per gather tile):
//   t_full  one plain GEMM on a pre-gathered A            t_seg  the fused kernel with communication off
//   t_ovl   the fused kernel pulling the peers' shards    seg_eff = t_full / t_seg, overlap_eff = t_seg / t_ovl
// Verification scrubs the peers' rows of the gathered buffer with 0x55, runs the dependent pipeline once and
// compares its output bit-wise with the pre-gathered run.
//
// --modes fused,ce adds the reference's own design as the measured alternative: the gathered A is cut in
// world x S row chunks (--chunks S, or --gather-rows), every remote chunk is one copy-engine peer copy on
// one of --comm-streams high-priority streams, and the compute stream launches a pre-built GEMM per chunk as
// soon as the chunk is there (own shard first).  Pull (default): the consumer issues the copies and waits on
// their events.  --push: every rank copies its own shard into the peers' buffers and raises a flag per chunk
// from its copy stream; the consumer's compute stream runs a one-thread kernel that waits (with a limit) for
// the flag.  t_comm is the transfers alone.  (The Python driver of the same name also has the NCCL mode.)
//
// Reference parity: comm_comp/exp2_ag_gemm_granularity.cu (flags :104-108, pipeline :168-300, verify :511-533,
// CSV :446-448).  There one process drives every GPU and only one rank computes; here every rank computes.
#include <string>

#include "../ptx/ldst_sys.cuh"
#include "../ptx/mbarrier.cuh"
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

// Push form of the copy-engine pipeline: the source's copy stream raises the chunk's flag at the consumer after
// the chunk's copy; the consumer's compute stream waits for it, with a limit, ahead of the chunk's GEMM.
__global__ void set_flag_kernel(int* flag, int value) { tcl::ptx::st_release_sys(flag, value); }
__global__ void wait_flag_kernel(const int* flag, int value, int* status, unsigned long long timeout_ns) {
  const unsigned long long deadline = tcl::ptx::globaltimer_ns() + timeout_ns;
  int seen = 0;
  if (!tcl::ptx::wait_ge<true>(flag, value, nullptr, deadline, &seen)) {
    if (atomicCAS(status, 0, 7) == 0) { status[1] = 0; status[2] = value; status[3] = seen; }   // 7: a gathered chunk never arrived
  }
}

struct CeChunk {
  int src = 0, chunk = 0;     // source rank, chunk index inside its shard
  size_t row0 = 0;
  void* plan = nullptr;
  cudaEvent_t ev = nullptr;   // pull: the chunk's copy is done
};

int main(int argc, char** argv) {
  int M = 32768, K = 8192, N = 0, n_global = 28672, ndev = 0, iters = 20, warm = 3, cta_group = 2, comm_streams = 1;
  std::vector<int> grains, chunk_counts;
  bool verify = false, push = false;
  std::string csv_path, modes = "fused";
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
    else if (f == "--modes") modes = need();
    else if (f == "--chunks") parse_int_list(need(), &chunk_counts);
    else if (f == "--comm-streams") comm_streams = std::max(1, std::atoi(need().c_str()));
    else if (f == "--push") push = true;
    else {
      std::printf("usage: %s [--m M] [--k K] [--n N_local | --n-global N] [--gather-rows LIST | --chunks LIST] [--modes fused,ce] [--comm-streams N] [--push]\n"
                  "          [--ndev W] [--iters I] [--warmup W] [--cta-group 1|2] [--verify] [--csv FILE]\n", argv[0]);
      return f == "-h" || f == "--help" ? 0 : 1;
    }
  }
  const int have = Launcher::probe_device_count();
  const int world = ndev > 0 ? ndev : have;
  if (world < 1 || world > have || world > TCL_MAX_WORLD) { std::fprintf(stderr, "need %d GPUs, have %d\n", world, have); return 1; }
  if (N <= 0) N = n_global / world;
  const int seg = M / world;
  if (M % (world * 128 * cta_group) || N % 256 || K % 8) { std::fprintf(stderr, "shape not supported\n"); return 1; }
  for (int S : chunk_counts) if (S > 0 && seg % S == 0) grains.push_back(seg / S);     // --chunks S: S chunks per shard
  if (grains.empty()) grains = {128, 512, 2048, 4096};
  bool do_fused = false, do_ce = false;
  for (auto& m : split_csv(modes)) {
    if (m == "fused") do_fused = true;
    else if (m == "ce") do_ce = true;
    else { std::fprintf(stderr, "--modes: unknown mode %s (fused, ce)\n", m.c_str()); return 1; }
  }

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
  // ---- copy-engine pipeline (the reference's design) ----
  std::vector<cudaStream_t> comm(comm_streams);
  {
    int lo = 0, hi = 0;
    TCL_CUDA_CHECK(cudaDeviceGetStreamPriorityRange(&lo, &hi));
    for (auto& c : comm) TCL_CUDA_CHECK(cudaStreamCreateWithPriority(&c, cudaStreamNonBlocking, hi));
  }
  cudaEvent_t gate, comm_done;
  TCL_CUDA_CHECK(cudaEventCreateWithFlags(&gate, cudaEventDisableTiming));
  TCL_CUDA_CHECK(cudaEventCreateWithFlags(&comm_done, cudaEventDisableTiming));
  int ce_epoch = 0;
  auto chunk_plan = [&](size_t row0, int rows) {
    tcl_gemm_desc d;
    std::memset(&d, 0, sizeof(d));
    d.mode = TCL_MODE_PLAIN; d.cta_group = (rows % (128 * cta_group) == 0) ? cta_group : 1; d.M = rows; d.N = N; d.K = K; d.lda = K; d.ldb = K; d.ldc = N;
    d.A = static_cast<char*>(afull.local) + row0 * K * 2; d.B = B;
    d.world = 1; d.seg_rows = rows; d.dst_base[0] = static_cast<char*>(out) + row0 * N * 2; d.status = status;
    void* p = tcl_gemm_plan_create(&d, err, sizeof(err));
    if (!p) die(L, err);
    return p;
  };
  // One pass of the pipeline on stream st.  comm / compute select the transfers and the GEMMs.
  auto ce_run = [&](std::vector<CeChunk>& chunks, int g, bool with_comm, bool with_compute, std::vector<int>& epochs) {
    const int S = seg / g;
    const size_t bytes = size_t(g) * K * 2;
    int32_t* my_flags = static_cast<int32_t*>(flags.local);
    if (with_comm) {
      ++ce_epoch;
      TCL_CUDA_CHECK(cudaEventRecord(gate, st));
      for (auto& c : comm) TCL_CUDA_CHECK(cudaStreamWaitEvent(c, gate, 0));   // this pass's transfers start when the previous pass is done
      int k = 0;
      if (!push) {
        for (auto& ch : chunks) {
          if (ch.src == rank) continue;
          cudaStream_t cs = comm[k++ % comm_streams];
          TCL_CUDA_CHECK(cudaMemcpyAsync(static_cast<char*>(afull.local) + ch.row0 * K * 2, static_cast<char*>(afull.peer[ch.src]) + ch.row0 * K * 2, bytes,
                                         cudaMemcpyDefault, cs));
          TCL_CUDA_CHECK(cudaEventRecord(ch.ev, cs));
        }
      } else {
        for (int c = 0; c < S; ++c)
          for (int i = 1; i < world; ++i) {
            const int peer = (rank + i) % world;
            const size_t off = (size_t(rank) * seg + size_t(c) * g) * K * 2;
            cudaStream_t cs = comm[k++ % comm_streams];
            TCL_CUDA_CHECK(cudaMemcpyAsync(static_cast<char*>(afull.peer[peer]) + off, static_cast<char*>(afull.local) + off, bytes, cudaMemcpyDefault, cs));
            set_flag_kernel<<<1, 1, 0, cs>>>(static_cast<int32_t*>(flags.peer[peer]) + rank * S + c, ce_epoch);
          }
      }
    }
    if (with_compute) {
      size_t i = 0;
      for (auto& ch : chunks) {
        if (with_comm && ch.src != rank) {
          if (!push) TCL_CUDA_CHECK(cudaStreamWaitEvent(st, ch.ev, 0));
          else wait_flag_kernel<<<1, 1, 0, st>>>(my_flags + ch.src * S + ch.chunk, ce_epoch, status, 4000000000ull);
        }
        if (tcl_gemm_plan_run(ch.plan, ++epochs[i++], st) != 0) die(L, "launch failed");
      }
    } else if (with_comm) {
      if (push) {
        for (auto& ch : chunks)
          if (ch.src != rank) wait_flag_kernel<<<1, 1, 0, st>>>(my_flags + ch.src * S + ch.chunk, ce_epoch, status, 4000000000ull);
      }
    }
    if (with_comm) {
      // the pass ends when this rank's own transfers have ended too (they read or write a peer's buffer)
      for (auto& c : comm) { TCL_CUDA_CHECK(cudaEventRecord(comm_done, c)); TCL_CUDA_CHECK(cudaStreamWaitEvent(st, comm_done, 0)); }
    }
  };
  auto ce_timed = [&](std::vector<CeChunk>& chunks, int g, bool with_comm, bool with_compute, std::vector<int>& epochs) {
    bar.run(st);
    TCL_CUDA_CHECK(cudaEventRecord(e0, st));
    ce_run(chunks, g, with_comm, with_compute, epochs);
    TCL_CUDA_CHECK(cudaEventRecord(e1, st));
    TCL_CUDA_CHECK(cudaEventSynchronize(e1));
    return elapsed_us(e0, e1);
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
    if (do_ce) {
      const int S = seg / g;
      std::vector<CeChunk> chunks;
      auto add = [&](int src, int c) {
        CeChunk ch;
        ch.src = src; ch.chunk = c; ch.row0 = size_t(src) * seg + size_t(c) * g;
        ch.plan = chunk_plan(ch.row0, g);
        if (src != rank) TCL_CUDA_CHECK(cudaEventCreateWithFlags(&ch.ev, cudaEventDisableTiming));
        chunks.push_back(ch);
      };
      for (int c = 0; c < S; ++c) add(rank, c);                                    // the own shard needs no transfer: first
      if (!push) { for (int i = 1; i < world; ++i) for (int c = 0; c < S; ++c) add((rank + i) % world, c); }   // pull: one peer after the other
      else { for (int c = 0; c < S; ++c) for (int i = 1; i < world; ++i) add((rank + world - i) % world, c); } // push: all shards arrive at the same rate
      std::vector<int> epochs(chunks.size(), 0);
      const char* cver = "-";
      if (verify) {
        tcl_gemm_plan_run(full, ++ep_full, st);
        TCL_CUDA_CHECK(cudaMemsetAsync(afull.local, 0x55, size_t(rank) * seg * K * 2, st));
        TCL_CUDA_CHECK(cudaMemsetAsync(shard + size_t(seg) * K * 2, 0x55, size_t(world - 1 - rank) * seg * K * 2, st));
        TCL_CUDA_CHECK(cudaMemsetAsync(out, 0, mn * 2, st));
        TCL_CUDA_CHECK(cudaStreamSynchronize(st));
        if (!L.barrier()) die(L, "peer failed");
        bar.run(st);
        ce_run(chunks, g, true, true, epochs);
        TCL_CUDA_CHECK(cudaMemsetAsync(diff, 0, 8, st));
        count_diff_kernel<<<1024, 256, 0, st>>>(static_cast<const uint4*>(out), static_cast<const uint4*>(out_ref), mn * 2 / 16, diff);
        unsigned long long h = 1;
        TCL_CUDA_CHECK(cudaMemcpyAsync(&h, diff, 8, cudaMemcpyDeviceToHost, st));
        TCL_CUDA_CHECK(cudaStreamSynchronize(st));
        cver = h == 0 ? "ok" : "FAIL";
        if (h) rc = 4;
        if (!L.barrier()) die(L, "peer failed");
      }
      // t_seg needs the gathered rows in place
      TCL_CUDA_CHECK(cudaMemcpyAsync(afull.local, gathered, size_t(rank) * seg * K * 2, cudaMemcpyDefault, st));
      TCL_CUDA_CHECK(cudaMemcpyAsync(shard + size_t(seg) * K * 2, static_cast<char*>(gathered) + size_t(rank + 1) * seg * K * 2, size_t(world - 1 - rank) * seg * K * 2, cudaMemcpyDefault, st));
      TCL_CUDA_CHECK(cudaStreamSynchronize(st));
      if (!L.barrier()) die(L, "peer failed");
      std::vector<double> tf, ts, to, tc;
      for (int it = 0; it < warm + iters; ++it) {
        if (L.failed()) die(L, "a peer failed during timing");
        const double a0 = timed_run(full, &ep_full, bar, st, e0, e1);
        const double a1 = ce_timed(chunks, g, false, true, epochs);
        const double a2 = ce_timed(chunks, g, true, true, epochs);
        const double a3 = (it % 3 == 0) ? ce_timed(chunks, g, true, false, epochs) : -1;
        if (a0 < 0) die(L, "launch failed");
        if (it >= warm) { tf.push_back(a0); ts.push_back(a1); to.push_back(a2); if (a3 >= 0) tc.push_back(a3); }
        L.beat();
      }
      int hst[16];
      TCL_CUDA_CHECK(cudaMemcpy(hst, status, 64, cudaMemcpyDeviceToHost));
      if (hst[0] || hst[8]) { std::fprintf(stderr, "rank %d: %s\n", rank, tcl_status_string(hst[0] ? hst[0] : hst[8])); die(L, "a device wait ran out"); }
      double* res = L.shm()->results[rank];
      res[0] = make_stats(tf).mean; res[1] = make_stats(ts).mean; res[2] = make_stats(to).mean; res[3] = std::strcmp(cver, "FAIL") == 0; res[4] = make_stats(tc).mean;
      if (!L.barrier()) die(L, "peer failed");
      if (rank == 0) {
        double f = 0, sg = 0, o = 0, cm = 0, bad = 0;
        for (int r = 0; r < world; ++r) {
          const double* q = L.shm()->results[r];
          f = std::max(f, q[0]); sg = std::max(sg, q[1]); o = std::max(o, q[2]); cm = std::max(cm, q[4]); bad += q[3];
        }
        const double flop = 2.0 * M * N * K;
        if (bad) { cver = "FAIL"; rc = 4; }
        const double gbps = cm > 0 ? double(world - 1) * seg * K * 2 / (cm * 1e-6) / 1e9 : 0.0;
        const double ovl_eff = o > 0 ? std::max(sg, cm) / o : 0.0;
        std::printf("%5d %10d | %10.1f %10.1f %10.1f | %7.3f %7.3f | %8.0f | %s   (%s, %d stream%s, t_comm %.1f us = %.0f GB/s)\n", S, g, f, sg, o, f / sg, ovl_eff,
                    flop / o / 1e6, cver, push ? "ce push" : "ce pull", comm_streams, comm_streams > 1 ? "s" : "", cm, gbps);
        csv.row("%d,%d,%d,%d,%d,%d,%.2f,%s,%d,%.2f,%.2f,%.2f,%.2f,%.4f,%.1f,%.4f,%.1f,%s,%.2f,,,,,bf16", M, N, K, world, S, g, double(g) * K * 2 / 1048576.0,
                push ? "ce_push" : "ce", comm_streams, f, sg, cm, o, f / sg, gbps, ovl_eff, flop / o / 1e6, cver, o);
      }
      if (!L.barrier()) die(L, "peer failed");
      for (auto& ch : chunks) { tcl_gemm_plan_destroy(ch.plan); if (ch.ev) cudaEventDestroy(ch.ev); }
      // the fused mode below expects clean counters
      TCL_CUDA_CHECK(cudaMemset(flags.local, 0, (M / 128 + 32) * 4));
      TCL_CUDA_CHECK(cudaDeviceSynchronize());
      if (!L.barrier()) die(L, "peer failed");
    }
    if (!do_fused) continue;
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
