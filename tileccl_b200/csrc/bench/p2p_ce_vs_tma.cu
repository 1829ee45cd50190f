// p2p_ce_vs_tma: moving a [tokens x hidden] activation block to a peer, nine ways.
//   ce / ce_pull        copy engine, issued for the source / the destination device's stream
//   sm / sm_pull        16-byte ld/st kernel running on the source (push) / destination (pull) GPU
//   tma / tma_pull      bulk-copy ring through shared memory, push / pull
//   tma_store           shared memory -> peer only (upper bound for a fused producer)
//   tma_load            peer -> shared memory only (model of a fused consumer)
//   sm_load             peer -> shared memory with 16-byte ld.global + st.shared (the same model on the register path)
// Reports the average time of back-to-back transfers, the p50 / p99 of single transfers, GB/s, and a
// host-side comparison of the destination (not for tma_store / tma_load / sm_load, which move no complete copy).
//
// Reference parity: tests/p2p_ce_vs_tma.cu (kernels :185-360, timing :483-550, tile plan :553-600,
// table :873-879).  --csv is added here: method,tokens,hidden,bytes,avg_us,p50_us,p99_us,gbps,verify.
#include <string>
#include <vector>

#include "../common/host_common.hpp"
#include "movers.cuh"

using namespace tcl::host;
using namespace tcl::bench;

int main(int argc, char** argv) {
  std::vector<int> tokens = {1, 4, 16, 64, 256, 1024, 4096};
  int hidden = 7168, elt = 2, tile_tokens = 0, stages = 4, blocks = 0, iters = 100, warmup = 20, src = 0, dst = 1;
  std::vector<std::string> methods = {"ce", "ce_pull", "sm", "sm_pull", "tma", "tma_pull", "tma_store", "tma_load", "sm_load"};
  bool check = true;
  std::string csv_path, dtype = "bf16";
  Args a(argc, argv);
  while (a.more()) {
    std::string f = a.flag(), v;
    auto need = [&]() { if (!a.value(&v)) std::exit(1); return v; };
    if (f == "--tokens") parse_int_list(need(), &tokens);
    else if (f == "--hidden") hidden = std::atoi(need().c_str());
    else if (f == "--dtype") { dtype = need(); elt = dtype == "fp32" ? 4 : dtype == "fp8" ? 1 : 2; }
    else if (f == "--tile-tokens") tile_tokens = std::atoi(need().c_str());
    else if (f == "--stages") stages = std::atoi(need().c_str());
    else if (f == "--blocks") blocks = std::atoi(need().c_str());
    else if (f == "--iters") iters = std::atoi(need().c_str());
    else if (f == "--warmup") warmup = std::atoi(need().c_str());
    else if (f == "--src") src = std::atoi(need().c_str());
    else if (f == "--dst") dst = std::atoi(need().c_str());
    else if (f == "--methods") methods = split_csv(need());
    else if (f == "--no-check") check = false;
    else if (f == "--csv") csv_path = need();
    else {
      std::printf("usage: %s [--tokens LIST] [--hidden N] [--dtype bf16|fp16|fp32|fp8] [--tile-tokens N] [--stages 3|4|6|8] [--blocks N]\n"
                  "          [--iters N] [--warmup N] [--src N] [--dst N] [--methods LIST] [--no-check] [--csv FILE]\n", argv[0]);
      return f == "-h" || f == "--help" ? 0 : 1;
    }
  }
  if (stages != 3 && stages != 4 && stages != 6 && stages != 8) stages = 4;
  const int ndev = device_count();
  if (src >= ndev || dst >= ndev) { std::fprintf(stderr, "need GPUs %d and %d, have %d\n", src, dst, ndev); return 1; }
  if (src != dst && !enable_peer_all(std::max(src, dst) + 1)) return 1;
  const size_t row = static_cast<size_t>(hidden) * elt;
  if (row % 16) { std::fprintf(stderr, "hidden * element size must be a multiple of 16 bytes\n"); return 1; }
  int max_tok = 0;
  for (int t : tokens) max_tok = std::max(max_tok, t);
  const size_t max_bytes = row * max_tok;
  char *buf_s, *buf_d;
  int *err_s, *err_d;
  cudaStream_t st[2];
  cudaEvent_t e0[2], e1[2];
  const int devs[2] = {src, dst};
  TCL_CUDA_CHECK(cudaSetDevice(dst));
  TCL_CUDA_CHECK(cudaMalloc(&buf_d, max_bytes));
  TCL_CUDA_CHECK(cudaMalloc(&err_d, 4));
  unsigned* sink_d = nullptr;
  TCL_CUDA_CHECK(cudaMalloc(&sink_d, 4));
  TCL_CUDA_CHECK(cudaMemset(err_d, 0, 4));
  TCL_CUDA_CHECK(cudaSetDevice(src));
  TCL_CUDA_CHECK(cudaMalloc(&buf_s, max_bytes));
  TCL_CUDA_CHECK(cudaMalloc(&err_s, 4));
  TCL_CUDA_CHECK(cudaMemset(err_s, 0, 4));
  fill_pattern_kernel<<<1024, 256>>>(reinterpret_cast<uint32_t*>(buf_s), max_bytes / 4, 99u);
  TCL_CUDA_CHECK(cudaDeviceSynchronize());
  for (int k = 0; k < 2; ++k) {
    TCL_CUDA_CHECK(cudaSetDevice(devs[k]));
    TCL_CUDA_CHECK(cudaStreamCreateWithFlags(&st[k], cudaStreamNonBlocking));
    TCL_CUDA_CHECK(cudaEventCreate(&e0[k]));
    TCL_CUDA_CHECK(cudaEventCreate(&e1[k]));
  }
  cudaDeviceProp prop;
  TCL_CUDA_CHECK(cudaGetDeviceProperties(&prop, src));
  const int sms = prop.multiProcessorCount;
  const size_t smem_budget = (prop.sharedMemPerBlockOptin - 8 * stages) / stages / 128 * 128;
  print_device_line(src);
  std::printf("# p2p_ce_vs_tma src=%d dst=%d hidden=%d dtype=%s row=%zu B stages=%d iters=%d\n", src, dst, hidden, dtype.c_str(), row, stages, iters);
  Csv csv;
  if (!csv.open(csv_path, "method,tokens,hidden,bytes,avg_us,p50_us,p99_us,gbps,verify")) return 1;
  std::printf("%-10s %7s %12s | %10s %10s %10s %10s | %s\n", "method", "tokens", "bytes", "avg_us", "p50_us", "p99_us", "GB/s", "verify");
  std::vector<char> host_s(max_bytes), host_d(max_bytes);
  TCL_CUDA_CHECK(cudaMemcpy(host_s.data(), buf_s, max_bytes, cudaMemcpyDeviceToHost));

  for (int tok : tokens) {
    const size_t bytes = row * tok;
    // Tile = k whole tokens that fit a shared-memory slot (or a slice of a row when one token does not fit).
    size_t tile = tile_tokens > 0 ? row * tile_tokens : std::max<size_t>(row, smem_budget / row * row);
    if (tile > smem_budget) tile = smem_budget / 16 * 16;
    if (tile > bytes) tile = bytes;
    for (auto& m : methods) {
      const bool pull = m == "ce_pull" || m == "sm_pull" || m == "tma_pull" || m == "tma_load" || m == "sm_load";
      const int k = pull ? 1 : 0;  // which device runs the transfer
      int* err = pull ? err_d : err_s;
      TCL_CUDA_CHECK(cudaSetDevice(dst));
      TCL_CUDA_CHECK(cudaMemset(buf_d, 0, bytes));
      TCL_CUDA_CHECK(cudaDeviceSynchronize());
      TCL_CUDA_CHECK(cudaSetDevice(devs[k]));
      const int nb = blocks > 0 ? blocks : static_cast<int>(std::min<size_t>(sms, std::max<size_t>(1, bytes / tile)));
      auto once = [&]() {
        if (m == "ce" || m == "ce_pull") {
          TCL_CUDA_CHECK(cudaMemcpyPeerAsync(buf_d, dst, buf_s, src, bytes, st[k]));
        } else if (m == "sm" || m == "sm_pull") {
          const int b = static_cast<int>(std::min<size_t>(4 * sms, (bytes / 16 + 255) / 256));
          flat_copy_kernel<<<std::max(1, b), 256, 0, st[k]>>>(reinterpret_cast<const uint4*>(buf_s), reinterpret_cast<uint4*>(buf_d), bytes / 16);
        } else if (m == "sm_load") {
          TCL_CUDA_CHECK(launch_ldst_load_only(nb, st[k], buf_s, bytes / 16 * 16, static_cast<uint32_t>(tile / 16 * 16), sink_d));
        } else {
          const int kind = m == "tma_store" ? kBulkStoreOnly : m == "tma_load" ? kBulkLoadOnly : kBulkCopy;
          TCL_CUDA_CHECK(launch_bulk_pipe(stages, nb, st[k], buf_s, buf_d, bytes, static_cast<uint32_t>(tile), kind, err, 2000000000ull));
        }
      };
      for (int i = 0; i < warmup; ++i) once();
      TCL_CUDA_CHECK(cudaStreamSynchronize(st[k]));
      TCL_CUDA_CHECK(cudaEventRecord(e0[k], st[k]));
      for (int i = 0; i < iters; ++i) once();
      TCL_CUDA_CHECK(cudaEventRecord(e1[k], st[k]));
      TCL_CUDA_CHECK(cudaStreamSynchronize(st[k]));
      const double avg = elapsed_us(e0[k], e1[k]) / iters;
      std::vector<double> lat;
      for (int i = 0; i < iters; ++i) {
        TCL_CUDA_CHECK(cudaEventRecord(e0[k], st[k]));
        once();
        TCL_CUDA_CHECK(cudaEventRecord(e1[k], st[k]));
        TCL_CUDA_CHECK(cudaStreamSynchronize(st[k]));
        lat.push_back(elapsed_us(e0[k], e1[k]));
      }
      Stats s = make_stats(lat);
      int herr = 0;
      TCL_CUDA_CHECK(cudaMemcpy(&herr, err, 4, cudaMemcpyDeviceToHost));
      const char* ver = "-";
      if (herr) ver = "TIMEOUT";
      else if (check && m != "tma_store" && m != "tma_load" && m != "sm_load") {
        TCL_CUDA_CHECK(cudaMemcpy(host_d.data(), buf_d, bytes, cudaMemcpyDeviceToHost));
        ver = std::memcmp(host_d.data(), host_s.data(), bytes) == 0 ? "ok" : "FAIL";
      }
      const double gbps = bytes / avg / 1e3;
      std::printf("%-10s %7d %12zu | %10.2f %10.2f %10.2f %10.1f | %s\n", m.c_str(), tok, bytes, avg, s.p50, s.p99, gbps, ver);
      csv.row("%s,%d,%d,%zu,%.3f,%.3f,%.3f,%.2f,%s", m.c_str(), tok, hidden, bytes, avg, s.p50, s.p99, gbps, ver);
      if (herr) return 3;
    }
  }
  return 0;
}
