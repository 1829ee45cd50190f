// pipeline_e2e: a synthetic producer -> transfer -> consumer pipeline across two GPUs, measured
// against the max() cost model.
//   producer (source GPU): `intensity` FMAs per float, tile by tile
//   transfer: ce   the whole payload in `chunks` copy-engine copies, each followed by an event the
//                  consumer's stream waits on
//             ldst the producer stores each tile straight into the destination GPU and publishes a
//                  per-tile flag with st.release.sys
//             tma  the producer computes into shared memory and sends the tile with a bulk store;
//                  the flag of a tile is published one tile later, after its bulk store completed
//   consumer (destination GPU): acquire-polls the tile flag (bounded), runs the same FMA chain,
//                  re-computes element 0 of every tile as a check
// Reports Tc_src (compute alone), Tm (transfer alone), Tc_dst, To (overlapped), pred = max of the
// three, err% = (pred - To) / To.
//
// Reference parity: tests/pipeline_e2e.cu (kernels :140-210, timing :419-455, ce pipeline :457-500,
// loop :511-560, CSV :503-504).
#include <string>
#include <vector>

#include "../common/host_common.hpp"
#include "movers.cuh"

using namespace tcl::host;
namespace ptx = tcl::ptx;

__device__ __forceinline__ float work(float x, int intensity) {
  float a = x;
  for (int i = 0; i < intensity; ++i) a = fmaf(a, 1.0000001f, 0.5f);
  return a;
}
__device__ __forceinline__ float seed_of(size_t i) { return static_cast<float>(i & 1023) * 0.001f; }

// mode 0: compute only into `out` (local); mode 1: compute and store to `out` (peer) + flag per tile.
__global__ void produce_ldst_kernel(float* out, int* flags, size_t tile_floats, size_t n_tiles, int intensity, int publish, int epoch) {
  for (size_t t = blockIdx.x; t < n_tiles; t += gridDim.x) {
    float* o = out + t * tile_floats;
    for (size_t i = threadIdx.x; i < tile_floats; i += blockDim.x) o[i] = work(seed_of(t * tile_floats + i), intensity);
    __syncthreads();
    if (publish && threadIdx.x == 0) ptx::st_release_sys(flags + t, epoch);
  }
}

// Computes into double-buffered shared memory, sends with a bulk store; the flag lags one tile.
__global__ void produce_tma_kernel(float* out, int* flags, size_t tile_floats, size_t n_tiles, int intensity, int epoch) {
  extern __shared__ __align__(128) float sm[];
  long long prev = -1;
  int buf = 0;
  for (size_t t = blockIdx.x; t < n_tiles; t += gridDim.x, buf ^= 1) {
    float* s = sm + buf * tile_floats;
    // The bulk store that last read this buffer (two tiles ago) must have finished reading it.
    if (threadIdx.x == 0) ptx::bulk_wait_read<1>();
    __syncthreads();
    for (size_t i = threadIdx.x; i < tile_floats; i += blockDim.x) s[i] = work(seed_of(t * tile_floats + i), intensity);
    ptx::fence_proxy_async();
    __syncthreads();
    if (threadIdx.x == 0) {
      ptx::bulk_store(out + t * tile_floats, ptx::smem_u32(s), static_cast<uint32_t>(tile_floats * 4));
      ptx::bulk_commit();
      if (prev >= 0) {
        ptx::bulk_wait<1>();  // the previous tile's store is complete
        ptx::fence_sys();
        ptx::st_release_sys(flags + prev, epoch);
      }
      prev = static_cast<long long>(t);
    }
  }
  if (threadIdx.x == 0) {
    ptx::bulk_wait<0>();
    if (prev >= 0) { ptx::fence_sys(); ptx::st_release_sys(flags + prev, epoch); }
  }
}

__global__ void consume_kernel(const float* in, const int* flags, float* sink, size_t tile_floats, size_t n_tiles, int intensity,
                               int prod_intensity, int wait, int epoch, unsigned long long* errors, int* timed_out,
                               unsigned long long timeout_ns) {
  const unsigned long long deadline = ptx::globaltimer_ns() + timeout_ns;
  __shared__ int ok;
  float acc = 0.f;
  for (size_t t = blockIdx.x; t < n_tiles; t += gridDim.x) {
    if (wait) {
      if (threadIdx.x == 0) ok = ptx::wait_ge<true>(flags + t, epoch, nullptr, deadline, nullptr, 128) ? 1 : 0;
      __syncthreads();
      if (!ok) { if (threadIdx.x == 0) atomicExch(timed_out, 1); return; }
    }
    const float* p = in + t * tile_floats;
    for (size_t i = threadIdx.x; i < tile_floats; i += blockDim.x) acc += work(p[i], intensity);
    if (wait && threadIdx.x == 0) {
      const float want = work(seed_of(t * tile_floats), prod_intensity);
      if (p[0] != want) atomicAdd(errors, 1ull);
    }
    __syncthreads();
  }
  if (acc == 12345.678f) sink[0] = acc;
}

int main(int argc, char** argv) {
  std::vector<std::string> methods = {"ce", "ldst", "tma"};
  std::vector<int> intens = {0, 64, 256, 1024, 4096};
  size_t total = size_t(256) << 20, tile = 16384;
  int blocks = 0, chunks = 16, reps = 3, src = 0, dst = 1;
  bool check = true;
  std::string csv_path;
  Args a(argc, argv);
  while (a.more()) {
    std::string f = a.flag(), v;
    auto need = [&]() { if (!a.value(&v)) std::exit(1); return v; };
    if (f == "--methods") methods = split_csv(need());
    else if (f == "--intensity") parse_int_list(need(), &intens);
    else if (f == "--total") parse_bytes(need(), &total);
    else if (f == "--tile") parse_bytes(need(), &tile);
    else if (f == "--blocks") blocks = std::atoi(need().c_str());
    else if (f == "--chunks") chunks = std::atoi(need().c_str());
    else if (f == "--reps") reps = std::atoi(need().c_str());
    else if (f == "--src") src = std::atoi(need().c_str());
    else if (f == "--dst") dst = std::atoi(need().c_str());
    else if (f == "--no-check") check = false;
    else if (f == "--csv") csv_path = need();
    else {
      std::printf("usage: %s [--methods ce,ldst,tma] [--intensity LIST] [--total B] [--tile B] [--blocks N] [--chunks N] [--reps N]\n"
                  "          [--src N] [--dst N] [--no-check] [--csv FILE]\n", argv[0]);
      return f == "-h" || f == "--help" ? 0 : 1;
    }
  }
  const int ndev = device_count();
  if (src == dst || src >= ndev || dst >= ndev) {
    std::fprintf(stderr, "pipeline_e2e needs two different GPUs (producer and consumer wait on one another); have %d\n", ndev);
    return 1;
  }
  if (!enable_peer_all(std::max(src, dst) + 1)) return 1;
  tile = tile / 16 * 16;
  const size_t tile_floats = tile / 4;
  const size_t n_tiles = total / tile;
  total = n_tiles * tile;
  cudaDeviceProp prop;
  TCL_CUDA_CHECK(cudaGetDeviceProperties(&prop, src));
  if (blocks <= 0) blocks = prop.multiProcessorCount;
  print_device_line(src);
  std::printf("# pipeline_e2e src=%d dst=%d total=%zu tile=%zu tiles=%zu blocks=%d\n", src, dst, total, tile, n_tiles, blocks);

  float *stage_s, *buf_d, *sink;
  int *flags_d, *timed_out;
  unsigned long long* errors;
  TCL_CUDA_CHECK(cudaSetDevice(dst));
  TCL_CUDA_CHECK(cudaMalloc(&buf_d, total));
  TCL_CUDA_CHECK(cudaMalloc(&flags_d, n_tiles * 4));
  TCL_CUDA_CHECK(cudaMemset(flags_d, 0, n_tiles * 4));
  TCL_CUDA_CHECK(cudaMalloc(&sink, 64));
  TCL_CUDA_CHECK(cudaMalloc(&errors, 8));
  TCL_CUDA_CHECK(cudaMalloc(&timed_out, 4));
  TCL_CUDA_CHECK(cudaMemset(timed_out, 0, 4));
  cudaStream_t st_d, st_s;
  TCL_CUDA_CHECK(cudaStreamCreateWithFlags(&st_d, cudaStreamNonBlocking));
  cudaEvent_t d0, d1;
  TCL_CUDA_CHECK(cudaEventCreate(&d0));
  TCL_CUDA_CHECK(cudaEventCreate(&d1));
  TCL_CUDA_CHECK(cudaSetDevice(src));
  TCL_CUDA_CHECK(cudaMalloc(&stage_s, total));
  TCL_CUDA_CHECK(cudaStreamCreateWithFlags(&st_s, cudaStreamNonBlocking));
  cudaEvent_t s0, s1;
  TCL_CUDA_CHECK(cudaEventCreate(&s0));
  TCL_CUDA_CHECK(cudaEventCreate(&s1));
  std::vector<cudaEvent_t> chunk_ev(chunks);
  for (auto& e : chunk_ev) TCL_CUDA_CHECK(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
  TCL_CUDA_CHECK(cudaFuncSetAttribute(produce_tma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(2 * tile)));

  Csv csv;
  if (!csv.open(csv_path, "method,intensity,flop_per_byte,Tc_src_ms,Tm_ms,Tc_dst_ms,To_ms,pred_ms,err_pct,errors")) return 1;
  std::printf("%-6s %9s %9s | %9s %9s %9s | %9s %9s %7s | %s\n", "method", "intensity", "flop/B", "Tc_src", "Tm", "Tc_dst", "To", "pred", "err%", "errors");
  int epoch = 0;
  auto min_of = [&](auto fn) { double best = 1e30; for (int r = 0; r < reps; ++r) best = std::min(best, fn()); return best; };

  for (int I : intens) {
    // Stage times, each alone.
    const double tc_src = min_of([&]() {
      TCL_CUDA_CHECK(cudaSetDevice(src));
      TCL_CUDA_CHECK(cudaEventRecord(s0, st_s));
      produce_ldst_kernel<<<blocks, 256, 0, st_s>>>(stage_s, nullptr, tile_floats, n_tiles, I, 0, 0);
      TCL_CUDA_CHECK(cudaEventRecord(s1, st_s));
      TCL_CUDA_CHECK(cudaStreamSynchronize(st_s));
      return elapsed_us(s0, s1) / 1000.0;
    });
    const double tc_dst = min_of([&]() {
      TCL_CUDA_CHECK(cudaSetDevice(dst));
      TCL_CUDA_CHECK(cudaEventRecord(d0, st_d));
      consume_kernel<<<blocks, 256, 0, st_d>>>(buf_d, flags_d, sink, tile_floats, n_tiles, I, I, 0, 0, errors, timed_out, 4000000000ull);
      TCL_CUDA_CHECK(cudaEventRecord(d1, st_d));
      TCL_CUDA_CHECK(cudaStreamSynchronize(st_d));
      return elapsed_us(d0, d1) / 1000.0;
    });
    for (auto& m : methods) {
      // Transfer alone.
      const double tm = min_of([&]() {
        TCL_CUDA_CHECK(cudaSetDevice(src));
        TCL_CUDA_CHECK(cudaEventRecord(s0, st_s));
        if (m == "ce") {
          for (int ch = 0; ch < chunks; ++ch)
            TCL_CUDA_CHECK(cudaMemcpyPeerAsync(reinterpret_cast<char*>(buf_d) + total / chunks * ch, dst,
                                               reinterpret_cast<char*>(stage_s) + total / chunks * ch, src, total / chunks, st_s));
        } else if (m == "ldst") {
          tcl::bench::flat_copy_kernel<<<blocks, 256, 0, st_s>>>(reinterpret_cast<const uint4*>(stage_s), reinterpret_cast<uint4*>(buf_d), total / 16);
        } else {
          int* e = timed_out;  // any device int; the mover only writes it on a time-out
          TCL_CUDA_CHECK(tcl::bench::launch_bulk_pipe(4, blocks, st_s, stage_s, buf_d, total, static_cast<uint32_t>(tile), tcl::bench::kBulkCopy, e, 2000000000ull));
        }
        TCL_CUDA_CHECK(cudaEventRecord(s1, st_s));
        TCL_CUDA_CHECK(cudaStreamSynchronize(st_s));
        return elapsed_us(s0, s1) / 1000.0;
      });
      // The dependent pipeline: wall time from producer start to consumer end.
      unsigned long long herr = 0;
      const double to = min_of([&]() {
        ++epoch;
        TCL_CUDA_CHECK(cudaSetDevice(dst));
        TCL_CUDA_CHECK(cudaMemsetAsync(errors, 0, 8, st_d));
        TCL_CUDA_CHECK(cudaStreamSynchronize(st_d));
        TCL_CUDA_CHECK(cudaSetDevice(src));
        TCL_CUDA_CHECK(cudaStreamSynchronize(st_s));
        const double w0 = now_ms();
        if (m == "ce") {
          // Produce chunk by chunk so that a chunk's copy can start when it is computed.
          const size_t tiles_per_chunk = n_tiles / chunks;
          for (int ch = 0; ch < chunks; ++ch) {
            produce_ldst_kernel<<<blocks, 256, 0, st_s>>>(stage_s + ch * tiles_per_chunk * tile_floats, nullptr, tile_floats, tiles_per_chunk, I, 0, 0);
            TCL_CUDA_CHECK(cudaMemcpyPeerAsync(buf_d + ch * tiles_per_chunk * tile_floats, dst, stage_s + ch * tiles_per_chunk * tile_floats, src,
                                               tiles_per_chunk * tile, st_s));
            TCL_CUDA_CHECK(cudaEventRecord(chunk_ev[ch], st_s));
          }
          TCL_CUDA_CHECK(cudaSetDevice(dst));
          for (int ch = 0; ch < chunks; ++ch) {
            TCL_CUDA_CHECK(cudaStreamWaitEvent(st_d, chunk_ev[ch], 0));
            consume_kernel<<<blocks, 256, 0, st_d>>>(buf_d + ch * tiles_per_chunk * tile_floats, flags_d, sink, tile_floats, tiles_per_chunk, I, I, 0, 0,
                                                     errors, timed_out, 4000000000ull);
          }
        } else {
          if (m == "ldst") produce_ldst_kernel<<<blocks, 256, 0, st_s>>>(buf_d, flags_d, tile_floats, n_tiles, I, 1, epoch);
          else produce_tma_kernel<<<blocks, 256, 2 * tile, st_s>>>(buf_d, flags_d, tile_floats, n_tiles, I, epoch);
          TCL_CUDA_CHECK(cudaGetLastError());
          TCL_CUDA_CHECK(cudaSetDevice(dst));
          consume_kernel<<<blocks, 256, 0, st_d>>>(buf_d, flags_d, sink, tile_floats, n_tiles, I, I, 1, epoch, errors, timed_out, 4000000000ull);
        }
        TCL_CUDA_CHECK(cudaGetLastError());
        TCL_CUDA_CHECK(cudaSetDevice(dst));
        TCL_CUDA_CHECK(cudaStreamSynchronize(st_d));
        TCL_CUDA_CHECK(cudaSetDevice(src));
        TCL_CUDA_CHECK(cudaStreamSynchronize(st_s));
        const double ms = now_ms() - w0;
        unsigned long long e = 0;
        TCL_CUDA_CHECK(cudaMemcpy(&e, errors, 8, cudaMemcpyDeviceToHost));
        herr += e;
        return ms;
      });
      int to_flag = 0;
      TCL_CUDA_CHECK(cudaMemcpy(&to_flag, timed_out, 4, cudaMemcpyDeviceToHost));
      if (to_flag) { std::fprintf(stderr, "consumer wait ran out (method %s)\n", m.c_str()); return 3; }
      const double pred = std::max(tc_src, std::max(tm, tc_dst));
      const double errp = (pred - to) / to * 100.0;
      const double fpb = 2.0 * I / 4.0;
      if (!check) herr = 0;
      std::printf("%-6s %9d %9.1f | %9.3f %9.3f %9.3f | %9.3f %9.3f %7.1f | %llu\n", m.c_str(), I, fpb, tc_src, tm, tc_dst, to, pred, errp, herr);
      csv.row("%s,%d,%.2f,%.4f,%.4f,%.4f,%.4f,%.4f,%.2f,%llu", m.c_str(), I, fpb, tc_src, tm, tc_dst, to, pred, errp, herr);
    }
  }
  return 0;
}
