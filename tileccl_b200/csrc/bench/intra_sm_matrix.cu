// intra_sm_matrix: what communication warps cost the compute warps of the SAME CTA (the layout of
// a fused kernel: one CTA per SM, a few warps move data to a peer, the others compute).
//   full  probe rate with all W warps computing
//   base  probe rate when C warps exit at once (W - C warps compute)
//   ovl   probe rate when those C warps communicate instead
//   S_warp = full / base   static cost of giving up C warps
//   S_intra = base / ovl   dynamic cost of the communication itself (issue slots, LSU, memory pipe)
//   S_pure = the same ratio for CTAs that carry no communication warps (--comm-ctas N)
// Communication: ldst (16-byte ld/st by the whole warp) or tma (lane 0 drives a double-buffered
// bulk-copy ring, polite __nanosleep polling).  Probes per warp: mma (legacy mma.sync), ffma, smem, hbm.
// (A tcgen05 probe is a whole-CTA resource - one issuing thread, TMEM - and lives in interference_matrix.)
//
// Reference parity: tests/intra_sm_matrix.cu (fused_kernel :162-314, run :564-615, ratios :655-660,
// CSV :621-622).
#include <map>
#include <string>
#include <thread>
#include <vector>

#include <mma.h>
#include <cuda_bf16.h>

#include "../common/host_common.hpp"
#include "movers.cuh"

using namespace tcl::host;
namespace ptx = tcl::ptx;

enum { kProbeMma = 0, kProbeFfma = 1, kProbeSmem = 2, kProbeHbm = 3 };
enum { kCommNone = 0, kCommLdst = 1, kCommTma = 2 };
static const char* kProbeNames[] = {"mma", "ffma", "smem", "hbm"};

struct FusedArgs {
  volatile int* stop;
  unsigned long long* comp_comm;   // iterations of compute warps in CTAs that carry comm warps
  unsigned long long* comp_pure;   // ... in CTAs without comm warps
  unsigned long long* comm_bytes;
  unsigned long long budget_ns;
  int probe, comm, comm_warps, comm_ctas;
  const char* src;   // local
  char* dst;         // peer
  size_t cbuf, msg;
  uint4* pbuf;       // hbm probe buffer
  size_t pbuf_vec_per_warp;
  float* sink;
};

__global__ void __launch_bounds__(1024, 1) fused_kernel(FusedArgs a) {
  extern __shared__ __align__(128) uint8_t dyn[];
  __shared__ uint32_t chase[8192];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const unsigned long long deadline = ptx::globaltimer_ns() + a.budget_ns;
  for (int i = threadIdx.x; i < 8192; i += blockDim.x) chase[i] = (i * 33 + 17) & 8191;
  __syncthreads();
  const bool comm_cta = a.comm_ctas <= 0 || static_cast<int>(blockIdx.x) < a.comm_ctas;
  const bool is_comm_warp = comm_cta && warp < a.comm_warps;
  if (is_comm_warp) {
    if (a.comm == kCommNone) return;
    // Messages are dealt round-robin to the comm warps of the whole grid.
    const size_t n_msgs = a.cbuf / a.msg;
    const size_t gw = static_cast<size_t>(blockIdx.x) * a.comm_warps + warp;
    const size_t n_gw = static_cast<size_t>(a.comm_ctas > 0 ? a.comm_ctas : gridDim.x) * a.comm_warps;
    size_t m = gw % n_msgs;
    unsigned long long moved = 0;
    if (a.comm == kCommLdst) {
      const size_t vec = a.msg / 16;
      for (unsigned it = 0;; ++it) {
        const uint4* s = reinterpret_cast<const uint4*>(a.src + m * a.msg);
        uint4* d = reinterpret_cast<uint4*>(a.dst + m * a.msg);
        for (size_t i = lane; i < vec; i += 32) ptx::st_v4(d + i, ptx::ld_v4_stream(s + i));
        moved += a.msg;
        m += n_gw;
        if (m >= n_msgs) m -= n_msgs * (m / n_msgs);
        if ((it & 7) == 7) {
          if (lane == 0) atomicAdd(a.comm_bytes, moved);
          moved = 0;
          if (*a.stop != 0 || ptx::globaltimer_ns() > deadline) break;
        }
      }
    } else if (lane == 0) {
      // Two slots per comm warp: [slot0 | slot1 | bar0 | bar1].
      const uint32_t slot_stride = static_cast<uint32_t>((a.msg + 127) & ~size_t(127));
      const uint32_t base = ptx::smem_u32(dyn) + warp * (2 * slot_stride + 128);
      const uint32_t bars = base + 2 * slot_stride;
      ptx::mbar_init(bars, 1);
      ptx::mbar_init(bars + 8, 1);
      ptx::fence_mbar_init();
      for (unsigned it = 0;; ++it) {
        const int s = it & 1;
        ptx::bulk_wait_read<1>();   // the store that used this slot two messages ago has read it
        ptx::mbar_arrive_expect_tx(bars + 8 * s, static_cast<uint32_t>(a.msg));
        ptx::bulk_load(base + s * slot_stride, a.src + m * a.msg, static_cast<uint32_t>(a.msg), bars + 8 * s);
        bool ok = false;
        for (int spin = 0; spin < (1 << 22); ++spin) {
          if (ptx::mbar_try_wait(bars + 8 * s, (it >> 1) & 1)) { ok = true; break; }
          __nanosleep(64);
          if ((spin & 255) == 255 && ptx::globaltimer_ns() > deadline + 1000000000ull) break;
        }
        if (!ok) break;
        ptx::bulk_store(a.dst + m * a.msg, base + s * slot_stride, static_cast<uint32_t>(a.msg));
        ptx::bulk_commit();
        moved += a.msg;
        m += n_gw;
        if (m >= n_msgs) m -= n_msgs * (m / n_msgs);
        if ((it & 7) == 7) {
          atomicAdd(a.comm_bytes, moved);
          moved = 0;
          if (*a.stop != 0 || ptx::globaltimer_ns() > deadline) break;
        }
      }
      ptx::bulk_wait<0>();
    }
    return;
  }
  // ---- compute warp ----
  unsigned long long n = 0;
  unsigned long long* counter = comm_cta ? a.comp_comm : a.comp_pure;
  if (a.probe == kProbeFfma) {
    float x = lane * 1e-3f;
    for (;;) {
#pragma unroll 64
      for (int i = 0; i < 512; ++i) x = fmaf(x, 1.0000001f, 0.5f);
      ++n;
      if ((n & 31) == 0) { if (lane == 0) atomicAdd(counter, 32ull); if (*a.stop != 0 || ptx::globaltimer_ns() > deadline) break; }
    }
    if (x == 123.f) a.sink[0] = x;
  } else if (a.probe == kProbeMma) {
    using namespace nvcuda;
    wmma::fragment<wmma::matrix_a, 16, 16, 16, __nv_bfloat16, wmma::row_major> fa;
    wmma::fragment<wmma::matrix_b, 16, 16, 16, __nv_bfloat16, wmma::col_major> fb;
    wmma::fragment<wmma::accumulator, 16, 16, 16, float> fc;
    wmma::fill_fragment(fa, __float2bfloat16(0.001f));
    wmma::fill_fragment(fb, __float2bfloat16(0.002f));
    wmma::fill_fragment(fc, 0.f);
    for (;;) {
#pragma unroll 16
      for (int i = 0; i < 64; ++i) wmma::mma_sync(fc, fa, fb, fc);
      ++n;
      if ((n & 31) == 0) { if (lane == 0) atomicAdd(counter, 32ull); if (*a.stop != 0 || ptx::globaltimer_ns() > deadline) break; }
    }
    if (fc.x[0] == 123.f) a.sink[0] = fc.x[0];
  } else if (a.probe == kProbeSmem) {
    uint32_t idx = threadIdx.x & 8191;
    for (;;) {
#pragma unroll 16
      for (int i = 0; i < 256; ++i) idx = chase[idx];
      ++n;
      if ((n & 31) == 0) { if (lane == 0) atomicAdd(counter, 32ull); if (*a.stop != 0 || ptx::globaltimer_ns() > deadline) break; }
    }
    if (idx == 0xffffffffu) a.sink[0] = 1.f;
  } else {
    const size_t gw = static_cast<size_t>(blockIdx.x) * (blockDim.x >> 5) + warp;
    const uint4* p = a.pbuf + gw * a.pbuf_vec_per_warp;
    uint32_t acc = 0;
    for (;;) {
      for (size_t i = lane; i + 96 < a.pbuf_vec_per_warp; i += 128) {
        const uint4 v0 = ptx::ld_v4_cg(p + i), v1 = ptx::ld_v4_cg(p + i + 32), v2 = ptx::ld_v4_cg(p + i + 64), v3 = ptx::ld_v4_cg(p + i + 96);
        acc += v0.x + v1.x + v2.x + v3.x;
      }
      ++n;
      if (lane == 0) atomicAdd(counter, 1ull);
      if (*a.stop != 0 || ptx::globaltimer_ns() > deadline) break;
    }
    if (acc == 0xdeadbeefu) a.sink[0] = 1.f;
  }
}

struct RunOut {
  double comp_comm = 0, comp_pure = 0, comm_gbps = 0;
};

int main(int argc, char** argv) {
  std::vector<std::string> probes = {"mma", "ffma", "smem", "hbm"}, comms = {"ldst", "tma"};
  std::vector<int> comm_warps = {1, 2, 4};
  int warps = 16, blocks = 0, comm_ctas = 0, window_ms = 300, src = 0, dst = 1;
  size_t msg = 16384, cbuf = size_t(64) << 20, pbuf = size_t(256) << 20;
  std::string csv_path;
  bool once = false;
  Args a(argc, argv);
  while (a.more()) {
    std::string f = a.flag(), v;
    auto need = [&]() { if (!a.value(&v)) std::exit(1); return v; };
    if (f == "--probes") probes = split_csv(need());
    else if (f == "--once") once = true;
    else if (f == "--comms") comms = split_csv(need());
    else if (f == "--comm-warps") parse_int_list(need(), &comm_warps);
    else if (f == "--warps") warps = std::atoi(need().c_str());
    else if (f == "--blocks") blocks = std::atoi(need().c_str());
    else if (f == "--comm-ctas") comm_ctas = std::atoi(need().c_str());
    else if (f == "--msg") parse_bytes(need(), &msg);
    else if (f == "--cbuf") parse_bytes(need(), &cbuf);
    else if (f == "--pbuf") parse_bytes(need(), &pbuf);
    else if (f == "--window-ms") window_ms = std::atoi(need().c_str());
    else if (f == "--src") src = std::atoi(need().c_str());
    else if (f == "--dst") dst = std::atoi(need().c_str());
    else if (f == "--csv") csv_path = need();
    else {
      std::printf("usage: %s [--probes mma,ffma,smem,hbm] [--comms ldst,tma] [--comm-warps LIST] [--warps N] [--blocks N] [--comm-ctas N]\n"
                  "          [--msg B] [--cbuf B] [--pbuf B] [--window-ms MS] [--src N] [--dst N] [--csv FILE] [--once]\n"
                  "--once: for a profiler: every (probe, comm, comm-warps) combination is launched once for --window-ms and left to end on\n"
                  "        its own time budget; nothing is measured and the host does not touch the kernel while it runs\n", argv[0]);
      return f == "-h" || f == "--help" ? 0 : 1;
    }
  }
  warps = std::max(2, std::min(32, warps));
  msg = msg / 16 * 16;
  const int ndev = device_count();
  if (src >= ndev || dst >= ndev) { std::fprintf(stderr, "need GPUs %d and %d, have %d\n", src, dst, ndev); return 1; }
  if (src != dst && !enable_peer_all(std::max(src, dst) + 1)) return 1;
  TCL_CUDA_CHECK(cudaSetDevice(src));
  cudaDeviceProp prop;
  TCL_CUDA_CHECK(cudaGetDeviceProperties(&prop, src));
  if (blocks <= 0) blocks = prop.multiProcessorCount;
  print_device_line(src);
  int max_cw = 1;
  for (int c : comm_warps) max_cw = std::max(max_cw, c);
  const size_t dyn_smem = static_cast<size_t>(max_cw) * (2 * ((msg + 127) & ~size_t(127)) + 128);
  const bool tma_ok = dyn_smem + 34000 <= prop.sharedMemPerBlockOptin;
  if (tma_ok) TCL_CUDA_CHECK(cudaFuncSetAttribute(fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(dyn_smem)));

  FusedArgs fa{};
  // Stop flag and counters live in device memory; the host raises / snapshots them with async
  // copies on its own stream, so the kernel's polling and counting never crosses PCIe.
  int* stop_h;
  unsigned long long* cnt_h;
  TCL_CUDA_CHECK(cudaHostAlloc(&stop_h, 4, cudaHostAllocDefault));
  TCL_CUDA_CHECK(cudaHostAlloc(&cnt_h, 64, cudaHostAllocDefault));
  int* stop_d;
  unsigned long long* cnt_d;
  TCL_CUDA_CHECK(cudaMalloc(&stop_d, 4));
  TCL_CUDA_CHECK(cudaMalloc(&cnt_d, 64));
  cudaStream_t snap;
  TCL_CUDA_CHECK(cudaStreamCreateWithFlags(&snap, cudaStreamNonBlocking));
  fa.stop = stop_d;
  fa.comp_comm = cnt_d; fa.comp_pure = cnt_d + 1; fa.comm_bytes = cnt_d + 2;
  char *cs, *cd;
  TCL_CUDA_CHECK(cudaMalloc(&cs, cbuf));
  TCL_CUDA_CHECK(cudaMalloc(&fa.pbuf, pbuf));
  TCL_CUDA_CHECK(cudaMemset(fa.pbuf, 1, pbuf));
  TCL_CUDA_CHECK(cudaMalloc(&fa.sink, 64));
  TCL_CUDA_CHECK(cudaSetDevice(dst));
  TCL_CUDA_CHECK(cudaMalloc(&cd, cbuf));
  TCL_CUDA_CHECK(cudaSetDevice(src));
  fa.src = cs; fa.dst = cd; fa.cbuf = cbuf / msg * msg; fa.msg = msg;
  fa.pbuf_vec_per_warp = pbuf / 16 / (static_cast<size_t>(blocks) * warps);
  fa.comm_ctas = comm_ctas;
  cudaStream_t st;
  TCL_CUDA_CHECK(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking));

  auto run = [&](int probe, int comm, int cw) {
    fa.probe = probe; fa.comm = comm; fa.comm_warps = cw;
    fa.budget_ns = static_cast<unsigned long long>(window_ms + 2000) * 1000000ull;
    TCL_CUDA_CHECK(cudaMemsetAsync(stop_d, 0, 4, st));
    TCL_CUDA_CHECK(cudaMemsetAsync(cnt_d, 0, 64, st));
    auto snapshot = [&]() {
      TCL_CUDA_CHECK(cudaMemcpyAsync(cnt_h, cnt_d, 24, cudaMemcpyDeviceToHost, snap));
      TCL_CUDA_CHECK(cudaStreamSynchronize(snap));
    };
    fused_kernel<<<blocks, warps * 32, comm == kCommTma ? dyn_smem : 0, st>>>(fa);
    TCL_CUDA_CHECK(cudaGetLastError());
    std::this_thread::sleep_for(std::chrono::milliseconds(30));
    volatile unsigned long long* c = cnt_h;
    snapshot();
    const unsigned long long a0 = c[0], p0 = c[1], b0 = c[2];
    const double t0 = now_ms();
    std::this_thread::sleep_for(std::chrono::milliseconds(window_ms));
    snapshot();
    const unsigned long long a1 = c[0], p1 = c[1], b1 = c[2];
    const double dt = (now_ms() - t0) / 1000.0;
    *stop_h = 1;
    TCL_CUDA_CHECK(cudaMemcpyAsync(stop_d, stop_h, 4, cudaMemcpyHostToDevice, snap));
    TCL_CUDA_CHECK(cudaStreamSynchronize(snap));
    TCL_CUDA_CHECK(cudaStreamSynchronize(st));
    RunOut o;
    o.comp_comm = (a1 - a0) / dt;
    o.comp_pure = (p1 - p0) / dt;
    o.comm_gbps = (b1 - b0) / dt / 1e9;
    return o;
  };

  if (once) {
    for (auto& pn : probes) {
      int pid = -1;
      for (int k = 0; k < 4; ++k) if (pn == kProbeNames[k]) pid = k;
      if (pid < 0) { std::fprintf(stderr, "unknown probe %s\n", pn.c_str()); return 1; }
      for (auto& cn : comms) {
        const int cid = cn == "tma" ? kCommTma : kCommLdst;
        if (cid == kCommTma && !tma_ok) continue;
        for (int cw : comm_warps) {
          if (cw < 1 || cw >= warps) continue;
          fa.probe = pid; fa.comm = cid; fa.comm_warps = cw;
          fa.budget_ns = static_cast<unsigned long long>(window_ms) * 1000000ull;
          TCL_CUDA_CHECK(cudaMemsetAsync(stop_d, 0, 4, st));
          TCL_CUDA_CHECK(cudaMemsetAsync(cnt_d, 0, 64, st));
          fused_kernel<<<blocks, warps * 32, cid == kCommTma ? dyn_smem : 0, st>>>(fa);
          TCL_CUDA_CHECK(cudaGetLastError());
          TCL_CUDA_CHECK(cudaStreamSynchronize(st));
          std::printf("once: %s x %s, %d comm warps, %d ms\n", pn.c_str(), cn.c_str(), cw, window_ms);
        }
      }
    }
    return 0;
  }
  Csv csv;
  if (!csv.open(csv_path, "probe,comm,warps,comm_warps,comm_ctas,msg_bytes,comm_gbps,full,base,ovl,unit,S_warp,S_intra,S_pure")) return 1;
  std::printf("# intra_sm_matrix: %d CTAs x %d warps, msg %zu B, window %d ms, comm-ctas %d\n", blocks, warps, msg, window_ms, comm_ctas);
  std::printf("%-5s %-5s %3s | %10s | %12s %12s %12s %8s | %7s %7s %7s\n", "probe", "comm", "cw", "comm GB/s", "full", "base", "ovl", "unit", "S_warp", "S_intra", "S_pure");
  for (auto& pn : probes) {
    int pid = -1;
    for (int k = 0; k < 4; ++k) if (pn == kProbeNames[k]) pid = k;
    if (pid < 0) { std::fprintf(stderr, "unknown probe %s\n", pn.c_str()); return 1; }
    const RunOut full = run(pid, kCommNone, 0);
    std::map<int, RunOut> base;
    for (auto& cn : comms) {
      const int cid = cn == "tma" ? kCommTma : kCommLdst;
      if (cid == kCommTma && !tma_ok) { std::printf("%-5s %-5s : skipped (no shared memory for the staging slots)\n", pn.c_str(), cn.c_str()); continue; }
      for (int cw : comm_warps) {
        if (cw < 1 || cw >= warps) continue;
        if (!base.count(cw)) base[cw] = run(pid, kCommNone, cw);
        const RunOut ovl = run(pid, cid, cw);
        const RunOut& b = base[cw];
        const double s_warp = b.comp_comm > 0 ? full.comp_comm / b.comp_comm : 0;
        const double s_intra = ovl.comp_comm > 0 ? b.comp_comm / ovl.comp_comm : 0;
        const double s_pure = ovl.comp_pure > 0 ? b.comp_pure / ovl.comp_pure : 0;
        if (ovl.comp_comm <= 0) std::printf("%-5s %-5s %3d | [!] probe made NO progress\n", pn.c_str(), cn.c_str(), cw);
        std::printf("%-5s %-5s %3d | %10.2f | %12.3e %12.3e %12.3e %8s | %7.3f %7.3f %7.3f\n", pn.c_str(), cn.c_str(), cw, ovl.comm_gbps, full.comp_comm,
                    b.comp_comm, ovl.comp_comm, "iter/s", s_warp, s_intra, s_pure);
        csv.row("%s,%s,%d,%d,%d,%zu,%.2f,%.4e,%.4e,%.4e,iter/s,%.3f,%.3f,%.3f", pn.c_str(), cn.c_str(), warps, cw, comm_ctas, msg, ovl.comm_gbps, full.comp_comm,
                b.comp_comm, ovl.comp_comm, s_warp, s_intra, s_pure);
      }
    }
  }
  return 0;
}
