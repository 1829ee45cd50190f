// Persistent, warp-specialised bf16 GEMM for sm_100a: tcgen05.mma with the
// accumulator in tensor memory (TMEM), operands staged in shared memory by
// TMA, and three fused forms that share one mainloop:
//
//   kModePlain   D = A * B^T, D may live anywhere (local, a peer, or row
//                segments scattered over peers: the epilogue-remote experiment)
//   kModeGemmRs  GEMM -> reduce-scatter: the epilogue pushes bf16 partial tiles
//                with 16-byte st.global into the staging slot of the rank that
//                owns the rows; a signalling warp fences at system scope and
//                bumps the owner's per-tile counter; this rank's reduce warps
//                sum the slots of its own segment in fp32 as soon as a tile has
//                all its partials (or, NVLS variant, read the sum through the
//                NVSwitch with multimem.ld_reduce)
//   kModeAgGemm  all-gather -> GEMM: gather warps pull the peers' A shards row
//                by row with 16-byte P2P loads into the local gathered A and
//                publish per-row-block counters; the TMA producer acquires a
//                row block's counter before it loads tiles from it
//
// A is [M, K] row-major, B is [N, K] row-major (the "column-major B[K, N]" of
// the reference), D is row-major.  fp32 accumulation, bf16 output.
//
// Warp roles (352 threads, one CTA per SM):
//   warp 0      TMA producer (one lane)
//   warp 1      TMEM allocation + tcgen05.mma issue (one lane, leader CTA only)
//   warps 2-5   epilogue: tcgen05.ld -> bf16 -> swizzled smem transpose ->
//               coalesced 16-byte global stores, 256 contiguous bytes per row (local or peer);
//               options: 32-byte stores (epi_st256), TMA stores from the same buffer (epi_tma_store),
//               SiLU(gate)*up on the accumulators (epi_silu_mul)
//   warps 6-9   communication: reduce warps (GEMM+RS) or gather warps (AG+GEMM)
//   warp 10     GEMM+RS signalling: publishes finished tiles to their owners
//
// kCtaGroup = 2 pairs two CTAs (a 2x1 cluster) on one 256x256 tile: each CTA
// loads its own 128 rows of A and its own 128 rows of B (no multicast), the
// leader issues cta_group::2 MMAs that read both CTAs' shared memory, and each
// CTA drains its own 128 accumulator rows.
//
// No TMA load here touches another GPU's memory, and in the fused modes no TMA
// instruction at all does: remote data moves by plain ld/st.  (The optional
// TMA-store epilogue of the plain mode stores wherever D lives, a peer included:
// that is the epilogue-remote experiment's second epilogue.)  Every wait is bounded (deadline from %globaltimer); on
// time-out the CTA records a status word, lets its copies land, frees its TMEM
// and returns.
//
// The call number that the flag counters are compared with comes from the host with every
// launch, or from a device word that the kernel advances itself (GemmParams::epoch_dev), which
// lets a captured CUDA graph replay the launch.
//
// Reference parity: comm_comp/gemm_sm90.cuh:48-140 (plain GEMM, TMA-store and
// direct-store epilogues), comm_comp/rs_gemm_kernel_sm90.cuh:90-892 and
// comm_comp/rs_dma_sm90.cuh:53-351 (fused GEMM+RS, which pulls peer tiles with
// TMA and reduces in fp16 with red.global.add; here the partials are pushed
// and summed in fp32), comm_comp/exp2_ag_gemm_granularity.cu:15-20 (the
// in-kernel flag-gated all-gather GEMM that the reference describes but does
// not implement).
#pragma once
#include <cstdint>
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "../ptx/ldst_sys.cuh"
#include "../ptx/mbarrier.cuh"
#include "../ptx/tcgen05.cuh"
#include "../ptx/tma.cuh"
#include "tile_sched.hpp"

namespace tcl {

enum GemmMode : int { kModePlain = 0, kModeGemmRs = 1, kModeAgGemm = 2 };

constexpr int kMaxWorld = 8;

// Status codes written to status[0] by the first role that gives up.
enum GemmStatus : int {
  kOk = 0,
  kErrProducerEmpty = 1,   // TMA producer: stage never freed
  kErrMmaFull = 2,         // MMA issuer: operands never landed
  kErrMmaTmemEmpty = 3,    // MMA issuer: accumulator never drained
  kErrEpiTmemFull = 4,     // epilogue: accumulator never completed
  kErrStartBarrier = 5,    // a peer never arrived at the start barrier
  kErrRsTileCount = 6,     // reduce warps: a tile never got all its partials
  kErrAgFlag = 7,          // TMA producer: a gathered row block never arrived
  kErrAgEndBarrier = 8,    // a peer never finished reading this rank's shard
  kErrBounds = 9           // debug build only: an address fell outside the range it must stay in (access skipped)
};

struct GemmParams {
  int mode;
  int M, N, K;
  int ldc;        // output row pitch in elements
  TileSched sched;
  int world, rank;
  int epoch;      // 1-based call number of the plan that owns the flag buffers
  int* epoch_dev; // optional, two ints in device memory: [0] calls of this plan that have completed, [1] CTAs of
                  // the running call that have finished.  When set, the call number is [0] + 1 instead of `epoch`
                  // and the last CTA to finish advances it: the launch can then be replayed from a CUDA graph.
  int comm_enabled;
  int epi_silu_mul;  // epilogue computes silu(gate) * up from the two 128-column halves of every tile; D is [M, N/2]
  int epi_tma_store;  // the plain epilogue leaves through TMA: cp.async.bulk.tensor stores of 32 x 64 boxes from the
                      // warp's staging buffer (not with GEMM+RS communication, not with epi_silu_mul)
  int epi_st256;  // the plain epilogue stores 32 bytes per lane (st.global.v8.b32); needs 32-byte aligned destinations and pitch
  int ablate;     // experiment knobs: bit 0 = no reduce warps, bit 1 = no tile signals (and no reduce warps), bit 2 = AG+GEMM producer
                  // does not wait for gathered rows (these three: timing only, the output is not valid);
                  // bit 3 = the last epilogue warp sleeps a few microseconds before the final stores of every
                  // tile (the output stays valid: a test of the publish-after-all-stores rule)

  // Output routing.  Rows are split in segments of seg_rows; row r of segment
  // s goes to dst_base[s] + (dst_row_off[s] + r - s * seg_rows) * ldc.
  int seg_rows;
  __nv_bfloat16* dst_base[kMaxWorld];
  long long dst_row_off[kMaxWorld];

  // GEMM+RS
  int* rs_tile_cnt[kMaxWorld];        // owner's counters, one per 128x256 tile of its segment
  const __nv_bfloat16* rs_stage;      // this rank's staging [world][seg_rows][N]
  __nv_bfloat16* rs_out;              // this rank's reduced shard [seg_rows][ld_out]
  int ld_out;
  int rs_signal_batch;                // finished tiles the signalling warp lets accumulate before it fences and signals
                                      // (the last tiles of the CTA are always signalled at once)
  // NVLS variant: partial tiles stay in the producer's own full-size staging [M][N]; the owner's reduce
  // warps read this multicast address of it, and the NVSwitch returns the sum over all ranks.
  const __nv_bfloat16* rs_mc_stage;   // multicast mapping of the staging buffer, or nullptr (P2P push)

  // AG+GEMM
  const __nv_bfloat16* ag_src[kMaxWorld];  // rank s's shard [seg_rows][K] (a peer pointer)
  __nv_bfloat16* ag_full;                  // local gathered A [M][K]
  int* ag_flags;                           // local counters, one per gather_rows row block
  int gather_rows;
  int ag_item_rows;                        // rows one gather warp moves per work item (and per counter arrival);
                                           // small items make rows land progressively, in schedule order
  int ag_warps;                            // gather warps per CTA that take part (1..4); the others idle
  int ag_vec32;                            // pull form: 32-byte loads and stores (needs K % 16 == 0) instead of 16-byte ones
  int* ag_done;                            // local: gather warps that finished (monotonic)
  int* ag_read_done[kMaxWorld];            // rank s's "peers done reading me" counter
  // Push form of the all-gather: every rank stores its own shard into every peer's gathered buffer.
  int ag_push;                             // 0 = pull (loads from peers), 1 = push (stores to peers)
  __nv_bfloat16* ag_dst[kMaxWorld];        // rank s's gathered buffer [M][K] (a peer pointer)
  int* ag_flag_peer[kMaxWorld];            // rank s's row-block counters

  // Start barrier: rank s's arrival counter.
  int* barrier[kMaxWorld];

  // Debug build (TCL_DEBUG_BOUNDS): every data address that may be remote is checked against the
  // mapping of the rank it targets before it is used; a bad one is recorded and the access skipped.
  unsigned long long range_lo[kMaxWorld];
  unsigned long long range_hi[kMaxWorld];

  int* status;                   // [4]: code, blockIdx, detail0, detail1
  unsigned long long timeout_ns;
};

// Tensor maps of the output, one per row segment (box 32 rows x 64 columns, 128-byte swizzle); only read
// when GemmParams::epi_tma_store is set.
struct OutMaps {
  CUtensorMap m[kMaxWorld];
};

template <int kCtaGroup>
struct GemmCfg {
  static constexpr int BM = 128;                    // accumulator rows per CTA
  static constexpr int TILE_M = BM * kCtaGroup;     // rows per scheduled tile
  static constexpr int BN = 256;
  static constexpr int BK = 64;                     // one 128-byte swizzle atom of bf16
  static constexpr int UMMA_K = 16;
  static constexpr int B_ROWS = BN / kCtaGroup;     // B rows each CTA loads
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = B_ROWS * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (kCtaGroup == 1) ? 4 : 6;
  static constexpr int EPI_WARPS = 4;
  static constexpr int EPI_CHUNK_COLS = 64;         // bf16 columns per transpose chunk
  static constexpr int EPI_BUF_BYTES = 32 * 2 * EPI_CHUNK_COLS * 2;   // 8 KiB: 32 rows x 128 columns per warp
  static constexpr int EPI_BYTES = EPI_WARPS * EPI_BUF_BYTES;
  static constexpr int COMM_WARPS = 4;
  static constexpr int SIGNAL_WARP = 2 + EPI_WARPS + COMM_WARPS;  // index of the signalling warp
  static constexpr int THREADS = (3 + EPI_WARPS + COMM_WARPS) * 32;
  static constexpr int TMEM_COLS = 512;             // two accumulator buffers of BN columns
  static constexpr int CTRL_BYTES = 256;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_BYTES + CTRL_BYTES + 1024;
};

namespace detail {

// epoch * count in wrapping (unsigned) arithmetic: counters are compared by signed distance, so a
// long-lived plan may let them wrap.
__device__ __forceinline__ int epoch_times(int epoch, int count) {
  return static_cast<int>(static_cast<unsigned>(epoch) * static_cast<unsigned>(count));
}

__device__ __forceinline__ void report(const GemmParams& p, volatile int* s_abort, int code, int d0,
                                       int d1) {
  if (atomicCAS(p.status, 0, code) == 0) {
    p.status[1] = static_cast<int>(blockIdx.x);
    p.status[2] = d0;
    p.status[3] = d1;
  }
  *s_abort = 1;
}

// Debug-build address check: true if [addr, addr + bytes) lies inside rank `r`'s mapped range.
__device__ __forceinline__ bool in_range(const GemmParams& p, volatile int* s_abort, int r, const void* addr, unsigned bytes) {
#ifdef TCL_DEBUG_BOUNDS
  const unsigned long long a = reinterpret_cast<unsigned long long>(addr);
  if (a < p.range_lo[r] || a + bytes > p.range_hi[r]) {
    report(p, s_abort, kErrBounds, r, static_cast<int>((a - p.range_lo[r]) >> 4));
    return false;
  }
#endif
  return true;
}

// Sums the `kWorld` staged bf16 partials of one 128x256 tile in fp32 and writes
// the bf16 result.  128 threads; a thread owns one 16-byte column chunk and
// walks rows 4 apart.  kRows rows are in flight per thread (kRows * kWorld
// independent 16-byte loads) so that the loop is bandwidth- not latency-bound.
template <int kWorld, int kRows>
__device__ __forceinline__ void reduce_tile(const __nv_bfloat16* __restrict__ stage, size_t slot_elems,
                                            size_t tile_off, int ldn, __nv_bfloat16* __restrict__ out,
                                            size_t out_off, int ld_out, int ctid, int world_rt) {
  const int world = kWorld > 0 ? kWorld : world_rt;
  constexpr int kMaxW = kWorld > 0 ? kWorld : 8;
  const int r_base = ctid >> 5;  // 0..3
#pragma unroll 1
  for (int pass = 0; pass < 32; pass += kRows) {
    uint4 w[kRows][kMaxW];
#pragma unroll
    for (int j = 0; j < kRows; ++j) {
      const size_t row_off = static_cast<size_t>((pass + j) * 4 + r_base) * ldn;
#pragma unroll
      for (int src = 0; src < kMaxW; ++src) {
        if (src < world) w[j][src] = ptx::ld_v4_stream(stage + src * slot_elems + tile_off + row_off);
      }
    }
#pragma unroll
    for (int j = 0; j < kRows; ++j) {
      float acc[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] = 0.f;
#pragma unroll
      for (int src = 0; src < kMaxW; ++src) {
        if (src < world) {
          const uint32_t u[4] = {w[j][src].x, w[j][src].y, w[j][src].z, w[j][src].w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            acc[2 * e] += __uint_as_float(u[e] << 16);
            acc[2 * e + 1] += __uint_as_float(u[e] & 0xffff0000u);
          }
        }
      }
      uint4 o;
      o.x = ptx::pack_bf16x2(__float_as_uint(acc[0]), __float_as_uint(acc[1]));
      o.y = ptx::pack_bf16x2(__float_as_uint(acc[2]), __float_as_uint(acc[3]));
      o.z = ptx::pack_bf16x2(__float_as_uint(acc[4]), __float_as_uint(acc[5]));
      o.w = ptx::pack_bf16x2(__float_as_uint(acc[6]), __float_as_uint(acc[7]));
      ptx::st_v4(out + out_off + static_cast<size_t>((pass + j) * 4 + r_base) * ld_out, o);
    }
  }
}

// NVLS form of reduce_tile: one multimem.ld_reduce per 16 bytes returns the sum (fp32 accumulation in
// the switch) of the same tile in every rank's staging buffer.  8 loads in flight per thread.
__device__ __forceinline__ void reduce_tile_nvls(const __nv_bfloat16* mc_tile, int ldn, __nv_bfloat16* __restrict__ out,
                                                 size_t out_off, int ld_out, int ctid) {
  const int r_base = ctid >> 5;
#pragma unroll 1
  for (int pass = 0; pass < 32; pass += 8) {
    uint4 w[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) w[j] = ptx::multimem_ld_reduce_bf16x8(mc_tile + static_cast<size_t>((pass + j) * 4 + r_base) * ldn);
#pragma unroll
    for (int j = 0; j < 8; ++j) ptx::st_v4(out + out_off + static_cast<size_t>((pass + j) * 4 + r_base) * ld_out, w[j]);
  }
}

// One warp copies `item_bytes` (a multiple of sizeof(V)) from a peer's memory to local memory with loads that do not
// allocate in L1.  Two register banks of kUnroll vectors per lane: the loads of one step (kUnroll * 32 lanes *
// sizeof(V) = 4 KiB) are issued before the previous step is stored, so 4 to 8 KiB of peer loads per warp are
// always in flight.  V = uint4 moves 16 bytes per instruction, V = Vec8 32 bytes (half the instructions; the
// addresses must then be 32-byte aligned).
__device__ __forceinline__ void ld_item(uint4& v, const char* p) { v = ptx::ld_v4_stream(p); }
__device__ __forceinline__ void ld_item(ptx::Vec8& v, const char* p) { v = ptx::ld_v8_stream(p); }
__device__ __forceinline__ void st_item(char* p, const uint4& v) { ptx::st_v4(p, v); }
__device__ __forceinline__ void st_item(char* p, const ptx::Vec8& v) { ptx::st_v8(p, v); }

template <typename V, int kUnroll>
__device__ __forceinline__ void copy_item(const char* __restrict__ src, char* __restrict__ dst, size_t item_bytes, int lane) {
  constexpr size_t kRow = 32 * sizeof(V);          // bytes one warp-wide instruction moves
  constexpr size_t kStep = kUnroll * kRow;
  size_t off = static_cast<size_t>(lane) * sizeof(V);
  auto fits = [&](size_t o) { return o + (kUnroll - 1) * kRow < item_bytes; };
  if (fits(off)) {
    V wa[kUnroll], wb[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) ld_item(wa[u], src + off + u * kRow);
    size_t nxt = off + kStep;
    for (;;) {
      bool more = fits(nxt);
      if (more) {
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) ld_item(wb[u], src + nxt + u * kRow);
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) st_item(dst + off + u * kRow, wa[u]);
      off = nxt;
      nxt += kStep;
      if (!more) break;
      more = fits(nxt);
      if (more) {
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) ld_item(wa[u], src + nxt + u * kRow);
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) st_item(dst + off + u * kRow, wb[u]);
      off = nxt;
      nxt += kStep;
      if (!more) break;
    }
  }
  for (; off < item_bytes; off += kRow) {
    V v;
    ld_item(v, src + off);
    st_item(dst + off, v);
  }
}

}  // namespace detail

template <int kCtaGroup>
__global__ void __launch_bounds__(GemmCfg<kCtaGroup>::THREADS, 1)
gemm_sm100_kernel(const __grid_constant__ CUtensorMap tmap_a,
                  const __grid_constant__ CUtensorMap tmap_b,
                  const __grid_constant__ GemmParams p,
                  const __grid_constant__ OutMaps omaps) {
  using Cfg = GemmCfg<kCtaGroup>;
  using namespace ptx;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_u32 = smem_u32(smem_raw);
  const uint32_t base_u32 = (raw_u32 + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base_u32 - raw_u32);

  const uint32_t stage_u32 = base_u32;
  const uint32_t epi_u32 = base_u32 + Cfg::STAGES * Cfg::STAGE_BYTES;
  uint8_t* ctrl = smem + Cfg::STAGES * Cfg::STAGE_BYTES + Cfg::EPI_BYTES;
  const uint32_t ctrl_u32 = epi_u32 + Cfg::EPI_BYTES;
  // control block: full[S] | empty[S] | tmem_full[2] | tmem_empty[2] | drain | tmem_ptr | abort | bcast
  const uint32_t bar_full = ctrl_u32;
  const uint32_t bar_empty = bar_full + 8 * Cfg::STAGES;
  const uint32_t bar_tfull = bar_empty + 8 * Cfg::STAGES;
  const uint32_t bar_tempty = bar_tfull + 16;
  const uint32_t bar_drain = bar_tempty + 16;
  volatile uint32_t* s_tmem_ptr = reinterpret_cast<volatile uint32_t*>(ctrl + 16 * Cfg::STAGES + 40);
  volatile int* s_abort = reinterpret_cast<volatile int*>(ctrl + 16 * Cfg::STAGES + 44);
  volatile int* s_bcast = reinterpret_cast<volatile int*>(ctrl + 16 * Cfg::STAGES + 48);
  // tiles whose stores epilogue warp w has issued, one monotonic counter per warp (GEMM+RS): a tile may be
  // published once the smallest of the four has passed it
  volatile int* s_warp_tiles = reinterpret_cast<volatile int*>(ctrl + 16 * Cfg::STAGES + 64);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = (kCtaGroup == 2) ? cluster_ctarank() : 0u;
  const int group_id = blockIdx.x / kCtaGroup;
  const int num_groups = gridDim.x / kCtaGroup;
  const unsigned long long deadline = globaltimer_ns() + p.timeout_ns;
  // Call number: from the host, or from the plan's device word (stable during the call: it is advanced by the
  // last CTA to finish, after every CTA has read it here).
  const int epoch = p.epoch_dev ? ld_relaxed_sys(p.epoch_dev) + 1 : p.epoch;

  const TileSched sched = p.sched;
  const int num_tiles = sched.num_tiles();
  const int k_blocks = (p.K + Cfg::BK - 1) / Cfg::BK;
  const bool fused_comm = p.comm_enabled && p.world > 1;

  // ---- set-up ---------------------------------------------------------------
  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::STAGES; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_tfull + 8 * b, 1);
      mbar_init(bar_tempty + 8 * b, Cfg::EPI_WARPS * kCtaGroup);
    }
    mbar_init(bar_drain, 1);
    *s_abort = 0;
    *s_bcast = 0;
    for (int w = 0; w < Cfg::EPI_WARPS; ++w) s_warp_tiles[w] = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc<kCtaGroup>(smem_u32(const_cast<uint32_t*>(s_tmem_ptr)), Cfg::TMEM_COLS);
    tmem_relinquish<kCtaGroup>();
  }
  // Start barrier, arrival side: one CTA tells every rank (itself included)
  // that this rank has entered call `epoch`.
  if (fused_comm && blockIdx.x == 0 && warp == 6 && lane < p.world) {
    red_release_sys_add(p.barrier[lane], 1);
  }
  tc_fence_before_sync();
  __syncthreads();
  if constexpr (kCtaGroup == 2) {
    cluster_arrive();
    cluster_wait();
  }
  tc_fence_after_sync();
  const uint32_t tmem_base = *s_tmem_ptr;
  const int barrier_target = detail::epoch_times(epoch, p.world);

  // ---- roles ----------------------------------------------------------------
  if (warp == 0) {
    // ===== TMA producer =====
    if (lane == 0) {
      int it = 0;
      bool ok = true;
      for (int t = group_id; t < num_tiles && ok; t += num_groups) {
        int m_blk, n_blk;
        sched.tile(t, &m_blk, &n_blk);
        const int m0 = m_blk * Cfg::TILE_M + static_cast<int>(cta_rank) * Cfg::BM;
        const int n0 = n_blk * Cfg::BN + static_cast<int>(cta_rank) * Cfg::B_ROWS;
        if (p.mode == kModeAgGemm && fused_comm && !(p.ablate & 4) && (m0 / p.seg_rows) != p.rank) {
          // Rows [m0, m0+BM) lie in one gather block (gather_rows % BM == 0).
          const int blk = m0 / p.gather_rows;
          const int target = detail::epoch_times(epoch, p.gather_rows / p.ag_item_rows);
          int seen = 0;
          const bool landed = p.ag_push ? wait_ge<true>(p.ag_flags + blk, target, s_abort, deadline, &seen)
                                        : wait_ge<false>(p.ag_flags + blk, target, s_abort, deadline, &seen);
          if (!landed) {
            detail::report(p, s_abort, kErrAgFlag, blk, seen);
            ok = false;
            break;
          }
          fence_proxy_async();
        }
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % Cfg::STAGES;
          const uint32_t ph = (it / Cfg::STAGES) & 1;
          if (!mbar_wait<kCtaGroup == 2>(bar_empty + 8 * s, ph ^ 1u, s_abort, deadline)) {
            detail::report(p, s_abort, kErrProducerEmpty, t, kb);
            ok = false;
            break;
          }
          const uint32_t a_dst = stage_u32 + s * Cfg::STAGE_BYTES;
          const uint32_t b_dst = a_dst + Cfg::A_BYTES;
          if constexpr (kCtaGroup == 1) {
            mbar_arrive_expect_tx(bar_full + 8 * s, Cfg::STAGE_BYTES);
            tma_load_2d(a_dst, &tmap_a, bar_full + 8 * s, kb * Cfg::BK, m0);
            tma_load_2d(b_dst, &tmap_b, bar_full + 8 * s, kb * Cfg::BK, n0);
          } else {
            // Both CTAs' bytes are counted on the leader's barrier.
            if (cta_rank == 0) mbar_arrive_expect_tx(bar_full + 8 * s, 2 * Cfg::STAGE_BYTES);
            const uint32_t lead_bar = mapa(bar_full + 8 * s, 0);
            tma_load_2d_pair(a_dst, &tmap_a, lead_bar, kb * Cfg::BK, m0);
            tma_load_2d_pair(b_dst, &tmap_b, lead_bar, kb * Cfg::BK, n0);
          }
        }
      }
      if (*s_abort) {
        // Loads in flight must land before shared memory goes away.  The full barrier of a stage completes
        // when the bytes armed on it have arrived, so the leader (and the single CTA) waits, with its own
        // short limit, on the barriers of the last STAGES iterations it issued: no later arming can follow.
        // In a pair the barriers live in the leader and count both CTAs' bytes; the second CTA cannot wait on
        // them (mbarrier waits are CTA-local), so it pauses for a bounded time instead, and the cluster
        // barrier of the tear-down holds it until the leader has passed its own drain.
        if (cta_rank == 0) {
          const unsigned long long d2 = globaltimer_ns() + 2000000ull;
          for (int j = it > Cfg::STAGES ? it - Cfg::STAGES : 0; j < it; ++j) {
            const uint32_t bar = bar_full + 8 * (j % Cfg::STAGES);
            const uint32_t ph = (j / Cfg::STAGES) & 1;
            for (int spin = 0; spin < (1 << 20); ++spin) {
              if (mbar_try_wait(bar, ph) || globaltimer_ns() > d2) break;
            }
          }
        } else {
          for (int i = 0; i < 64; ++i) __nanosleep(4000);
        }
      }
    }
  } else if (warp == 1) {
    // ===== MMA issuer (leader CTA of the group) =====
    if (lane == 0 && cta_rank == 0) {
      constexpr uint32_t idesc = make_idesc_bf16_f32(Cfg::TILE_M, Cfg::BN);
      int it = 0;
      int lt = 0;
      bool ok = true;
      for (int t = group_id; t < num_tiles && ok; t += num_groups, ++lt) {
        const int b = lt & 1;
        if (!mbar_wait<kCtaGroup == 2>(bar_tempty + 8 * b, ((lt >> 1) & 1) ^ 1u, s_abort, deadline)) {
          detail::report(p, s_abort, kErrMmaTmemEmpty, t, lt);
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(b * Cfg::BN);
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % Cfg::STAGES;
          const uint32_t ph = (it / Cfg::STAGES) & 1;
          if (!mbar_wait(bar_full + 8 * s, ph, s_abort, deadline)) {
            detail::report(p, s_abort, kErrMmaFull, t, kb);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_u32 = stage_u32 + s * Cfg::STAGE_BYTES;
          const uint64_t a_desc = make_smem_desc_k_sw128(a_u32);
          const uint64_t b_desc = make_smem_desc_k_sw128(a_u32 + Cfg::A_BYTES);
#pragma unroll
          for (int k = 0; k < Cfg::BK / Cfg::UMMA_K; ++k) {
            mma_f16_ss<kCtaGroup>(d_tmem, advance_desc_k(a_desc, k * Cfg::UMMA_K * 2),
                                  advance_desc_k(b_desc, k * Cfg::UMMA_K * 2), idesc,
                                  (kb | k) != 0 ? 1u : 0u);
          }
          // Frees the stage (in both CTAs of a pair) once these MMAs have read it.
          if constexpr (kCtaGroup == 1) tc_commit_1cta(bar_empty + 8 * s);
          else tc_commit_2cta(bar_empty + 8 * s, 0x3);
        }
        if (!ok) break;
        if constexpr (kCtaGroup == 1) tc_commit_1cta(bar_tfull + 8 * b);
        else tc_commit_2cta(bar_tfull + 8 * b, 0x3);
      }
      if (*s_abort) {
        // Wait (bounded) for the MMAs already issued before TMEM is freed.
        if constexpr (kCtaGroup == 1) tc_commit_1cta(bar_drain);
        else tc_commit_2cta(bar_drain, 0x1);
        const unsigned long long d2 = globaltimer_ns() + 2000000ull;
        for (int i = 0; i < (1 << 20); ++i) {
          if (mbar_try_wait(bar_drain, 0) || globaltimer_ns() > d2) break;
        }
      }
    }
  } else if (warp < 2 + Cfg::EPI_WARPS) {
    // ===== epilogue =====
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    const int ew = warp - 2;
    const uint32_t my_buf = epi_u32 + ew * Cfg::EPI_BUF_BYTES;
    bool ok = true;
    bool barrier_passed = !(fused_comm && p.mode == kModeGemmRs);
    int lt = 0;
    for (int t = group_id; t < num_tiles && ok; t += num_groups, ++lt) {
      int m_blk, n_blk;
      sched.tile(t, &m_blk, &n_blk);
      const int b = lt & 1;
      const int row0 = m_blk * Cfg::TILE_M + static_cast<int>(cta_rank) * Cfg::BM;  // first row of this CTA's half
      const int seg = row0 / p.seg_rows;
      const int col0 = p.epi_silu_mul ? n_blk * (Cfg::BN / 2) : n_blk * Cfg::BN;   // first output column of the tile
      __nv_bfloat16* dst0 = p.dst_base[seg] +
                            (p.dst_row_off[seg] + row0 - static_cast<long long>(seg) * p.seg_rows) * p.ldc +
                            col0;

      if (!barrier_passed) {
        // Nobody may write a peer's staging before that peer has left the
        // previous call: wait until every rank has arrived at this call.
        int good = 1;
        if (lane == 0) {
          int seen = 0;
          if (!wait_ge<true>(p.barrier[p.rank], barrier_target, s_abort, deadline, &seen)) {
            detail::report(p, s_abort, kErrStartBarrier, barrier_target, seen);
            good = 0;
          }
        }
        good = __shfl_sync(0xffffffffu, good, 0);
        if (!good) { ok = false; break; }
        barrier_passed = true;
      }

      int good = 1;
      if (lane == 0) {
        if (!mbar_wait<kCtaGroup == 2>(bar_tfull + 8 * b, (lt >> 1) & 1, s_abort, deadline)) {
          detail::report(p, s_abort, kErrEpiTmemFull, t, lt);
          good = 0;
        }
      }
      good = __shfl_sync(0xffffffffu, good, 0);
      if (!good) { ok = false; break; }
      tc_fence_after_sync();

      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) +
                             static_cast<uint32_t>(b * Cfg::BN);
      if (p.epi_silu_mul) {
        // Gate columns [0,128) and up columns [128,256) of the tile belong to the same 128 features:
        // 32 features at a time, out = silu(gate) * up, into the 256-byte rows of the warp's buffer.
#pragma unroll 1
        for (int c4 = 0; c4 < 4; ++c4) {
          uint32_t g[32], u[32];
          tmem_ld_32x32b_x32(t_row + c4 * 32, g);
          tmem_ld_32x32b_x32(t_row + Cfg::BN / 2 + c4 * 32, u);
          tmem_ld_wait();
          if (c4 == 3) {
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
              if constexpr (kCtaGroup == 1) mbar_arrive(bar_tempty + 8 * b);
              else mbar_arrive_cluster(mapa(bar_tempty + 8 * b, 0));
            }
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint32_t o[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              const float gv = __uint_as_float(g[8 * j + e]);
              o[e] = __float_as_uint(gv / (1.f + __expf(-gv)) * __uint_as_float(u[8 * j + e]));
            }
            uint4 w;
            w.x = pack_bf16x2(o[0], o[1]);
            w.y = pack_bf16x2(o[2], o[3]);
            w.z = pack_bf16x2(o[4], o[5]);
            w.w = pack_bf16x2(o[6], o[7]);
            sts_v4(my_buf + lane * 256 + (((c4 * 4 + j) ^ (lane & 7)) << 4), w);
          }
        }
        __syncwarp();
        const int ch = lane & 15;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const int r = i * 2 + (lane >> 4);
          const uint4 w = lds_v4(my_buf + r * 256 + ((ch ^ (r & 7)) << 4));
          if (row0 + q * 32 + r < p.M && col0 + ch * 8 < p.N / 2)
            st_v4(dst0 + static_cast<long long>(q * 32 + r) * p.ldc + ch * 8, w);
        }
        __syncwarp();
        continue;
      }
#pragma unroll 1
      for (int c = 0; c < Cfg::BN / Cfg::EPI_CHUNK_COLS; ++c) {
        uint32_t v0[32], v1[32];
        tmem_ld_32x32b_x32(t_row + c * Cfg::EPI_CHUNK_COLS, v0);
        tmem_ld_32x32b_x32(t_row + c * Cfg::EPI_CHUNK_COLS + 32, v1);
        tmem_ld_wait();
        if (c == Cfg::BN / Cfg::EPI_CHUNK_COLS - 1) {
          // Last read of this accumulator buffer: hand it back to the MMA issuer.
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) {
            if constexpr (kCtaGroup == 1) mbar_arrive(bar_tempty + 8 * b);
            else mbar_arrive_cluster(mapa(bar_tempty + 8 * b, 0));
          }
        }
        // The warp's buffer holds 32 rows x 128 columns (256 bytes per row), filled by two
        // 64-column TMEM reads.  Row `lane`, 16-byte slot k is stored at slot k ^ (lane & 7):
        // the row-wise writes and the transposed reads are both bank-conflict free.
        const int half = c & 1;
        if (p.epi_tma_store && half == 0) {
          // the stores of the previous pair of chunks must have read the buffer before it is rewritten
          if (lane == 0) bulk_wait_read<0>();
          __syncwarp();
        }
        // Row `lane`, 64-column half `half`: eight 16-byte slots, slot k at k ^ (lane & 7).  For the TMA
        // epilogue the two halves are two 32 x 128-byte tiles in the 128-byte-swizzle layout of the tensor
        // map; otherwise they sit side by side in 256-byte rows (the same bytes, another pitch).
        const uint32_t wr = p.epi_tma_store ? my_buf + half * 4096 + lane * 128 : my_buf + lane * 256 + half * 128;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint4 w;
          w.x = pack_bf16x2(v0[8 * j + 0], v0[8 * j + 1]);
          w.y = pack_bf16x2(v0[8 * j + 2], v0[8 * j + 3]);
          w.z = pack_bf16x2(v0[8 * j + 4], v0[8 * j + 5]);
          w.w = pack_bf16x2(v0[8 * j + 6], v0[8 * j + 7]);
          sts_v4(wr + ((j ^ (lane & 7)) << 4), w);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint4 w;
          w.x = pack_bf16x2(v1[8 * j + 0], v1[8 * j + 1]);
          w.y = pack_bf16x2(v1[8 * j + 2], v1[8 * j + 3]);
          w.z = pack_bf16x2(v1[8 * j + 4], v1[8 * j + 5]);
          w.w = pack_bf16x2(v1[8 * j + 6], v1[8 * j + 7]);
          sts_v4(wr + (((j + 4) ^ (lane & 7)) << 4), w);
        }
        if (half == 0) continue;
        if (p.epi_tma_store) {
          // every lane orders its shared-memory writes before the asynchronous proxy reads them
          fence_proxy_async();
          __syncwarp();
          if (lane == 0) {
            const int x = col0 + (c - 1) * Cfg::EPI_CHUNK_COLS;                      // a multiple of 64 elements
            const int y = row0 - seg * p.seg_rows + q * 32;                          // row inside the segment's tensor
            tma_store_2d(&omaps.m[seg], my_buf, x, y);
            tma_store_2d(&omaps.m[seg], my_buf + 4096, x + Cfg::EPI_CHUNK_COLS, y);
            bulk_commit();
          }
          continue;
        }
        __syncwarp();
        // Test knob: the last epilogue warp falls behind by several microseconds per tile, after it has
        // handed the accumulator back, so the other three run ahead of it by a tile or two.
        if ((p.ablate & 8) && ew == Cfg::EPI_WARPS - 1 && c == Cfg::BN / Cfg::EPI_CHUNK_COLS - 1) __nanosleep(8000);
        if (p.epi_st256) {
          // 8 lanes cover one row's 256 contiguous bytes with 32-byte stores; 4 rows per store instruction.
          // A lane reads its two 16-byte slots in an order that keeps each quarter-warp on 8 different banks.
          const int ch8 = lane & 7;
          const int swap = ch8 >> 2;
          const int ccol8 = (c - 1) * Cfg::EPI_CHUNK_COLS + ch8 * 16;   // column inside the tile
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int r = i * 4 + (lane >> 3);
            const uint4 wa = lds_v4(my_buf + r * 256 + (((2 * ch8 + swap) ^ (r & 7)) << 4));
            const uint4 wb = lds_v4(my_buf + r * 256 + (((2 * ch8 + 1 - swap) ^ (r & 7)) << 4));
            const uint4 lo = swap ? wb : wa, hi = swap ? wa : wb;
            const int grow = row0 + q * 32 + r;
            if (grow < p.M && col0 + ccol8 < p.N) {
              __nv_bfloat16* a = dst0 + static_cast<long long>(q * 32 + r) * p.ldc + ccol8;
              if (p.mode != kModeGemmRs || detail::in_range(p, s_abort, seg, a, 32)) {
                Vec8 v;
                v.w[0] = lo.x; v.w[1] = lo.y; v.w[2] = lo.z; v.w[3] = lo.w;
                v.w[4] = hi.x; v.w[5] = hi.y; v.w[6] = hi.z; v.w[7] = hi.w;
                st_v8(a, v);
              }
            }
          }
          __syncwarp();
          continue;
        }
        // 16 lanes cover one row's 256 contiguous bytes; 2 rows per store instruction.
        const int ch = lane & 15;
        const int ccol = (c - 1) * Cfg::EPI_CHUNK_COLS + ch * 8;   // column inside the tile
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const int r = i * 2 + (lane >> 4);
          const uint4 w = lds_v4(my_buf + r * 256 + ((ch ^ (r & 7)) << 4));
          const int grow = row0 + q * 32 + r;
          if (grow < p.M && col0 + ccol < p.N) {
            __nv_bfloat16* a = dst0 + static_cast<long long>(q * 32 + r) * p.ldc + ccol;
            // in GEMM+RS the row segment is the destination rank
            if (p.mode != kModeGemmRs || detail::in_range(p, s_abort, seg, a, 16)) st_v4(a, w);
          }
        }
        __syncwarp();   // the buffer is rewritten by the next pair of reads
      }
      if (p.mode == kModeGemmRs && p.comm_enabled) {
        // This warp's 32 rows of the tile are stored.  Publishing them needs a
        // fence at system scope, which waits for the peer's acknowledgements;
        // that wait is taken by the signalling warp, not here, so that the
        // stores of the next tile keep streaming.
        __syncwarp();
        if (lane == 0) {
          __threadfence_block();
          s_warp_tiles[ew] = lt + 1;
        }
      }
    }
    // TMA epilogue: the stores must have left shared memory and reached global memory before the CTA ends
    if (p.epi_tma_store && lane == 0) bulk_wait<0>();
  } else if (warp < Cfg::SIGNAL_WARP) {
    // ===== communication warps =====
    const int cw = warp - (2 + Cfg::EPI_WARPS);
    const int ctid = threadIdx.x - (2 + Cfg::EPI_WARPS) * 32;  // 0..127
    if (p.mode == kModeGemmRs && p.comm_enabled && !(p.ablate & 3)) {   // without tile signals there is nothing to wait for either
      // ---- reduce warps: sum the `world` staged partials of each tile of this
      // rank's segment, in the order in which the producers complete them ----
      const int items = (p.seg_rows / Cfg::BM) * sched.n_tiles;
      const int target = detail::epoch_times(epoch, p.world);
      const size_t slot_elems = static_cast<size_t>(p.seg_rows) * p.N;
      for (int j = blockIdx.x; j < items; j += gridDim.x) {
        if (ctid == 0) {
          int seen = 0;
          if (!wait_ge<true>(p.rs_tile_cnt[p.rank] + j, target, s_abort, deadline, &seen, 256)) {
            detail::report(p, s_abort, kErrRsTileCount, j, seen);
            *s_bcast = 1;
          }
        }
        named_bar_sync(2, Cfg::COMM_WARPS * 32);
        if (*s_bcast) break;
        const int seg_row = j / sched.n_tiles;
        const int n_blk = j - seg_row * sched.n_tiles;
        const int colc = ctid & 31;  // 16-byte column chunk of the 256-column tile
        const size_t tile_off = static_cast<size_t>(seg_row) * Cfg::BM * p.N + n_blk * Cfg::BN + colc * 8;
        const size_t out_off = static_cast<size_t>(seg_row) * Cfg::BM * p.ld_out + n_blk * Cfg::BN + colc * 8;
        if (p.rs_mc_stage != nullptr) {
          // this rank's segment starts at row rank * seg_rows of every rank's full-size staging
          const size_t row0 = static_cast<size_t>(p.rank) * p.seg_rows + static_cast<size_t>(seg_row) * Cfg::BM;
          detail::reduce_tile_nvls(p.rs_mc_stage + row0 * p.N + n_blk * Cfg::BN + colc * 8, p.N, p.rs_out, out_off, p.ld_out, ctid);
          continue;
        }
        switch (p.world) {
          case 1: detail::reduce_tile<1, 8>(p.rs_stage, slot_elems, tile_off, p.N, p.rs_out, out_off, p.ld_out, ctid, 1); break;
          case 2: detail::reduce_tile<2, 8>(p.rs_stage, slot_elems, tile_off, p.N, p.rs_out, out_off, p.ld_out, ctid, 2); break;
          case 4: detail::reduce_tile<4, 4>(p.rs_stage, slot_elems, tile_off, p.N, p.rs_out, out_off, p.ld_out, ctid, 4); break;
          case 8: detail::reduce_tile<8, 2>(p.rs_stage, slot_elems, tile_off, p.N, p.rs_out, out_off, p.ld_out, ctid, 8); break;
          default: detail::reduce_tile<0, 2>(p.rs_stage, slot_elems, tile_off, p.N, p.rs_out, out_off, p.ld_out, ctid, p.world); break;
        }
      }
    } else if (p.mode == kModeAgGemm && fused_comm) {
      // ---- gather warps: pull the peers' shards into the local gathered A ----
      int good = 1;
      if (lane == 0) {
        int seen = 0;
        if (!wait_ge<true>(p.barrier[p.rank], barrier_target, s_abort, deadline, &seen)) {
          detail::report(p, s_abort, kErrStartBarrier, barrier_target, seen);
          good = 0;
        }
      }
      good = __shfl_sync(0xffffffffu, good, 0);
      if (good && p.ag_push) {
        // ---- push: store this rank's own shard into every peer's gathered buffer.  Stores need no
        // round trip, so a few warps per SM reach the link rate; items go out in row order, which is
        // the order in which every consumer's schedule needs them. ----
        const int items = p.seg_rows / p.ag_item_rows;
        const int gw = blockIdx.x * p.ag_warps + cw;
        const int n_gw = gridDim.x * p.ag_warps;
        const size_t item_bytes = static_cast<size_t>(p.ag_item_rows) * p.K * 2;
        for (int j = cw < p.ag_warps ? gw : items; j < items; j += n_gw) {
          const size_t grow = static_cast<size_t>(p.rank) * p.seg_rows + static_cast<size_t>(j) * p.ag_item_rows;
          const size_t boff = grow * p.K * 2;
          const char* src = reinterpret_cast<const char*>(p.ag_full) + boff;
          constexpr int kUnroll = 4;
          size_t off = static_cast<size_t>(lane) * 16;
          for (; off + (kUnroll - 1) * 512 < item_bytes; off += kUnroll * 512) {
            uint4 w[kUnroll];
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) w[u] = ld_v4_stream(src + off + u * 512);
            for (int step = 1; step < p.world; ++step) {
              const int peer = (p.rank + step) % p.world;
              char* dst = reinterpret_cast<char*>(p.ag_dst[peer]) + boff;
              if (!detail::in_range(p, s_abort, peer, dst + off, kUnroll * 512)) continue;
#pragma unroll
              for (int u = 0; u < kUnroll; ++u) st_v4(dst + off + u * 512, w[u]);
            }
          }
          for (; off < item_bytes; off += 512) {
            const uint4 w = ld_v4_stream(src + off);
            for (int step = 1; step < p.world; ++step)
              st_v4(reinterpret_cast<char*>(p.ag_dst[(p.rank + step) % p.world]) + boff + off, w);
          }
          // Every lane's stores are performed at system scope, then one lane per peer signals.
          fence_sys();
          __syncwarp();
          if (lane < p.world && lane != p.rank) red_relaxed_sys_add(p.ag_flag_peer[lane] + static_cast<int>(grow / p.gather_rows), 1);
        }
      } else if (good) {
        const int items_per_seg = p.seg_rows / p.ag_item_rows;
        const int total = (p.world - 1) * items_per_seg;
        const int gw = blockIdx.x * p.ag_warps + cw;
        const int n_gw = gridDim.x * p.ag_warps;
        const size_t item_bytes = static_cast<size_t>(p.ag_item_rows) * p.K * 2;
        for (int j = cw < p.ag_warps ? gw : total; j < total; j += n_gw) {
          const int step = j / items_per_seg + 1;
          const int i = j - (step - 1) * items_per_seg;
          const int seg = (p.rank + step) % p.world;
          const size_t row_in_seg = static_cast<size_t>(i) * p.ag_item_rows;
          const char* src = reinterpret_cast<const char*>(p.ag_src[seg] + row_in_seg * p.K);
          if (!detail::in_range(p, s_abort, seg, src, static_cast<unsigned>(item_bytes))) continue;
          const size_t grow = static_cast<size_t>(seg) * p.seg_rows + row_in_seg;
          char* dst = reinterpret_cast<char*>(p.ag_full + grow * p.K);
          if (p.ag_vec32) detail::copy_item<Vec8, 4>(src, dst, item_bytes, lane);
          else detail::copy_item<uint4, 8>(src, dst, item_bytes, lane);
          // The consumer of these rows is TMA (async proxy) on another SM.
          fence_proxy_async();
          __syncwarp();
          if (lane == 0) red_release_gpu_add(p.ag_flags + static_cast<int>(grow / p.gather_rows), 1);
        }
        // Tell the peers when this rank has read everything it needs from them:
        // the last gather warp of the grid sends one signal per peer.
        if (lane == 0 && cw < p.ag_warps) {
          const int done = atom_add_acq_rel_gpu(p.ag_done, 1) + 1;
          if (done == detail::epoch_times(epoch, n_gw)) {
            for (int s = 0; s < p.world; ++s)
              if (s != p.rank) red_release_sys_add(p.ag_read_done[s], 1);
          }
        }
        // One warp keeps the kernel alive until every peer has finished reading
        // this rank's shard, so the caller may overwrite it after the kernel.
        if (blockIdx.x == 0 && cw == 0 && lane == 0) {
          int seen = 0;
          if (!wait_ge<true>(p.ag_read_done[p.rank], detail::epoch_times(epoch, p.world - 1), s_abort, deadline, &seen, 512)) {
            detail::report(p, s_abort, kErrAgEndBarrier, detail::epoch_times(epoch, p.world - 1), seen);
          }
        }
      }
    }
  }

  else {
    // ===== signalling warp (GEMM+RS) =====
    // Walks the same tile sequence as the epilogue.  Whenever more tiles have
    // been stored by all four epilogue warps, one fence at system scope orders
    // every store observed so far, then each finished tile's owner gets +1 on
    // the tile's counter.  One fence may cover several tiles.
    if (p.mode == kModeGemmRs && p.comm_enabled && !(p.ablate & 2) && lane == 0) {
      int signalled = 0;
      int t = group_id;
      unsigned spins = 0;
      // A fence at system scope holds this SM's stores back until the peers have acknowledged everything in
      // flight (a link round trip), so it is not taken per tile: finished tiles accumulate up to a batch, and the
      // tail of this CTA's tile list goes out as soon as it is stored.
      const int my_tiles = group_id < num_tiles ? (num_tiles - group_id + num_groups - 1) / num_groups : 0;
      const int batch = p.rs_signal_batch > 0 ? p.rs_signal_batch : 1;
      while (t < num_tiles) {
        // A tile is finished when every epilogue warp has stored its 32 rows of it.  The warps are not in
        // lock step (a warp may be a tile or two ahead of the slowest one), so the count is the minimum of
        // the per-warp counters, never their sum.
        int done = s_warp_tiles[0];
#pragma unroll
        for (int w = 1; w < Cfg::EPI_WARPS; ++w) done = min(done, s_warp_tiles[w]);
        if (done - signalled >= batch || (done > signalled && done == my_tiles)) {
          fence_sys();
          for (; signalled < done && t < num_tiles; ++signalled, t += num_groups) {
            int m_blk, n_blk;
            sched.tile(t, &m_blk, &n_blk);
            const int row0 = m_blk * Cfg::TILE_M + static_cast<int>(cta_rank) * Cfg::BM;
            const int seg = row0 / p.seg_rows;
            const int seg_row = (row0 - seg * p.seg_rows) / Cfg::BM;
            red_relaxed_sys_add(p.rs_tile_cnt[seg] + seg_row * sched.n_tiles + n_blk, 1);
          }
          spins = 0;
        } else {
          __nanosleep(100);
          if ((++spins & 63u) == 0u && (*s_abort != 0 || globaltimer_ns() > deadline)) break;
        }
      }
    }
  }

  // ---- tear-down ------------------------------------------------------------
  tc_fence_before_sync();
  __syncthreads();
  if constexpr (kCtaGroup == 2) {
    // The peer CTA may still be read by the leader's MMAs or signal our barriers.
    cluster_arrive();
    cluster_wait();
  }
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc<kCtaGroup>(tmem_base, Cfg::TMEM_COLS);
  }
  if (p.epoch_dev != nullptr && threadIdx.x == 0) {
    // Count this CTA out; the last one resets the count and advances the plan's call number.
    __threadfence();
    if (atomicAdd(p.epoch_dev + 1, 1) == static_cast<int>(gridDim.x) - 1) {
      p.epoch_dev[1] = 0;
      __threadfence();
      atomicAdd(p.epoch_dev, 1);
    }
  }
}

}  // namespace tcl
