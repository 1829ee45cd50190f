// Host side of libtileccl.so: plan construction / validation / launch for the
// sm_100a GEMM family, and the small stand-alone kernels (device barrier,
// SiLU*mul, N(0,1) fill, verify).  See tileccl_ops.h for the contract.
#include "tileccl_ops.h"

#include <cstdio>
#include <cstddef>
#include <cstring>
#include <new>

#include "../gemm/gemm_sm100.cuh"

namespace {

using namespace tcl;

// Finished tiles per system-scope fence of the GEMM+RS signalling warp when the caller does not say.
constexpr int kDefaultRsSignalBatch = 4;

struct GemmPlan {
  CUtensorMap tmap_a;
  CUtensorMap tmap_b;
  GemmParams params;
  OutMaps omaps;     // encoded only for the TMA-store epilogue
  int cta_group;
  int grid;
  int lda, ldb;      // operand row pitches (elements), kept for tcl_gemm_plan_set_operands
  const void* a_ptr;
};

void set_err(char* err, int errlen, const char* msg) {
  if (err && errlen > 0) {
    std::snprintf(err, static_cast<size_t>(errlen), "%s", msg);
  }
}

// Opt-in to the kernel's dynamic shared memory on the current device.  Called when a plan is created (plans
// are per device), so that a launch touches no host state shared between threads.
template <int G>
cudaError_t prepare_gemm() {
  return cudaFuncSetAttribute(gemm_sm100_kernel<G>, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmCfg<G>::SMEM_BYTES);
}

template <int G>
cudaError_t launch_gemm(const GemmPlan* pl, const GemmParams& params, cudaStream_t stream) {
  using Cfg = GemmCfg<G>;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(pl->grid), 1, 1);
  cfg.blockDim = dim3(Cfg::THREADS, 1, 1);
  cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = G;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, gemm_sm100_kernel<G>, pl->tmap_a, pl->tmap_b, params, pl->omaps);
}

// ---------------------------------------------------------------------------
// Device barrier (stand-alone form of the barrier built into the fused kernels)
// ---------------------------------------------------------------------------
struct BarrierArgs {
  int* counters[kMaxWorld];
};

__global__ void barrier_all_kernel(BarrierArgs a, int world, int rank, int epoch, int* status,
                                   unsigned long long timeout_ns) {
  const int lane = threadIdx.x;
  if (lane < world) ptx::red_release_sys_add(a.counters[lane], 1);
  if (lane == 0) {
    const unsigned long long deadline = ptx::globaltimer_ns() + timeout_ns;
    int seen = 0;
    const int target = static_cast<int>(static_cast<unsigned>(epoch) * static_cast<unsigned>(world));  // may wrap
    if (!ptx::wait_ge<true>(a.counters[rank], target, nullptr, deadline, &seen)) {
      if (atomicCAS(status, 0, kErrStartBarrier) == 0) {
        status[1] = rank;
        status[2] = target;
        status[3] = seen;
      }
    }
  }
}

// ---------------------------------------------------------------------------
// SiLU(gate) * up
// ---------------------------------------------------------------------------
__global__ void silu_mul_kernel(const uint4* __restrict__ gu, uint4* __restrict__ out, long long rows,
                                long long ffn8) {
  // One thread per 8 output elements; a row of gu holds 2*ffn8 chunks.  Two independent chunks
  // (four 16-byte loads) are in flight per thread per iteration.
  const long long total = rows * ffn8;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  auto one = [](const uint4& g, const uint4& u) {
    const uint32_t gw[4] = {g.x, g.y, g.z, g.w};
    const uint32_t uw[4] = {u.x, u.y, u.z, u.w};
    uint32_t ow[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float g0 = __uint_as_float(gw[e] << 16), g1 = __uint_as_float(gw[e] & 0xffff0000u);
      const float u0 = __uint_as_float(uw[e] << 16), u1 = __uint_as_float(uw[e] & 0xffff0000u);
      const float o0 = g0 / (1.f + __expf(-g0)) * u0;
      const float o1 = g1 / (1.f + __expf(-g1)) * u1;
      ow[e] = ptx::pack_bf16x2(__float_as_uint(o0), __float_as_uint(o1));
    }
    return make_uint4(ow[0], ow[1], ow[2], ow[3]);
  };
  long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  for (; i + stride < total; i += 2 * stride) {
    const long long j = i + stride;
    const long long r0 = i / ffn8, c0 = i - r0 * ffn8, r1 = j / ffn8, c1 = j - r1 * ffn8;
    const uint4 ga = gu[r0 * 2 * ffn8 + c0], ua = gu[r0 * 2 * ffn8 + ffn8 + c0];
    const uint4 gb = gu[r1 * 2 * ffn8 + c1], ub = gu[r1 * 2 * ffn8 + ffn8 + c1];
    out[i] = one(ga, ua);
    out[j] = one(gb, ub);
  }
  for (; i < total; i += stride) {
    const long long r = i / ffn8, c = i - r * ffn8;
    out[i] = one(gu[r * 2 * ffn8 + c], gu[r * 2 * ffn8 + ffn8 + c]);
  }
}

// ---------------------------------------------------------------------------
// N(mean, std) bf16 fill: counter-based hash -> two uniforms -> Box-Muller.
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint64_t mix64(uint64_t z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

__global__ void fill_normal_bf16_kernel(__nv_bfloat16* dst, long long n, uint64_t seed, float mean,
                                        float stdv) {
  // Each thread produces a pair (2i, 2i+1) from one hash value.
  const long long pairs = (n + 1) / 2;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < pairs;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const uint64_t h = mix64(seed * 0xD1342543DE82EF95ull + static_cast<uint64_t>(i));
    const float u1 = (static_cast<float>(static_cast<uint32_t>(h >> 40)) + 1.0f) * (1.0f / 16777217.0f);
    const float u2 = static_cast<float>(static_cast<uint32_t>(h) >> 8) * (1.0f / 16777216.0f);
    const float rad = sqrtf(-2.0f * __logf(u1));
    float s, c;
    __sincosf(6.283185307179586f * u2, &s, &c);
    dst[2 * i] = __float2bfloat16_rn(mean + stdv * rad * c);
    if (2 * i + 1 < n) dst[2 * i + 1] = __float2bfloat16_rn(mean + stdv * rad * s);
  }
}

// ---------------------------------------------------------------------------
// Verify: max |got - ref| / (|ref| + 1).  Two passes through a scratch array
// of per-block maxima.
// ---------------------------------------------------------------------------
constexpr int kVerifyBlocks = 1024;

__global__ void max_rel_err_partial(const __nv_bfloat16* got, const float* ref, long long n,
                                    float* scratch) {
  float m = 0.f;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float r = ref[i];
    const float g = __bfloat162float(got[i]);
    float e = fabsf(g - r) / (fabsf(r) + 1.f);
    if (!(e == e)) e = 3.4e38f;  // NaN counts as the worst error
    m = fmaxf(m, e);
  }
  __shared__ float sm[256];
  sm[threadIdx.x] = m;
  __syncthreads();
  for (int s = 128; s > 0; s >>= 1) {
    if (threadIdx.x < s) sm[threadIdx.x] = fmaxf(sm[threadIdx.x], sm[threadIdx.x + s]);
    __syncthreads();
  }
  if (threadIdx.x == 0) scratch[blockIdx.x] = sm[0];
}

__global__ void max_rel_err_final(const float* scratch, int nblocks, float* result) {
  __shared__ float sm[256];
  float m = 0.f;
  for (int i = threadIdx.x; i < nblocks; i += blockDim.x) m = fmaxf(m, scratch[i]);
  sm[threadIdx.x] = m;
  __syncthreads();
  for (int s = 128; s > 0; s >>= 1) {
    if (threadIdx.x < s) sm[threadIdx.x] = fmaxf(sm[threadIdx.x], sm[threadIdx.x + s]);
    __syncthreads();
  }
  if (threadIdx.x == 0) result[0] = sm[0];
}

}  // namespace

extern "C" {

int tcl_gemm_desc_size(void) { return static_cast<int>(sizeof(tcl_gemm_desc)); }

int tcl_gemm_desc_offset(const char* field) {
  if (!field) return -1;
#define TCL_OFF(name) if (std::strcmp(field, #name) == 0) return static_cast<int>(offsetof(tcl_gemm_desc, name));
  TCL_OFF(mode) TCL_OFF(M) TCL_OFF(lda) TCL_OFF(A) TCL_OFF(world) TCL_OFF(seg_rows) TCL_OFF(dst_base) TCL_OFF(dst_row_off)
  TCL_OFF(rs_tile_cnt) TCL_OFF(rs_stage) TCL_OFF(rs_chunks) TCL_OFF(ag_src) TCL_OFF(ag_flags) TCL_OFF(gather_rows) TCL_OFF(ag_done)
  TCL_OFF(ag_push) TCL_OFF(ag_dst) TCL_OFF(barrier) TCL_OFF(status) TCL_OFF(timeout_ns) TCL_OFF(group_m) TCL_OFF(rs_mc_stage)
  TCL_OFF(range_lo) TCL_OFF(epi_silu_mul) TCL_OFF(ablate) TCL_OFF(epi_st256) TCL_OFF(epi_tma_store) TCL_OFF(epoch_dev) TCL_OFF(ag_warps) TCL_OFF(rs_signal_batch) TCL_OFF(ag_vec32)
#undef TCL_OFF
  return -1;
}

int tcl_gemm_smem_bytes(int cta_group) {
  return cta_group == 2 ? GemmCfg<2>::SMEM_BYTES : GemmCfg<1>::SMEM_BYTES;
}

void tcl_sched_tile(int m_tiles, int n_tiles, int group_m, int order, int world, int rank,
                    int rs_chunks, int t, int* m_blk, int* n_blk) {
  TileSched s{m_tiles, n_tiles, group_m, order, world, rank, rs_chunks};
  s.tile(t, m_blk, n_blk);
}

void* tcl_gemm_plan_create(const tcl_gemm_desc* d, char* err, int errlen) {
  const int G = d->cta_group;
  if (G != 1 && G != 2) { set_err(err, errlen, "cta_group must be 1 or 2"); return nullptr; }
  const int tile_m = 128 * G;
  if (d->M <= 0 || d->N <= 0 || d->K <= 0) { set_err(err, errlen, "M, N, K must be positive"); return nullptr; }
  if (d->M % tile_m != 0) { set_err(err, errlen, "M must be a multiple of 128 * cta_group"); return nullptr; }
  if (d->N % 256 != 0) { set_err(err, errlen, "N must be a multiple of 256"); return nullptr; }
  if (d->K % 8 != 0 || d->lda % 8 != 0 || d->ldb % 8 != 0 || d->ldc % 8 != 0) {
    set_err(err, errlen, "K and the row pitches must be multiples of 8 elements (16 bytes)");
    return nullptr;
  }
  if ((reinterpret_cast<uintptr_t>(d->A) & 15) || (reinterpret_cast<uintptr_t>(d->B) & 15)) {
    set_err(err, errlen, "A and B must be 16-byte aligned");
    return nullptr;
  }
  if (d->world < 1 || d->world > TCL_MAX_WORLD || d->rank < 0 || d->rank >= d->world) {
    set_err(err, errlen, "world must be 1..8 and rank inside it");
    return nullptr;
  }
  if (d->seg_rows <= 0 || d->seg_rows % tile_m != 0 || d->M % d->seg_rows != 0 ||
      d->M / d->seg_rows > TCL_MAX_WORLD) {
    set_err(err, errlen, "seg_rows must divide M into at most 8 segments of whole tiles");
    return nullptr;
  }
  const int nseg = d->M / d->seg_rows;
  for (int s = 0; s < nseg; ++s) {
    if (!d->dst_base[s] || (reinterpret_cast<uintptr_t>(d->dst_base[s]) & 15)) {
      set_err(err, errlen, "every dst_base must be set and 16-byte aligned");
      return nullptr;
    }
  }
  if (!d->status) { set_err(err, errlen, "status buffer missing"); return nullptr; }

  GemmPlan* pl = new (std::nothrow) GemmPlan();
  if (!pl) { set_err(err, errlen, "out of host memory"); return nullptr; }
  std::memset(pl, 0, sizeof(*pl));
  GemmParams& p = pl->params;
  p.mode = d->mode;
  p.M = d->M; p.N = d->N; p.K = d->K; p.ldc = d->ldc;
  p.world = d->world; p.rank = d->rank;
  p.comm_enabled = d->comm_enabled;
  p.ablate = d->ablate;
  p.epi_silu_mul = d->epi_silu_mul;
  p.epi_st256 = d->epi_st256;
  p.epoch_dev = d->epoch_dev;
  p.epi_tma_store = d->epi_tma_store;
  if (d->epi_tma_store) {
    if (d->epi_silu_mul || d->epi_st256 || (d->mode == TCL_MODE_GEMM_RS && d->comm_enabled)) {
      set_err(err, errlen, "epi_tma_store excludes epi_silu_mul, epi_st256 and the communicating GEMM+RS");
      delete pl;
      return nullptr;
    }
    for (int s = 0; s < nseg; ++s) {
      const __nv_bfloat16* base = static_cast<const __nv_bfloat16*>(d->dst_base[s]) + d->dst_row_off[s] * static_cast<long long>(d->ldc);
      if (ptx::encode_tmap_bf16_k64(&pl->omaps.m[s], base, static_cast<uint64_t>(d->seg_rows), static_cast<uint64_t>(d->N),
                                    static_cast<uint64_t>(d->ldc), 32) != 0) {
        set_err(err, errlen, "cuTensorMapEncodeTiled failed for an output segment");
        delete pl;
        return nullptr;
      }
    }
  }
  if (d->epi_st256) {
    bool aligned = d->ldc % 16 == 0 && !d->epi_silu_mul;
    for (int s = 0; s < nseg; ++s) aligned = aligned && (reinterpret_cast<uintptr_t>(d->dst_base[s]) & 31) == 0;
    if (!aligned) { set_err(err, errlen, "epi_st256 needs 32-byte aligned dst_base, ldc a multiple of 16 and no epi_silu_mul"); delete pl; return nullptr; }
  }
  if (d->epi_silu_mul && d->mode == TCL_MODE_GEMM_RS) { set_err(err, errlen, "epi_silu_mul is not available for GEMM+RS"); delete pl; return nullptr; }
  p.seg_rows = d->seg_rows;
  for (int s = 0; s < TCL_MAX_WORLD; ++s) {
    p.dst_base[s] = static_cast<__nv_bfloat16*>(d->dst_base[s]);
    p.dst_row_off[s] = d->dst_row_off[s];
    p.rs_tile_cnt[s] = d->rs_tile_cnt[s];
    p.ag_src[s] = static_cast<const __nv_bfloat16*>(d->ag_src[s]);
    p.ag_read_done[s] = d->ag_read_done[s];
    p.ag_dst[s] = static_cast<__nv_bfloat16*>(d->ag_dst[s]);
    p.range_lo[s] = d->range_lo[s];
    p.range_hi[s] = d->range_hi[s] ? d->range_hi[s] : ~0ull;
    p.ag_flag_peer[s] = d->ag_flag_peer[s];
    p.barrier[s] = d->barrier[s];
  }
  p.status = d->status;
  p.timeout_ns = d->timeout_ns ? d->timeout_ns : 4000000000ull;

  TileSched& sc = p.sched;
  sc.m_tiles = d->M / tile_m;
  sc.n_tiles = d->N / 256;
  sc.world = 1; sc.rank = 0; sc.rs_chunks = 1; sc.order = kOrderPlain;
  sc.group_m = d->group_m > 0 ? d->group_m : (G == 2 ? 8 : 16);

  auto fail = [&](const char* m) -> void* { set_err(err, errlen, m); delete pl; return nullptr; };

  if (d->mode == TCL_MODE_GEMM_RS) {
    if (nseg != d->world) return fail("GEMM+RS: M / seg_rows must equal world");
    if (d->ldc != d->N) return fail("GEMM+RS: staging pitch (ldc) must equal N");
    sc.order = kOrderRsPush; sc.world = d->world; sc.rank = d->rank;
    const int st = sc.m_tiles / d->world;
    // Default: one tile row per step (rs_chunks = tile rows of a segment) and a
    // raster group that spans every segment, so that the tiles in flight at any
    // instant target all owners evenly whatever the drift between ranks.
    int g = d->rs_chunks > 0 ? d->rs_chunks : st;
    if (st % g != 0) return fail("GEMM+RS: rs_chunks must divide the tile rows of a segment");
    sc.rs_chunks = g;
    if (d->group_m <= 0) {
      const int per = 8 / d->world > 0 ? 8 / d->world : 1;
      sc.group_m = d->world * per;
    }
    if (d->comm_enabled) {
      if (!d->rs_stage || !d->rs_out || d->ld_out % 8 != 0 || d->ld_out < d->N)
        return fail("GEMM+RS: rs_stage / rs_out / ld_out invalid");
      for (int s = 0; s < d->world; ++s) {
        if (!d->rs_tile_cnt[s]) return fail("GEMM+RS: rs_tile_cnt missing for a rank");
        if (d->world > 1 && !d->barrier[s]) return fail("GEMM+RS: barrier counter missing for a rank");
      }
    }
    p.rs_stage = static_cast<const __nv_bfloat16*>(d->rs_stage);
    p.rs_out = static_cast<__nv_bfloat16*>(d->rs_out);
    p.ld_out = d->ld_out;
    p.rs_mc_stage = static_cast<const __nv_bfloat16*>(d->rs_mc_stage);
    p.rs_signal_batch = d->rs_signal_batch > 0 ? d->rs_signal_batch : kDefaultRsSignalBatch;
  } else if (d->mode == TCL_MODE_AG_GEMM) {
    if (nseg != d->world) return fail("AG+GEMM: M / seg_rows must equal world");
    if (d->lda != d->K) return fail("AG+GEMM: gathered A must be dense (lda == K)");
    sc.order = d->ag_push ? kOrderAgPush : kOrderAgPull; sc.world = d->world; sc.rank = d->rank;
    p.ag_push = d->ag_push;
    if (d->ag_push && d->group_m <= 0 && d->world > 1) {
      // keep one raster group inside a band of schedule rows that arrive together
      const int band = d->world - 1;
      sc.group_m = band >= 4 ? band : band * (8 / band > 0 ? 8 / band : 1);
    }
    if (d->comm_enabled && d->world > 1) {
      if (d->gather_rows < 128 || d->gather_rows % tile_m != 0 && d->gather_rows % 128 != 0)
        return fail("AG+GEMM: gather_rows must be a multiple of 128");
      if (d->gather_rows % 128 != 0 || d->seg_rows % d->gather_rows != 0)
        return fail("AG+GEMM: gather_rows must be a multiple of 128 that divides seg_rows");
      if (!d->ag_flags || !d->ag_done) return fail("AG+GEMM: flag buffers missing");
      for (int s = 0; s < d->world; ++s) {
        if (!d->ag_src[s] || !d->ag_read_done[s] || !d->barrier[s])
          return fail("AG+GEMM: peer pointers missing for a rank");
        if (d->ag_push && (!d->ag_dst[s] || !d->ag_flag_peer[s])) return fail("AG+GEMM push: peer buffers missing for a rank");
        if (reinterpret_cast<uintptr_t>(d->ag_src[s]) & 15) return fail("AG+GEMM: ag_src must be 16-byte aligned");
      }
    }
    p.ag_full = static_cast<__nv_bfloat16*>(const_cast<void*>(d->A));
    p.ag_flags = d->ag_flags;
    p.gather_rows = d->gather_rows > 0 ? d->gather_rows : d->seg_rows;
    p.ag_done = d->ag_done;
    p.ag_item_rows = d->ag_item_rows > 0 ? d->ag_item_rows : 1;
    p.ag_vec32 = d->ag_vec32 ? 1 : 0;
    if (p.ag_vec32 && (d->K % 16 != 0 || (reinterpret_cast<uintptr_t>(d->A) & 31))) return fail("AG+GEMM: ag_vec32 needs K % 16 == 0 and a 32-byte aligned gathered buffer");
    if (p.ag_vec32 && d->comm_enabled && d->world > 1)
      for (int s = 0; s < d->world; ++s)
        if (reinterpret_cast<uintptr_t>(d->ag_src[s]) & 31) return fail("AG+GEMM: ag_vec32 needs 32-byte aligned ag_src");
    p.ag_warps = d->ag_warps > 0 ? d->ag_warps : GemmCfg<1>::COMM_WARPS;
    if (p.ag_warps > GemmCfg<1>::COMM_WARPS) return fail("AG+GEMM: ag_warps must lie in 1..4");
    if (p.gather_rows % p.ag_item_rows != 0) return fail("AG+GEMM: ag_item_rows must divide gather_rows");
  } else if (d->mode != TCL_MODE_PLAIN) {
    return fail("unknown mode");
  } else {
    p.comm_enabled = 0;
  }

  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
    return fail("no CUDA device");
  int grid = d->num_ctas > 0 ? d->num_ctas : sms;
  if (grid > sms) grid = sms;
  const int max_useful = sc.num_tiles() * G;
  if (grid > max_useful && d->mode == TCL_MODE_PLAIN) grid = max_useful;
  grid -= grid % G;
  if (grid < G) return fail("grid too small");
  pl->grid = grid;
  pl->cta_group = G;
  pl->lda = d->lda;
  pl->ldb = d->ldb;
  pl->a_ptr = d->A;
  if ((G == 2 ? prepare_gemm<2>() : prepare_gemm<1>()) != cudaSuccess) return fail("cudaFuncSetAttribute (dynamic shared memory) failed");

  const int box_b = 256 / G;
  int r = ptx::encode_tmap_bf16_k64(&pl->tmap_a, d->A, static_cast<uint64_t>(d->M),
                                    static_cast<uint64_t>(d->K), static_cast<uint64_t>(d->lda), 128);
  if (r != 0) return fail("cuTensorMapEncodeTiled failed for A");
  r = ptx::encode_tmap_bf16_k64(&pl->tmap_b, d->B, static_cast<uint64_t>(d->N),
                                static_cast<uint64_t>(d->K), static_cast<uint64_t>(d->ldb),
                                static_cast<uint32_t>(box_b));
  if (r != 0) return fail("cuTensorMapEncodeTiled failed for B");
  return pl;
}

int tcl_gemm_plan_run(void* plan, int epoch, void* stream) {
  GemmPlan* pl = static_cast<GemmPlan*>(plan);
  if (!pl) return static_cast<int>(cudaErrorInvalidValue);
  // The call number travels in a copy of the parameters: a launch does not write to the plan.
  GemmParams params = pl->params;
  params.epoch = epoch;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e = pl->cta_group == 2 ? launch_gemm<2>(pl, params, st) : launch_gemm<1>(pl, params, st);
  return static_cast<int>(e);
}

int tcl_gemm_plan_set_operands(void* plan, const void* A, const void* B) {
  GemmPlan* pl = static_cast<GemmPlan*>(plan);
  if (!pl || !A || !B) return static_cast<int>(cudaErrorInvalidValue);
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) return static_cast<int>(cudaErrorMisalignedAddress);
  if (pl->params.mode == kModeAgGemm && A != pl->a_ptr) return static_cast<int>(cudaErrorInvalidValue);  // A is the gathered buffer the plan was built on
  CUtensorMap ta, tb;
  if (ptx::encode_tmap_bf16_k64(&ta, A, static_cast<uint64_t>(pl->params.M), static_cast<uint64_t>(pl->params.K),
                                static_cast<uint64_t>(pl->lda), 128) != 0 ||
      ptx::encode_tmap_bf16_k64(&tb, B, static_cast<uint64_t>(pl->params.N), static_cast<uint64_t>(pl->params.K),
                                static_cast<uint64_t>(pl->ldb), static_cast<uint32_t>(256 / pl->cta_group)) != 0)
    return static_cast<int>(cudaErrorInvalidValue);
  pl->tmap_a = ta;
  pl->tmap_b = tb;
  pl->a_ptr = A;
  return 0;
}

void tcl_gemm_plan_destroy(void* plan) { delete static_cast<GemmPlan*>(plan); }
int tcl_gemm_plan_grid(void* plan) { return plan ? static_cast<GemmPlan*>(plan)->grid : 0; }
int tcl_gemm_plan_launches(void* plan) { return plan ? 1 : 0; }

int tcl_barrier_all(int32_t* const* counters, int world, int rank, int epoch, int32_t* status,
                    uint64_t timeout_ns, void* stream) {
  if (world < 1 || world > TCL_MAX_WORLD || rank < 0 || rank >= world) return static_cast<int>(cudaErrorInvalidValue);
  BarrierArgs a = {};
  for (int i = 0; i < world; ++i) a.counters[i] = counters[i];
  barrier_all_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
      a, world, rank, epoch, status, timeout_ns ? timeout_ns : 4000000000ull);
  return static_cast<int>(cudaGetLastError());
}

int tcl_silu_mul(const void* gate_up, void* out, int64_t rows, int64_t ffn, void* stream) {
  if (ffn % 8 != 0 || rows <= 0) return static_cast<int>(cudaErrorInvalidValue);
  const long long total = rows * (ffn / 8);
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  silu_mul_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(gate_up), static_cast<uint4*>(out), rows, ffn / 8);
  return static_cast<int>(cudaGetLastError());
}

int tcl_fill_normal_bf16(void* dst, int64_t n, uint64_t seed, float mean, float stdv, void* stream) {
  if (n <= 0) return 0;
  long long blocks = ((n + 1) / 2 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  fill_normal_bf16_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16*>(dst), n, seed, mean, stdv);
  return static_cast<int>(cudaGetLastError());
}

int tcl_max_rel_err(const void* got_bf16, const float* ref, int64_t n, float* scratch, float* result,
                    void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  long long blocks = (n + 255) / 256;
  if (blocks > kVerifyBlocks) blocks = kVerifyBlocks;
  if (blocks < 1) blocks = 1;
  max_rel_err_partial<<<static_cast<unsigned>(blocks), 256, 0, st>>>(
      static_cast<const __nv_bfloat16*>(got_bf16), ref, n, scratch);
  max_rel_err_final<<<1, 256, 0, st>>>(scratch, static_cast<int>(blocks), result);
  return static_cast<int>(cudaGetLastError());
}

// Descriptor encoders, exposed so that their bit layouts can be checked on a machine without a GPU.
uint64_t tcl_make_smem_desc_k_sw128(uint32_t smem_addr) { return tcl::ptx::make_smem_desc_k_sw128(smem_addr); }
uint64_t tcl_advance_desc_k(uint64_t desc, uint32_t bytes) { return tcl::ptx::advance_desc_k(desc, bytes); }
uint32_t tcl_make_idesc_bf16_f32(uint32_t m, uint32_t n) { return tcl::ptx::make_idesc_bf16_f32(m, n); }

int tcl_debug_bounds_enabled(void) {
#ifdef TCL_DEBUG_BOUNDS
  return 1;
#else
  return 0;
#endif
}

const char* tcl_status_string(int code) {
  switch (code) {
    case kOk: return "ok";
    case kErrProducerEmpty: return "TMA producer timed out waiting for a free stage";
    case kErrMmaFull: return "MMA issuer timed out waiting for operands";
    case kErrMmaTmemEmpty: return "MMA issuer timed out waiting for a drained accumulator";
    case kErrEpiTmemFull: return "epilogue timed out waiting for an accumulator";
    case kErrStartBarrier: return "a peer never arrived at the start barrier";
    case kErrRsTileCount: return "reduce warps timed out waiting for a tile's partials";
    case kErrAgFlag: return "TMA producer timed out waiting for a gathered row block";
    case kErrAgEndBarrier: return "a peer never finished reading this rank's shard";
    case kErrBounds: return "debug build: an address fell outside its rank's mapped range (access skipped)";
    default: return "unknown status";
  }
}

}  // extern "C"
