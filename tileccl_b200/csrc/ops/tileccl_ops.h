/* C interface of libtileccl.so: GEMM plans (plain, fused GEMM->reduce-scatter,
 * fused all-gather->GEMM), the device barrier, the fused SiLU*mul, fill and
 * verify kernels.  Everything takes raw device pointers and a CUDA stream so
 * that Python (ctypes), the C++ benchmarks and other runtimes can call it.
 *
 * Reference parity: the init-once / run-many GEMM wrapper
 * (comm_comp/gemm_sm90.cuh:99-140), the fused kernel's arguments
 * (comm_comp/rs_dma_sm90.cuh:93-126), barrier_all_on_stream
 * (comm_comp/ipc_multiproc.cuh:184-201), verify_kernel
 * (comm_comp/exp3_gemm_rs_fused.cu:252-270), fill_half
 * (comm_comp/common.cuh:190-223).
 */
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TCL_MAX_WORLD 8

enum { TCL_MODE_PLAIN = 0, TCL_MODE_GEMM_RS = 1, TCL_MODE_AG_GEMM = 2 };

typedef struct tcl_gemm_desc {
  int32_t mode;         /* TCL_MODE_* */
  int32_t cta_group;    /* 1: one CTA per 128x256 tile; 2: CTA pair per 256x256 tile */
  int32_t M, N, K;      /* A is [M,K] (gathered size for AG), B is [N,K], D is [M,N] */
  int32_t lda, ldb, ldc;/* row pitches in elements */
  const void* A;        /* local; for TCL_MODE_AG_GEMM the gathered buffer ag_full */
  const void* B;
  int32_t world, rank;
  int32_t seg_rows;     /* rows per output segment (M for a single segment) */
  int32_t comm_enabled; /* 0: same schedule, no peer traffic, no flags (the "ctrl" variant) */
  void* dst_base[TCL_MAX_WORLD];
  int64_t dst_row_off[TCL_MAX_WORLD];
  /* GEMM+RS */
  int32_t* rs_tile_cnt[TCL_MAX_WORLD];
  const void* rs_stage;
  void* rs_out;
  int32_t ld_out;
  int32_t rs_chunks;
  /* AG+GEMM */
  const void* ag_src[TCL_MAX_WORLD];
  int32_t* ag_flags;
  int32_t gather_rows;
  int32_t ag_item_rows; /* rows per gather work item; 0 = 1 row */
  int32_t* ag_done;
  int32_t* ag_read_done[TCL_MAX_WORLD];
  int32_t ag_push;       /* 0 = gather warps load from peers, 1 = they store the own shard to every peer */
  void* ag_dst[TCL_MAX_WORLD];        /* push: rank s's gathered buffer */
  int32_t* ag_flag_peer[TCL_MAX_WORLD]; /* push: rank s's row-block counters */
  /* common */
  int32_t* barrier[TCL_MAX_WORLD];
  int32_t* status;      /* 4 ints, zeroed by the caller */
  uint64_t timeout_ns;  /* bound of every device-side wait; 0 = 4 s */
  int32_t group_m;      /* raster group height; 0 = default */
  int32_t num_ctas;     /* 0 = one per SM */
  const void* rs_mc_stage; /* GEMM+RS NVLS variant: multicast mapping of the [M][N] staging buffer, else NULL */
  uint64_t range_lo[TCL_MAX_WORLD]; /* debug build: mapped range of the memory of rank s that this plan may touch */
  uint64_t range_hi[TCL_MAX_WORLD];
  int32_t epi_silu_mul; /* plain / AG+GEMM: every 256-column tile holds 128 gate columns then the 128 up columns of the same
                           features; the epilogue writes silu(gate) * up: D is [M, N/2] (ldc is its pitch) */
  int32_t ablate;       /* experiments only: bit 0 = no reduce warps, bit 1 = no tile signals (nor reduce warps), bit 2 = AG+GEMM producer does not wait, bit 3 = one epilogue warp lags (output stays valid) */
  int32_t epi_st256;    /* the epilogue stores 32 bytes per lane (st.global.v8.b32) instead of 16; every dst_base must be
                           32-byte aligned and ldc a multiple of 16 elements; not with epi_silu_mul */
  int32_t epi_tma_store; /* the epilogue leaves through TMA (cp.async.bulk.tensor stores from the staging buffer) instead of
                            st.global; plain and AG+GEMM modes and the non-communicating GEMM+RS; not with epi_silu_mul */
  int32_t rs_signal_batch; /* GEMM+RS: finished tiles per system-scope fence of the signalling warp; 0 = default */
  int32_t ag_vec32;      /* AG+GEMM pull: gather with 32-byte loads/stores (K % 16 == 0 and 32-byte aligned buffers) */
  int32_t ag_warps;      /* AG+GEMM: gather warps per CTA that take part, 1..4; 0 = all four */
  int32_t* epoch_dev;    /* optional: two zeroed ints in device memory.  When set, the kernel takes the call number from
                            epoch_dev[0] + 1 (and advances it when the call ends) instead of the `epoch` argument of
                            tcl_gemm_plan_run, so that a captured CUDA graph can replay the launch */
} tcl_gemm_desc;

/* Layout check for bindings that restate the struct: its size, and the offset of the named field
 * (-1 for an unknown name). */
int tcl_gemm_desc_size(void);
int tcl_gemm_desc_offset(const char* field);

/* Returns NULL and fills err on invalid arguments.  A plan belongs to the device that is current when it is
 * created (tensor maps, shared-memory opt-in); create and run it with that device current. */
void* tcl_gemm_plan_create(const tcl_gemm_desc* d, char* err, int errlen);
/* Launches one call; epoch is the 1-based call number shared by all ranks.  A launch reads the plan and writes
 * nothing to it, so several host threads may launch one plan.  The fused modes, however, own flag counters and
 * staging buffers that one call uses at a time: calls of one fused plan must not overlap on the GPU (issue them
 * on one stream, or order the streams with events), and every rank must make the same sequence of calls. */
int tcl_gemm_plan_run(void* plan, int epoch, void* stream);
/* Points the plan at other A / B operands of the same shape, pitch and alignment (re-encodes the two tensor
 * maps on the host; no device work).  Takes effect for launches made after it returns; not safe while another
 * thread launches the same plan.  For TCL_MODE_AG_GEMM, A is the gathered buffer and must stay what it was. */
int tcl_gemm_plan_set_operands(void* plan, const void* A, const void* B);
void tcl_gemm_plan_destroy(void* plan);
int tcl_gemm_plan_grid(void* plan);
int tcl_gemm_smem_bytes(int cta_group);
/* Number of kernels one run launches (for launch accounting). */
int tcl_gemm_plan_launches(void* plan);

/* Schedule, exposed for host-side tests: tile t -> (m_blk, n_blk). */
void tcl_sched_tile(int m_tiles, int n_tiles, int group_m, int order, int world, int rank,
                    int rs_chunks, int t, int* m_blk, int* n_blk);

/* Device barrier over `world` ranks: every rank adds 1 to every rank's counter
 * and waits until its own reaches epoch * world.  status[0] != 0 on time-out. */
int tcl_barrier_all(int32_t* const* counters, int world, int rank, int epoch, int32_t* status,
                    uint64_t timeout_ns, void* stream);

/* The same barrier with one store per rank: a multimem.red.release on the counter's multicast address
 * adds 1 to every rank's copy inside the switch.  `mc_counter` is the multicast address of a counter in
 * a multicast-bound symmetric heap, `local_counter` this rank's own copy.  Keep one counter per barrier
 * flavour: both count epochs.  The reference has no multicast path. */
int tcl_barrier_all_mc(int32_t* mc_counter, const int32_t* local_counter, int world, int rank, int epoch,
                       int32_t* status, uint64_t timeout_ns, void* stream);

/* All-to-all store: slice p of src goes to slot `rank` of dst[p] (every peer written at once; the own slice
 * is skipped).  dst[] holds `world` device addresses, one per rank's buffer of world * slice_bytes. */
int tcl_p2p_scatter(void* const* dst, const void* src, size_t slice_bytes, int world, int rank, int blocks, void* stream);

/* Flag ping-pong between two ranks, one launch on each: mode 0 st.release.sys, 1 red.release.sys.add,
 * 2 multimem.red.release.add (remote_flag is then the multicast address; every copy counts both sides'
 * signals).  `base` = value of the flags at the start.  The initiator writes the mean round trip in ns.
 * The reference's ping-pong is tests/sync_cost.cu:82 (st.release only). */
int tcl_signal_pingpong(const int32_t* local_flag, int32_t* remote_flag, int mode, int initiator, int base, int rounds,
                        float* ns_per_rtt, int32_t* status, uint64_t timeout_ns, void* stream);

/* out[r, c] = silu(gu[r, c]) * gu[r, ffn + c]; gu is [rows, 2*ffn] bf16. */
int tcl_silu_mul(const void* gate_up, void* out, int64_t rows, int64_t ffn, void* stream);

/* N(mean, std) bf16 fill, counter-based (same seed+offset => same values). */
int tcl_fill_normal_bf16(void* dst, int64_t n, uint64_t seed, float mean, float std, void* stream);

/* max over i of |got - ref| / (|ref| + 1) with ref fp32; result[0] gets the
 * maximum.  `scratch` holds 1024 floats. */
int tcl_max_rel_err(const void* got_bf16, const float* ref, int64_t n, float* scratch,
                    float* result, void* stream);

/* tcgen05 descriptor encoders (host-callable, for layout tests). */
uint64_t tcl_make_smem_desc_k_sw128(uint32_t smem_addr);
uint64_t tcl_advance_desc_k(uint64_t desc, uint32_t bytes);
uint32_t tcl_make_idesc_bf16_f32(uint32_t m, uint32_t n);

const char* tcl_status_string(int code);
/* 1 if the library was built with TCL_DEBUG_BOUNDS (address checks on every possibly-remote access). */
int tcl_debug_bounds_enabled(void);

#ifdef __cplusplus
}
#endif
