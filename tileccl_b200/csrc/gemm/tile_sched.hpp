// Static persistent tile schedule shared by every warp role of the GEMM
// kernels, by the host planners and (through a C wrapper) by the CPU tests.
//
// A schedule maps a linear work index t in [0, m_tiles*n_tiles) to a tile
// (m_blk, n_blk).  Two things are layered:
//   1. an M permutation that depends on the fused collective, so that what a
//      rank computes first is what the collective needs first;
//   2. a grouped raster (groups of `group_m` schedule rows, M fastest inside a
//      group) so that the tiles that run at the same time share operand
//      panels in L2.
//
// Reference parity: the reference pins CUTLASS's static persistent scheduler
// and XOR-swizzles the M segment so that ranks do not all pull from the same
// peer (comm_comp/rs_gemm_kernel_sm90.cuh:130,321-330).  The XOR form needs a
// power-of-two world; the rotation used here works for any world size.
#pragma once
#include <cstdint>

#if defined(__CUDACC__)
#define TCL_HD __host__ __device__ __forceinline__
#else
#define TCL_HD inline
#endif

namespace tcl {

enum MOrder : int {
  kOrderPlain = 0,   // schedule row p is tile row p
  kOrderRsPush = 1,  // reduce-scatter: rounds of chunks, peers rotated, own segment last
  kOrderAgPull = 2,  // all-gather by pull: own segment first, then peers in rotation, one after the other
  kOrderAgPush = 3   // all-gather by push: own segment first, then tile row i of every peer before row i+1
                     // (all shards arrive at the same rate, so rows are consumed in arrival order)
};

struct TileSched {
  int m_tiles;    // tile rows in the whole problem
  int n_tiles;    // tile columns
  int group_m;    // raster group height in schedule rows
  int order;      // MOrder
  int world;      // ranks (segments along M)
  int rank;       // this rank
  int rs_chunks;  // kOrderRsPush: chunks per segment (G); segment tile rows % G == 0

  TCL_HD int num_tiles() const { return m_tiles * n_tiles; }
  TCL_HD int seg_tiles() const { return m_tiles / world; }

  // Schedule row p -> tile row.
  TCL_HD int m_of_row(int p) const {
    if (order == kOrderRsPush) {
      const int st = seg_tiles();
      const int cpr = st / rs_chunks;           // tile rows per chunk
      const int per_round = world * cpr;        // schedule rows per round
      const int g = p / per_round;              // round = chunk index
      const int q = p - g * per_round;
      const int step = q / cpr;                 // 0 .. world-1
      const int i = q - step * cpr;
      const int seg = (rank + 1 + step) % world;  // own segment at the last step
      return seg * st + g * cpr + i;
    }
    if (order == kOrderAgPush) {
      const int st = seg_tiles();
      if (p < st) return rank * st + p;             // own segment
      const int q = p - st;
      const int i = q / (world - 1);                // tile row inside the segments
      const int step = q - i * (world - 1) + 1;     // 1 .. world-1
      return ((rank + step) % world) * st + i;
    }
    if (order == kOrderAgPull) {
      const int st = seg_tiles();
      const int step = p / st;
      const int i = p - step * st;
      const int seg = (rank + step) % world;  // own segment first
      return seg * st + i;
    }
    return p;
  }

  // Linear work index -> (schedule row, tile column).
  TCL_HD void row_col(int t, int* p, int* n) const {
    const int per_group = group_m * n_tiles;
    const int grp = t / per_group;
    const int first = grp * group_m;
    const int rem = t - grp * per_group;
    int gm = m_tiles - first;
    if (gm > group_m) gm = group_m;
    *n = rem / gm;
    *p = first + (rem - (*n) * gm);
  }

  TCL_HD void tile(int t, int* m_blk, int* n_blk) const {
    int p;
    row_col(t, &p, n_blk);
    *m_blk = m_of_row(p);
  }
};

// Reduce-scatter reduce work list of one rank: item j -> tile of the rank's own
// segment, in the order in which the schedule above completes them on every
// producer (round by round).  seg-local tile row and tile column.
TCL_HD void rs_reduce_item(const TileSched& s, int j, int* seg_row, int* n_blk) {
  // Rounds are contiguous in j: each round holds cpr * n_tiles tiles.
  *seg_row = j / s.n_tiles;
  *n_blk = j - (*seg_row) * s.n_tiles;
}

}  // namespace tcl
