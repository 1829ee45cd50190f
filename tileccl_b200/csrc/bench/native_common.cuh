// Pieces shared by the native (fork-launcher) drivers of the fused experiments: cudaIpc buffer
// sharing through the launcher's exchange table, device barrier bookkeeping, timing of one plan.
#pragma once
#include <unistd.h>

#include <vector>

#include "../common/host_common.hpp"
#include "../ops/tileccl_ops.h"
#include "../runtime/launcher.hpp"

namespace tcl {
namespace native {

struct Buf {
  void* local = nullptr;
  void* peer[TCL_MAX_WORLD] = {};
};

// Every rank publishes the cudaIpc handle of b.local in `slot` and opens the others.
inline bool share(rt::Launcher& L, int slot, Buf& b) {
  if (L.world() == 1) { b.peer[0] = b.local; return true; }
  cudaIpcMemHandle_t mine, all[TCL_MAX_WORLD];
  if (cudaIpcGetMemHandle(&mine, b.local) != cudaSuccess) { L.fail("cudaIpcGetMemHandle"); return false; }
  if (!L.exchange(slot, &mine, sizeof(mine), all)) return false;
  for (int r = 0; r < L.world(); ++r) {
    if (r == L.rank()) { b.peer[r] = b.local; continue; }
    if (cudaIpcOpenMemHandle(&b.peer[r], all[r], cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) { L.fail("cudaIpcOpenMemHandle"); return false; }
  }
  return L.barrier();
}

inline void unshare(rt::Launcher& L, Buf& b) {
  for (int r = 0; r < L.world(); ++r)
    if (r != L.rank() && b.peer[r]) cudaIpcCloseMemHandle(b.peer[r]);
}

// Leaves the process the way a rank must: children _exit, rank 0 reaps them.
[[noreturn]] inline void die(rt::Launcher& L, const char* why, int code = 3) {
  L.fail(why);
  std::fprintf(stderr, "rank %d: %s\n", L.rank(), why);
  if (L.rank() != 0) _exit(code);
  L.wait_children(10.0);
  std::exit(code);
}

struct DeviceBarrier {
  int32_t* ptrs[TCL_MAX_WORLD] = {};
  int epoch = 0, world = 1, rank = 0;
  int32_t* status = nullptr;
  void run(cudaStream_t st) { tcl_barrier_all(ptrs, world, rank, ++epoch, status, 0, st); }
};

// One timed launch of a plan behind a device barrier; returns microseconds.
inline double timed_run(void* plan, int* epoch, DeviceBarrier& bar, cudaStream_t st, cudaEvent_t e0, cudaEvent_t e1) {
  bar.run(st);
  TCL_CUDA_CHECK(cudaEventRecord(e0, st));
  if (tcl_gemm_plan_run(plan, ++*epoch, st) != 0) return -1;
  TCL_CUDA_CHECK(cudaEventRecord(e1, st));
  TCL_CUDA_CHECK(cudaEventSynchronize(e1));
  return host::elapsed_us(e0, e1);
}

}  // namespace native
}  // namespace tcl
