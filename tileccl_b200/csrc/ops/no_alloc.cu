// Allocation-free variant of the verify kernel pair: see no_alloc.h for who needs it and for the
// rules.  The scratch is a file-scope __device__ array; in host code that name is only a stand-in
// for the symbol, so the host asks the runtime for the array's device address once per device and
// hands that pointer to the kernels.
#include "no_alloc.h"

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <mutex>

namespace {

// One partial maximum per block; every GPU that loads this library holds these 64 KiB.
static __device__ __align__(256) float g_static_scratch[TCL_STATIC_SCRATCH_FLOATS];

constexpr int kThreads = 256;
constexpr int kMaxDevices = 64;

// Block b covers elements [b * 4096, (b + 1) * 4096) and writes scratch[b].
__global__ void static_partial_kernel(const __nv_bfloat16* __restrict__ got, const float* __restrict__ ref, long long n,
                                      float* __restrict__ scratch) {
  const long long base = static_cast<long long>(blockIdx.x) * TCL_STATIC_ELEMS_PER_BLOCK;
  float m = 0.f;
  for (int k = threadIdx.x; k < TCL_STATIC_ELEMS_PER_BLOCK; k += kThreads) {
    const long long i = base + k;
    if (i < n) {
      const float r = ref[i];
      const float g = __bfloat162float(got[i]);
      float e = fabsf(g - r) / (fabsf(r) + 1.f);
      if (!(e == e)) e = 3.4e38f;
      m = fmaxf(m, e);
    }
  }
  __shared__ float sm[kThreads];
  sm[threadIdx.x] = m;
  __syncthreads();
  for (int s = kThreads / 2; s > 0; s >>= 1) {
    if (threadIdx.x < s) sm[threadIdx.x] = fmaxf(sm[threadIdx.x], sm[threadIdx.x + s]);
    __syncthreads();
  }
  if (threadIdx.x == 0) scratch[blockIdx.x] = sm[0];
}

__global__ void static_final_kernel(const float* __restrict__ scratch, int nblocks, float* __restrict__ result) {
  __shared__ float sm[kThreads];
  float m = 0.f;
  for (int i = threadIdx.x; i < nblocks; i += kThreads) m = fmaxf(m, scratch[i]);
  sm[threadIdx.x] = m;
  __syncthreads();
  for (int s = kThreads / 2; s > 0; s >>= 1) {
    if (threadIdx.x < s) sm[threadIdx.x] = fmaxf(sm[threadIdx.x], sm[threadIdx.x + s]);
    __syncthreads();
  }
  if (threadIdx.x == 0) result[0] = sm[0];
}

std::mutex g_setup_mutex;
float* g_scratch_ptr[kMaxDevices] = {};

// Device address of the scratch array on the current device, looked up on first use.
float* scratch_for_current_device(int* rc) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) { *rc = TCL_ERR_STATIC_SETUP; return nullptr; }
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (!g_scratch_ptr[dev]) {
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_static_scratch);
    if (e != cudaSuccess || !p) { cudaGetLastError(); *rc = TCL_ERR_STATIC_SETUP; return nullptr; }
    g_scratch_ptr[dev] = p;
  }
  return g_scratch_ptr[dev];
}

}  // namespace

extern "C" {

int tcl_max_rel_err_static(const void* got_bf16, const float* ref, int64_t n, float* result, void* stream) {
  if (!got_bf16 || !ref || !result || n <= 0) return TCL_ERR_STATIC_BAD_ARG;
  if (n > TCL_STATIC_MAX_ELEMS) return TCL_ERR_STATIC_TOO_LARGE;
  int rc = 0;
  float* scratch = scratch_for_current_device(&rc);
  if (!scratch) return rc;
  const int blocks = static_cast<int>((n + TCL_STATIC_ELEMS_PER_BLOCK - 1) / TCL_STATIC_ELEMS_PER_BLOCK);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  static_partial_kernel<<<blocks, kThreads, 0, st>>>(static_cast<const __nv_bfloat16*>(got_bf16), ref, n, scratch);
  static_final_kernel<<<1, kThreads, 0, st>>>(scratch, blocks, result);
  return static_cast<int>(cudaGetLastError());
}

const char* tcl_max_rel_err_static_strerror(int code) {
  switch (code) {
    case 0: return "ok";
    case TCL_ERR_STATIC_TOO_LARGE: return "n exceeds TCL_STATIC_MAX_ELEMS (67,108,864 elements): the fixed scratch array cannot hold one partial per 4096 elements";
    case TCL_ERR_STATIC_BAD_ARG: return "null pointer or non-positive element count";
    case TCL_ERR_STATIC_SETUP: return "could not obtain the device address of the static scratch array on the current device";
    default: return code > 0 ? cudaGetErrorString(static_cast<cudaError_t>(code)) : "unknown error";
  }
}

}  // extern "C"
