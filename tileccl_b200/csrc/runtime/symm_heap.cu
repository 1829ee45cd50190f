// Symmetric-heap primitives of libtileccl.so.
//
// Two back ends behind one C interface:
//   * IPC:  cudaMalloc + cudaIpcGetMemHandle / cudaIpcOpenMemHandle.  Works
//           everywhere peer access works; no multicast.
//   * VMM:  cuMemCreate with a POSIX file-descriptor handle, mapped by every
//           rank, optionally bound to an NVLS multicast object so that
//           multimem.* instructions reach all GPUs through the NVSwitch.
// The rendezvous (who sends which handle to whom) is the caller's job: the
// Python layer uses the torch.distributed store for IPC handles and a Unix
// socket (SCM_RIGHTS) for file descriptors.
//
// Reference parity: comm_comp/ipc_multiproc.cuh:159-171 (exchange(): get handle,
// barrier, open peers) and comm_comp/common.cuh:154-173 (all-pairs peer
// enable).  The reference has no VMM heap and no multicast.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <cstring>

namespace {

template <typename Fn>
Fn drv(const char* name) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess ||
      q != cudaDriverEntryPointSuccess)
    return nullptr;
  return reinterpret_cast<Fn>(p);
}

#define DRV(name) static auto fn_##name = drv<decltype(&name)>(#name); if (!fn_##name) return -1

CUmemAllocationProp alloc_prop(int dev) {
  CUmemAllocationProp prop;
  std::memset(&prop, 0, sizeof(prop));
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = dev;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return prop;
}

int map_handle(CUmemGenericAllocationHandle h, size_t bytes, size_t gran, int dev, void** out) {
  DRV(cuMemAddressReserve);
  DRV(cuMemMap);
  DRV(cuMemSetAccess);
  DRV(cuMemAddressFree);
  CUdeviceptr va = 0;
  CUresult r = fn_cuMemAddressReserve(&va, bytes, gran, 0, 0);
  if (r != CUDA_SUCCESS) return static_cast<int>(r);
  r = fn_cuMemMap(va, bytes, 0, h, 0);
  if (r != CUDA_SUCCESS) { fn_cuMemAddressFree(va, bytes); return static_cast<int>(r); }
  CUmemAccessDesc acc;
  std::memset(&acc, 0, sizeof(acc));
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = dev;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  r = fn_cuMemSetAccess(va, bytes, &acc, 1);
  if (r != CUDA_SUCCESS) return static_cast<int>(r);
  *out = reinterpret_cast<void*>(va);
  return 0;
}

}  // namespace

extern "C" {

// ---- IPC back end -----------------------------------------------------------
int tcl_heap_alloc(size_t bytes, void** ptr) {
  cudaError_t e = cudaMalloc(ptr, bytes);
  if (e != cudaSuccess) return static_cast<int>(e);
  return static_cast<int>(cudaMemset(*ptr, 0, bytes));
}
int tcl_heap_free(void* ptr) { return static_cast<int>(cudaFree(ptr)); }
int tcl_ipc_handle_size() { return static_cast<int>(sizeof(cudaIpcMemHandle_t)); }
int tcl_ipc_get_handle(void* ptr, void* handle_out) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, ptr);
  if (e != cudaSuccess) return static_cast<int>(e);
  std::memcpy(handle_out, &h, sizeof(h));
  return 0;
}
int tcl_ipc_open(const void* handle, void** ptr) {
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle, sizeof(h));
  return static_cast<int>(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
}
int tcl_ipc_close(void* ptr) { return static_cast<int>(cudaIpcCloseMemHandle(ptr)); }

// Single-process multi-GPU helper: enable peer access from the current device
// to `peer` (already-enabled is not an error).
int tcl_enable_peer(int peer) {
  cudaError_t e = cudaDeviceEnablePeerAccess(peer, 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) { cudaGetLastError(); return 0; }
  return static_cast<int>(e);
}
int tcl_can_access_peer(int dev, int peer) {
  int ok = 0;
  if (cudaDeviceCanAccessPeer(&ok, dev, peer) != cudaSuccess) return 0;
  return ok;
}

// Copy-engine transport (the measured alternative to in-kernel ld/st): one
// asynchronous peer copy.  src/dst may be IPC or VMM mappings of peer memory.
int tcl_memcpy_peer_async(void* dst, int dst_dev, const void* src, int src_dev, size_t bytes, void* stream) {
  return static_cast<int>(cudaMemcpyPeerAsync(dst, dst_dev, src, src_dev, bytes, static_cast<cudaStream_t>(stream)));
}
int tcl_memcpy_async(void* dst, const void* src, size_t bytes, void* stream) {
  return static_cast<int>(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDefault, static_cast<cudaStream_t>(stream)));
}

// ---- VMM back end -------------------------------------------------------------
// Rounds `bytes` up to the allocation granularity of device `dev`.
int tcl_vmm_granularity(int dev, size_t* gran, int multicast, int world) {
  if (!multicast) {
    DRV(cuMemGetAllocationGranularity);
    CUmemAllocationProp prop = alloc_prop(dev);
    return static_cast<int>(fn_cuMemGetAllocationGranularity(gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED));
  }
  DRV(cuMulticastGetGranularity);
  CUmulticastObjectProp mp;
  std::memset(&mp, 0, sizeof(mp));
  mp.numDevices = static_cast<unsigned>(world);
  mp.size = size_t(1) << 21;
  mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return static_cast<int>(fn_cuMulticastGetGranularity(gran, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED));
}

int tcl_multicast_supported(int dev) {
  int v = 0;
  DRV(cuDeviceGetAttribute);
  if (fn_cuDeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev) != CUDA_SUCCESS) return 0;
  return v;
}

// Creates `bytes` (a multiple of the granularity) of physical memory on `dev`,
// maps it, zero-fills it, and exports a file descriptor for the peers.
int tcl_vmm_create(int dev, size_t bytes, size_t gran, uint64_t* handle_out, int* fd_out, void** ptr) {
  DRV(cuMemCreate);
  DRV(cuMemExportToShareableHandle);
  CUmemAllocationProp prop = alloc_prop(dev);
  CUmemGenericAllocationHandle h;
  CUresult r = fn_cuMemCreate(&h, bytes, &prop, 0);
  if (r != CUDA_SUCCESS) return static_cast<int>(r);
  int fd = -1;
  r = fn_cuMemExportToShareableHandle(&fd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
  if (r != CUDA_SUCCESS) return static_cast<int>(r);
  int rc = map_handle(h, bytes, gran, dev, ptr);
  if (rc != 0) return rc;
  *handle_out = static_cast<uint64_t>(h);
  *fd_out = fd;
  return static_cast<int>(cudaMemset(*ptr, 0, bytes));
}

// Imports a peer's allocation from a received file descriptor and maps it for `dev`.
int tcl_vmm_import(int dev, int fd, size_t bytes, size_t gran, uint64_t* handle_out, void** ptr) {
  DRV(cuMemImportFromShareableHandle);
  CUmemGenericAllocationHandle h;
  CUresult r = fn_cuMemImportFromShareableHandle(&h, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)),
                                                 CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
  if (r != CUDA_SUCCESS) return static_cast<int>(r);
  *handle_out = static_cast<uint64_t>(h);
  return map_handle(h, bytes, gran, dev, ptr);
}

int tcl_vmm_unmap(void* ptr, size_t bytes, uint64_t handle) {
  DRV(cuMemUnmap);
  DRV(cuMemAddressFree);
  DRV(cuMemRelease);
  CUdeviceptr va = reinterpret_cast<CUdeviceptr>(ptr);
  fn_cuMemUnmap(va, bytes);
  fn_cuMemAddressFree(va, bytes);
  return static_cast<int>(fn_cuMemRelease(static_cast<CUmemGenericAllocationHandle>(handle)));
}

// ---- NVLS multicast ----------------------------------------------------------
// Rank 0 creates the object and exports a descriptor; the others import it.
int tcl_mc_create(int world, size_t bytes, uint64_t* mc_out, int* fd_out) {
  DRV(cuMulticastCreate);
  DRV(cuMemExportToShareableHandle);
  CUmulticastObjectProp mp;
  std::memset(&mp, 0, sizeof(mp));
  mp.numDevices = static_cast<unsigned>(world);
  mp.size = bytes;
  mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  CUmemGenericAllocationHandle mc;
  CUresult r = fn_cuMulticastCreate(&mc, &mp);
  if (r != CUDA_SUCCESS) return static_cast<int>(r);
  int fd = -1;
  r = fn_cuMemExportToShareableHandle(&fd, mc, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
  if (r != CUDA_SUCCESS) return static_cast<int>(r);
  *mc_out = static_cast<uint64_t>(mc);
  *fd_out = fd;
  return 0;
}
int tcl_mc_import(int fd, uint64_t* mc_out) {
  DRV(cuMemImportFromShareableHandle);
  CUmemGenericAllocationHandle mc;
  CUresult r = fn_cuMemImportFromShareableHandle(&mc, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)),
                                                 CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
  if (r != CUDA_SUCCESS) return static_cast<int>(r);
  *mc_out = static_cast<uint64_t>(mc);
  return 0;
}
// Every rank, before anyone binds.
int tcl_mc_add_device(uint64_t mc, int dev) {
  DRV(cuMulticastAddDevice);
  return static_cast<int>(fn_cuMulticastAddDevice(static_cast<CUmemGenericAllocationHandle>(mc), dev));
}
// After every rank has added its device: bind this rank's physical memory and
// map the multicast object into this rank's address space.
int tcl_mc_bind_and_map(uint64_t mc, uint64_t mem_handle, size_t bytes, size_t gran, int dev, void** mc_ptr) {
  DRV(cuMulticastBindMem);
  CUresult r = fn_cuMulticastBindMem(static_cast<CUmemGenericAllocationHandle>(mc), 0,
                                     static_cast<CUmemGenericAllocationHandle>(mem_handle), 0, bytes, 0);
  if (r != CUDA_SUCCESS) return static_cast<int>(r);
  return map_handle(static_cast<CUmemGenericAllocationHandle>(mc), bytes, gran, dev, mc_ptr);
}

// Before the physical memory is released: detach this device's memory from the multicast object.
int tcl_mc_unbind(uint64_t mc, int dev, size_t bytes) {
  DRV(cuMulticastUnbind);
  return static_cast<int>(fn_cuMulticastUnbind(static_cast<CUmemGenericAllocationHandle>(mc), dev, 0, bytes));
}

}  // extern "C"
