// Team arenas as virtual-memory-management allocations shared through POSIX file descriptors.
//
// An arena made with cuMemCreate is a reference-counted physical allocation.  A peer that
// imports the exported file descriptor (cuMemImportFromShareableHandle) holds a reference of its
// own, so the memory it has mapped stays valid until that peer unmaps it and releases its
// handle: by the documented semantics of these calls a rank that has left the job cannot pull
// memory out from under the kernels of the ranks that stay.  (With the legacy cudaIpc handles the
// lifetime of an importer's mapping after the exporter's exit is not specified.)  The file
// descriptor itself travels between the processes over a Unix-domain socket (SCM_RIGHTS); that
// part is done by the Python side.
//
// Host-only code: the driver entry points are looked up at run time, so the library links
// against the runtime only.
#include <cuda.h>
#include <cuda_runtime.h>
#include <unistd.h>

#include <cstdint>
#include <mutex>
#include <unordered_map>

#include "ftb200_common.cuh"

namespace {

struct Api {
  CUresult (*getGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags) = nullptr;
  CUresult (*create)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long) = nullptr;
  CUresult (*release)(CUmemGenericAllocationHandle) = nullptr;
  CUresult (*reserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
  CUresult (*addressFree)(CUdeviceptr, size_t) = nullptr;
  CUresult (*map)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
  CUresult (*unmap)(CUdeviceptr, size_t) = nullptr;
  CUresult (*setAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) = nullptr;
  CUresult (*exportHandle)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long) = nullptr;
  CUresult (*importHandle)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType) = nullptr;
  bool ok = false;
};

template <typename F>
bool lookup(const char* name, F& fn) {
  void* sym = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &sym, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess ||
      sym == nullptr)
    return false;
  fn = reinterpret_cast<F>(sym);
  return true;
}

const Api& api() {
  static Api a;
  static std::once_flag once;
  std::call_once(once, [] {
    a.ok = lookup("cuMemGetAllocationGranularity", a.getGranularity) && lookup("cuMemCreate", a.create) &&
           lookup("cuMemRelease", a.release) && lookup("cuMemAddressReserve", a.reserve) &&
           lookup("cuMemAddressFree", a.addressFree) && lookup("cuMemMap", a.map) && lookup("cuMemUnmap", a.unmap) &&
           lookup("cuMemSetAccess", a.setAccess) && lookup("cuMemExportToShareableHandle", a.exportHandle) &&
           lookup("cuMemImportFromShareableHandle", a.importHandle);
  });
  return a;
}

struct Mapping {
  CUmemGenericAllocationHandle handle;
  size_t bytes;
};
std::mutex g_mu;
std::unordered_map<uintptr_t, Mapping> g_maps;  // mapped base address -> what to undo

CUmemAllocationProp props_for(int dev) {
  CUmemAllocationProp p = {};
  p.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  p.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  p.location.id = dev;
  p.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return p;
}

// reserve a range, map `handle` there and give the current device read/write access
int map_here(const Api& a, CUmemGenericAllocationHandle handle, size_t bytes, size_t gran, int dev, void** ptr) {
  CUdeviceptr va = 0;
  if (a.reserve(&va, bytes, gran, 0, 0) != CUDA_SUCCESS) return FTB200_E_DRIVER;
  if (a.map(va, bytes, 0, handle, 0) != CUDA_SUCCESS) {
    a.addressFree(va, bytes);
    return FTB200_E_DRIVER;
  }
  CUmemAccessDesc acc = {};
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = dev;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  if (a.setAccess(va, bytes, &acc, 1) != CUDA_SUCCESS) {
    a.unmap(va, bytes);
    a.addressFree(va, bytes);
    return FTB200_E_DRIVER;
  }
  {
    std::lock_guard<std::mutex> lk(g_mu);
    g_maps[static_cast<uintptr_t>(va)] = Mapping{handle, bytes};
  }
  *ptr = reinterpret_cast<void*>(va);
  return 0;
}

}  // namespace

// Allocates `bytes` (rounded up to the allocation granularity, reported in *padded) on the current device,
// maps it, and exports it as a file descriptor that the caller owns (close it when every peer has it).
FTB200_API int ftb200_vmm_alloc(void** ptr, unsigned long long bytes, int* fd_out, unsigned long long* padded) {
  const Api& a = api();
  if (!a.ok) return FTB200_E_DRIVER;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return FTB200_E_CUDA;
  cudaFree(nullptr);  // make sure the primary context exists
  const CUmemAllocationProp prop = props_for(dev);
  size_t gran = 0;
  if (a.getGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) != CUDA_SUCCESS || gran == 0)
    return FTB200_E_DRIVER;
  const size_t size = (static_cast<size_t>(bytes) + gran - 1) / gran * gran;
  CUmemGenericAllocationHandle handle;
  if (a.create(&handle, size, &prop, 0) != CUDA_SUCCESS) return FTB200_E_DRIVER;
  int fd = -1;
  if (a.exportHandle(&fd, handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0) != CUDA_SUCCESS) {
    a.release(handle);
    return FTB200_E_DRIVER;
  }
  const int rc = map_here(a, handle, size, gran, dev, ptr);
  if (rc != 0) {
    close(fd);
    a.release(handle);
    return rc;
  }
  *fd_out = fd;
  *padded = size;
  return 0;
}

// Maps a peer's arena, received as file descriptor `fd` (not closed here), of `bytes` (the exporter's padded
// size) into this process for the current device.
FTB200_API int ftb200_vmm_import(int fd, unsigned long long bytes, void** ptr) {
  const Api& a = api();
  if (!a.ok) return FTB200_E_DRIVER;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return FTB200_E_CUDA;
  cudaFree(nullptr);
  CUmemGenericAllocationHandle handle;
  if (a.importHandle(&handle, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)),
                     CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR) != CUDA_SUCCESS)
    return FTB200_E_DRIVER;
  const CUmemAllocationProp prop = props_for(dev);
  size_t gran = 0;
  if (a.getGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) != CUDA_SUCCESS || gran == 0) {
    a.release(handle);
    return FTB200_E_DRIVER;
  }
  const int rc = map_here(a, handle, static_cast<size_t>(bytes), gran, dev, ptr);
  if (rc != 0) a.release(handle);
  return rc;
}

// Unmaps an arena or a peer's arena mapped by the two calls above and drops this process's reference.
FTB200_API int ftb200_vmm_free(void* ptr) {
  const Api& a = api();
  if (!a.ok) return FTB200_E_DRIVER;
  Mapping m;
  {
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = g_maps.find(reinterpret_cast<uintptr_t>(ptr));
    if (it == g_maps.end()) return FTB200_E_BADARG;
    m = it->second;
    g_maps.erase(it);
  }
  const CUdeviceptr va = reinterpret_cast<CUdeviceptr>(ptr);
  int rc = 0;
  if (a.unmap(va, m.bytes) != CUDA_SUCCESS) rc = FTB200_E_DRIVER;
  if (a.addressFree(va, m.bytes) != CUDA_SUCCESS) rc = FTB200_E_DRIVER;
  if (a.release(m.handle) != CUDA_SUCCESS) rc = FTB200_E_DRIVER;
  return rc;
}
