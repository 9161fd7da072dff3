// Symmetric-memory arenas on the CUDA virtual-memory API, with an NVLink multicast mapping.
//
// An arena is physical memory created with cuMemCreate and exported as a POSIX file descriptor; the
// descriptors travel between the rank processes over a Unix-domain socket (SCM_RIGHTS, done by the
// Python side) and every rank maps every arena into its own address space.  When the devices
// support NVLink multicast, rank 0 also creates a multicast object, every rank adds its device and
// binds its arena to it, and the object is mapped as one more address range: a `multimem.ld_reduce`
// on that range returns the sum over all ranks' arenas, formed inside NVSwitch, and a `multimem.st`
// writes all of them at once.  This is the transport the tensor-parallel kernels in comm.cu use in
// place of the reference's `mx.distributed` ring / jaccl backends
// (src/exo/worker/engines/mlx/utils_mlx.py:104-143).
//
// The driver entry points are looked up at run time (cudaGetDriverEntryPoint), so the library loads
// on a machine without a driver.  Everything here is host code; nothing waits on the device.
#include <cuda.h>
#include <unistd.h>

#include <cstdint>
#include <cstring>
#include <mutex>
#include <vector>

#include "common.cuh"

namespace {

template <typename F>
F entry(const char* name) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
    return nullptr;
  return reinterpret_cast<F>(p);
}

#define DRV(name) static auto fn_##name = entry<decltype(&name)>(#name)

struct Mapping {          // one address range of this process backed by a VMM handle
  CUdeviceptr va = 0;
  size_t bytes = 0;
  CUmemGenericAllocationHandle handle = 0;
  bool multicast = false;
  bool bound = false;     // own arena bound to the multicast object
  bool owns_handle = true;
};
std::vector<Mapping> g_maps;
std::mutex g_mu;

int current_device() {
  int d = -1;
  cudaGetDevice(&d);
  return d;
}

CUmemAllocationProp arena_prop(int dev) {
  CUmemAllocationProp p;
  memset(&p, 0, sizeof(p));
  p.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  p.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  p.location.id = dev;
  p.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return p;
}

// Reserve an address range, map `h` there and give the current device read/write access.
CUdeviceptr map_handle(CUmemGenericAllocationHandle h, size_t bytes, size_t align) {
  DRV(cuMemAddressReserve);
  DRV(cuMemMap);
  DRV(cuMemSetAccess);
  DRV(cuMemAddressFree);
  if (!fn_cuMemAddressReserve || !fn_cuMemMap || !fn_cuMemSetAccess) return 0;
  CUdeviceptr va = 0;
  if (fn_cuMemAddressReserve(&va, bytes, align, 0, 0) != CUDA_SUCCESS) return 0;
  if (fn_cuMemMap(va, bytes, 0, h, 0) != CUDA_SUCCESS) {
    fn_cuMemAddressFree(va, bytes);
    return 0;
  }
  CUmemAccessDesc acc;
  memset(&acc, 0, sizeof(acc));
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = current_device();
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  if (fn_cuMemSetAccess(va, bytes, &acc, 1) != CUDA_SUCCESS) {
    DRV(cuMemUnmap);
    if (fn_cuMemUnmap) fn_cuMemUnmap(va, bytes);
    fn_cuMemAddressFree(va, bytes);
    return 0;
  }
  return va;
}

}  // namespace

// 1 when the current device can export VMM allocations as file descriptors; 2 when it also supports
// NVLink multicast objects; 0 otherwise (the CUDA-IPC arena is then the transport).
EXO_API int exo_vmm_supported() {
  DRV(cuDeviceGet);
  DRV(cuDeviceGetAttribute);
  DRV(cuMemCreate);
  if (!fn_cuDeviceGet || !fn_cuDeviceGetAttribute || !fn_cuMemCreate) return 0;
  cudaFree(0);   // make sure the primary context exists
  CUdevice d;
  if (fn_cuDeviceGet(&d, current_device()) != CUDA_SUCCESS) return 0;
  int fd_ok = 0, vmm = 0, mc = 0;
  fn_cuDeviceGetAttribute(&vmm, CU_DEVICE_ATTRIBUTE_VIRTUAL_MEMORY_MANAGEMENT_SUPPORTED, d);
  fn_cuDeviceGetAttribute(&fd_ok, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR_SUPPORTED, d);
  fn_cuDeviceGetAttribute(&mc, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, d);
  if (!vmm || !fd_ok) return 0;
  return mc ? 2 : 1;
}

// Size granule for arenas of `n_devices` ranks: the larger of the allocation granularity and (when
// multicast is available) the multicast granularity.  Arena sizes must be multiples of it.
EXO_API size_t exo_vmm_granularity(int n_devices, int with_multicast) {
  DRV(cuMemGetAllocationGranularity);
  DRV(cuMulticastGetGranularity);
  if (!fn_cuMemGetAllocationGranularity) return 0;
  CUmemAllocationProp p = arena_prop(current_device());
  size_t g = 0;
  if (fn_cuMemGetAllocationGranularity(&g, &p, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) != CUDA_SUCCESS) return 0;
  if (with_multicast && fn_cuMulticastGetGranularity) {
    CUmulticastObjectProp mp;
    memset(&mp, 0, sizeof(mp));
    mp.numDevices = n_devices;
    mp.size = g;
    mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    size_t mg = 0;
    if (fn_cuMulticastGetGranularity(&mg, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS && mg > g) g = mg;
  }
  return g;
}

// Allocates and maps this rank's arena (zero-filled).  Returns its address and, in *fd_out, a file
// descriptor to send to the peers (the caller closes it after sending).
EXO_API void* exo_vmm_alloc(size_t bytes, int* fd_out) {
  DRV(cuMemCreate);
  DRV(cuMemExportToShareableHandle);
  DRV(cuMemRelease);
  if (!fn_cuMemCreate || !fn_cuMemExportToShareableHandle || !fn_cuMemRelease) return nullptr;
  const int dev = current_device();
  CUmemAllocationProp p = arena_prop(dev);
  CUmemGenericAllocationHandle h;
  if (fn_cuMemCreate(&h, bytes, &p, 0) != CUDA_SUCCESS) return nullptr;
  int fd = -1;
  if (fn_cuMemExportToShareableHandle(&fd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0) != CUDA_SUCCESS) {
    fn_cuMemRelease(h);
    return nullptr;
  }
  CUdeviceptr va = map_handle(h, bytes, 2u << 20);
  if (!va) {
    close(fd);
    fn_cuMemRelease(h);
    return nullptr;
  }
  cudaMemset(reinterpret_cast<void*>(va), 0, bytes);
  cudaDeviceSynchronize();
  std::lock_guard<std::mutex> lk(g_mu);
  g_maps.push_back(Mapping{va, bytes, h, false, false, true});
  *fd_out = fd;
  return reinterpret_cast<void*>(va);
}

// Maps a peer's arena from the descriptor it sent.  The descriptor stays the caller's to close.
EXO_API void* exo_vmm_import(int fd, size_t bytes) {
  DRV(cuMemImportFromShareableHandle);
  DRV(cuMemRelease);
  if (!fn_cuMemImportFromShareableHandle || !fn_cuMemRelease) return nullptr;
  CUmemGenericAllocationHandle h;
  if (fn_cuMemImportFromShareableHandle(&h, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)),
                                        CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR) != CUDA_SUCCESS)
    return nullptr;
  CUdeviceptr va = map_handle(h, bytes, 2u << 20);
  if (!va) {
    fn_cuMemRelease(h);
    return nullptr;
  }
  std::lock_guard<std::mutex> lk(g_mu);
  g_maps.push_back(Mapping{va, bytes, h, false, false, true});
  return reinterpret_cast<void*>(va);
}

// Rank 0: creates the multicast object for `n_devices` arenas of `bytes` each; *fd_out goes to the peers.
// Returns an opaque handle (0 on failure).
EXO_API unsigned long long exo_mc_create(size_t bytes, int n_devices, int* fd_out) {
  DRV(cuMulticastCreate);
  DRV(cuMemExportToShareableHandle);
  DRV(cuMemRelease);
  if (!fn_cuMulticastCreate || !fn_cuMemExportToShareableHandle) return 0;
  CUmulticastObjectProp mp;
  memset(&mp, 0, sizeof(mp));
  mp.numDevices = n_devices;
  mp.size = bytes;
  mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  CUmemGenericAllocationHandle mc;
  if (fn_cuMulticastCreate(&mc, &mp) != CUDA_SUCCESS) return 0;
  int fd = -1;
  if (fn_cuMemExportToShareableHandle(&fd, mc, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0) != CUDA_SUCCESS) {
    if (fn_cuMemRelease) fn_cuMemRelease(mc);
    return 0;
  }
  *fd_out = fd;
  return (unsigned long long)mc;
}

// Other ranks: opens the multicast object from rank 0's descriptor.
EXO_API unsigned long long exo_mc_import(int fd) {
  DRV(cuMemImportFromShareableHandle);
  if (!fn_cuMemImportFromShareableHandle) return 0;
  CUmemGenericAllocationHandle mc;
  if (fn_cuMemImportFromShareableHandle(&mc, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)),
                                        CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR) != CUDA_SUCCESS)
    return 0;
  return (unsigned long long)mc;
}

// Every rank: adds its device to the object.  All ranks must have done this before any of them binds.
EXO_API int exo_mc_add_device(unsigned long long mc) {
  DRV(cuMulticastAddDevice);
  DRV(cuDeviceGet);
  if (!fn_cuMulticastAddDevice || !fn_cuDeviceGet) return -1;
  CUdevice d;
  if (fn_cuDeviceGet(&d, current_device()) != CUDA_SUCCESS) return -1;
  return (int)fn_cuMulticastAddDevice((CUmemGenericAllocationHandle)mc, d);
}

// Every rank: binds its own arena (the address exo_vmm_alloc returned) to the object and maps the object.
// Returns the multicast address of the arena (nullptr on failure).
EXO_API void* exo_mc_bind_and_map(unsigned long long mc, void* arena, size_t bytes) {
  DRV(cuMulticastBindMem);
  if (!fn_cuMulticastBindMem) return nullptr;
  CUmemGenericAllocationHandle mem = 0;
  {
    std::lock_guard<std::mutex> lk(g_mu);
    for (auto& m : g_maps)
      if (m.va == reinterpret_cast<CUdeviceptr>(arena)) mem = m.handle;
  }
  if (!mem) return nullptr;
  if (fn_cuMulticastBindMem((CUmemGenericAllocationHandle)mc, 0, mem, 0, bytes, 0) != CUDA_SUCCESS) return nullptr;
  CUdeviceptr va = map_handle((CUmemGenericAllocationHandle)mc, bytes, 2u << 20);
  std::lock_guard<std::mutex> lk(g_mu);
  if (!va) {
    DRV(cuMulticastUnbind);
    DRV(cuDeviceGet);
    CUdevice d;
    if (fn_cuMulticastUnbind && fn_cuDeviceGet && fn_cuDeviceGet(&d, current_device()) == CUDA_SUCCESS)
      fn_cuMulticastUnbind((CUmemGenericAllocationHandle)mc, d, 0, bytes);
    return nullptr;
  }
  g_maps.push_back(Mapping{va, bytes, (CUmemGenericAllocationHandle)mc, true, true, true});
  return reinterpret_cast<void*>(va);
}

// Unmaps one range obtained from the calls above (a multicast range is unbound first) and releases its
// handle.  The caller has synchronised the device and agreed with its peers that no kernel uses the range.
EXO_API int exo_vmm_unmap(void* p) {
  DRV(cuMemUnmap);
  DRV(cuMemAddressFree);
  DRV(cuMemRelease);
  DRV(cuMulticastUnbind);
  DRV(cuDeviceGet);
  if (!fn_cuMemUnmap || !fn_cuMemAddressFree || !fn_cuMemRelease) return -1;
  Mapping m;
  {
    std::lock_guard<std::mutex> lk(g_mu);
    size_t i = 0;
    for (; i < g_maps.size(); i++)
      if (g_maps[i].va == reinterpret_cast<CUdeviceptr>(p)) break;
    if (i == g_maps.size()) return -2;
    m = g_maps[i];
    g_maps.erase(g_maps.begin() + (long)i);
  }
  int rc = 0;
  rc |= (int)fn_cuMemUnmap(m.va, m.bytes);
  rc |= (int)fn_cuMemAddressFree(m.va, m.bytes);
  if (m.multicast && m.bound && fn_cuMulticastUnbind && fn_cuDeviceGet) {      // after the range is gone, before the handle
    CUdevice d;
    if (fn_cuDeviceGet(&d, current_device()) == CUDA_SUCCESS) rc |= (int)fn_cuMulticastUnbind(m.handle, d, 0, m.bytes);
  }
  rc |= (int)fn_cuMemRelease(m.handle);
  return rc;
}
