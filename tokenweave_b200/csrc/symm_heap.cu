// Symmetric-memory allocator on the CUDA virtual-memory-management API: physical allocations that
// can be exported to the other ranks of the node as POSIX file descriptors, peer mappings of every
// rank's allocation, and an NVLS multicast object bound to all of them.
//
// The reference relies on PyTorch's symmetric-memory rendezvous
// (vllm/model_executor/models/llama.py:437-441); this is the package's own equivalent. The file
// descriptors travel between processes over Unix sockets in Python
// (tokenweave_b200/parallel/symm_native.py); this file holds the driver calls. Driver entry points
// are resolved at run time (cudaGetDriverEntryPoint), so the library links without libcuda.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include "tw_host.h"

namespace tw {

struct DriverApi {
  CUresult (*memGetAllocationGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags);
  CUresult (*memCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long);
  CUresult (*memRelease)(CUmemGenericAllocationHandle);
  CUresult (*memExportToShareableHandle)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType,
                                         unsigned long long);
  CUresult (*memImportFromShareableHandle)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType);
  CUresult (*memAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long);
  CUresult (*memAddressFree)(CUdeviceptr, size_t);
  CUresult (*memMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long);
  CUresult (*memUnmap)(CUdeviceptr, size_t);
  CUresult (*memSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t);
  CUresult (*multicastCreate)(CUmemGenericAllocationHandle*, const CUmulticastObjectProp*);
  CUresult (*multicastAddDevice)(CUmemGenericAllocationHandle, CUdevice);
  CUresult (*multicastBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t,
                               size_t, unsigned long long);
  CUresult (*multicastUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t);
  CUresult (*multicastGetGranularity)(size_t*, const CUmulticastObjectProp*, CUmulticastGranularity_flags);
  CUresult (*deviceGetAttribute)(int*, CUdevice_attribute, CUdevice);
  bool ok;
};

template <typename F>
static bool resolve(F& fn, const char* name) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess ||
      p == nullptr) {
    set_last_error("symm_heap: driver entry point %s is not available", name);
    return false;
  }
  fn = reinterpret_cast<F>(p);
  return true;
}

static DriverApi* api() {
  static DriverApi a;
  static bool tried = false;
  if (!tried) {
    tried = true;
    a.ok = resolve(a.memGetAllocationGranularity, "cuMemGetAllocationGranularity") &&
           resolve(a.memCreate, "cuMemCreate") && resolve(a.memRelease, "cuMemRelease") &&
           resolve(a.memExportToShareableHandle, "cuMemExportToShareableHandle") &&
           resolve(a.memImportFromShareableHandle, "cuMemImportFromShareableHandle") &&
           resolve(a.memAddressReserve, "cuMemAddressReserve") && resolve(a.memAddressFree, "cuMemAddressFree") &&
           resolve(a.memMap, "cuMemMap") && resolve(a.memUnmap, "cuMemUnmap") &&
           resolve(a.memSetAccess, "cuMemSetAccess") && resolve(a.multicastCreate, "cuMulticastCreate") &&
           resolve(a.multicastAddDevice, "cuMulticastAddDevice") &&
           resolve(a.multicastBindMem, "cuMulticastBindMem") && resolve(a.multicastUnbind, "cuMulticastUnbind") &&
           resolve(a.multicastGetGranularity, "cuMulticastGetGranularity") &&
           resolve(a.deviceGetAttribute, "cuDeviceGetAttribute");
  }
  return a.ok ? &a : nullptr;
}

static bool check(CUresult r, const char* what) {
  if (r == CUDA_SUCCESS) return true;
  set_last_error("symm_heap: %s failed with CUresult %d", what, static_cast<int>(r));
  return false;
}

static CUmemAllocationProp local_prop(int device) {
  CUmemAllocationProp p;
  memset(&p, 0, sizeof(p));
  p.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  p.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  p.location.id = device;
  p.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return p;
}

static bool map_rw(DriverApi* d, CUdeviceptr* va, size_t size, size_t align, CUmemGenericAllocationHandle h,
                   int device) {
  if (!check(d->memAddressReserve(va, size, align, 0, 0), "cuMemAddressReserve")) return false;
  if (!check(d->memMap(*va, size, 0, h, 0), "cuMemMap")) return false;
  CUmemAccessDesc acc;
  memset(&acc, 0, sizeof(acc));
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = device;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  return check(d->memSetAccess(*va, size, &acc, 1), "cuMemSetAccess");
}

}  // namespace tw

using namespace tw;

// Size rounded up to what both the allocation and the multicast object accept.
extern "C" int tw_symm_granularity(int device, int world, unsigned long long* out) {
  DriverApi* d = api();
  if (!d) return 1;
  CUmemAllocationProp p = local_prop(device);
  size_t g = 0;
  if (!check(d->memGetAllocationGranularity(&g, &p, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED),
             "cuMemGetAllocationGranularity"))
    return 1;
  int mc_ok = 0;
  d->deviceGetAttribute(&mc_ok, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, device);
  if (mc_ok && world > 1) {
    CUmulticastObjectProp mp;
    memset(&mp, 0, sizeof(mp));
    mp.numDevices = world;
    mp.size = g;
    mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    size_t mg = 0;
    if (d->multicastGetGranularity(&mg, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS && mg > g) g = mg;
  }
  *out = g;
  return 0;
}

extern "C" int tw_symm_multicast_supported(int device) {
  DriverApi* d = api();
  if (!d) return 0;
  int ok = 0;
  d->deviceGetAttribute(&ok, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, device);
  return ok;
}

// Create this rank's physical allocation, map it locally, export it as a file descriptor.
extern "C" int tw_symm_alloc_local(int device, unsigned long long size, unsigned long long* handle_out,
                                   unsigned long long* va_out, int* fd_out) {
  DriverApi* d = api();
  if (!d) return 1;
  CUmemAllocationProp p = local_prop(device);
  CUmemGenericAllocationHandle h;
  if (!check(d->memCreate(&h, size, &p, 0), "cuMemCreate")) return 1;
  CUdeviceptr va = 0;
  if (!map_rw(d, &va, size, 0, h, device)) return 1;
  int fd = -1;
  if (!check(d->memExportToShareableHandle(&fd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0),
             "cuMemExportToShareableHandle"))
    return 1;
  *handle_out = static_cast<unsigned long long>(h);
  *va_out = static_cast<unsigned long long>(va);
  *fd_out = fd;
  return 0;
}

// Import a peer's allocation from its file descriptor and map it on this device.
extern "C" int tw_symm_import_peer(int device, int fd, unsigned long long size, unsigned long long* handle_out,
                                   unsigned long long* va_out) {
  DriverApi* d = api();
  if (!d) return 1;
  CUmemGenericAllocationHandle h;
  if (!check(d->memImportFromShareableHandle(&h, reinterpret_cast<void*>(static_cast<intptr_t>(fd)),
                                             CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR),
             "cuMemImportFromShareableHandle"))
    return 1;
  CUdeviceptr va = 0;
  if (!map_rw(d, &va, size, 0, h, device)) return 1;
  *handle_out = static_cast<unsigned long long>(h);
  *va_out = static_cast<unsigned long long>(va);
  return 0;
}

// Rank 0: create the multicast object and export it.
extern "C" int tw_symm_multicast_create(int world, unsigned long long size, unsigned long long* handle_out,
                                        int* fd_out) {
  DriverApi* d = api();
  if (!d) return 1;
  CUmulticastObjectProp mp;
  memset(&mp, 0, sizeof(mp));
  mp.numDevices = world;
  mp.size = size;
  mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  CUmemGenericAllocationHandle h;
  if (!check(d->multicastCreate(&h, &mp), "cuMulticastCreate")) return 1;
  int fd = -1;
  if (!check(d->memExportToShareableHandle(&fd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0),
             "cuMemExportToShareableHandle(multicast)"))
    return 1;
  *handle_out = static_cast<unsigned long long>(h);
  *fd_out = fd;
  return 0;
}

extern "C" int tw_symm_multicast_import(int fd, unsigned long long* handle_out) {
  DriverApi* d = api();
  if (!d) return 1;
  CUmemGenericAllocationHandle h;
  if (!check(d->memImportFromShareableHandle(&h, reinterpret_cast<void*>(static_cast<intptr_t>(fd)),
                                             CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR),
             "cuMemImportFromShareableHandle(multicast)"))
    return 1;
  *handle_out = static_cast<unsigned long long>(h);
  return 0;
}

// Every rank: join the multicast team. All ranks must have joined before anyone binds memory.
extern "C" int tw_symm_multicast_add_device(unsigned long long mc_handle, int device) {
  DriverApi* d = api();
  if (!d) return 1;
  return check(d->multicastAddDevice(static_cast<CUmemGenericAllocationHandle>(mc_handle), device),
               "cuMulticastAddDevice")
             ? 0
             : 1;
}

// Every rank: bind its physical allocation and map the multicast address range.
extern "C" int tw_symm_multicast_bind_map(unsigned long long mc_handle, unsigned long long local_handle, int device,
                                          unsigned long long size, unsigned long long* mc_va_out) {
  DriverApi* d = api();
  if (!d) return 1;
  if (!check(d->multicastBindMem(static_cast<CUmemGenericAllocationHandle>(mc_handle), 0,
                                 static_cast<CUmemGenericAllocationHandle>(local_handle), 0, size, 0),
             "cuMulticastBindMem"))
    return 1;
  CUdeviceptr va = 0;
  if (!map_rw(d, &va, size, 0, static_cast<CUmemGenericAllocationHandle>(mc_handle), device)) return 1;
  *mc_va_out = static_cast<unsigned long long>(va);
  return 0;
}

// Tear-down of one mapping (peer, local or multicast) and its handle. For the multicast object the
// caller unbinds first (unbind = 1) and every rank must have stopped using the multicast address.
extern "C" int tw_symm_release(unsigned long long va, unsigned long long size, unsigned long long handle, int unbind,
                               int device) {
  DriverApi* d = api();
  if (!d) return 1;
  bool ok = true;
  if (va != 0) {
    ok &= check(d->memUnmap(static_cast<CUdeviceptr>(va), size), "cuMemUnmap");
    ok &= check(d->memAddressFree(static_cast<CUdeviceptr>(va), size), "cuMemAddressFree");
  }
  if (unbind) ok &= check(d->multicastUnbind(static_cast<CUmemGenericAllocationHandle>(handle), device, 0, size),
                          "cuMulticastUnbind");
  if (handle != 0) ok &= check(d->memRelease(static_cast<CUmemGenericAllocationHandle>(handle)), "cuMemRelease");
  return ok ? 0 : 1;
}
