// Sleep-capable device allocator on the CUDA virtual-memory-management API, pluggable into PyTorch's
// caching allocator (torch.cuda.memory.CUDAPluggableAllocator + torch.cuda.MemPool).
//
// Every allocation is a reserved virtual range with its own physical allocation mapped behind it.
// tw_vmm_sleep() copies the ranges whose tag is selected to pinned host memory, then unmaps and
// releases ALL physical memory while the virtual addresses stay reserved, so tensors keep their
// pointers; tw_vmm_wake() maps fresh physical memory at the same addresses and copies the saved
// contents back. Counterpart of the reference's cumem allocator (csrc/cumem_allocator.cpp:1-349,
// vllm/device_allocator/cumem.py:1-280), which keeps the bookkeeping in Python callbacks; here the
// table lives in this file and Python only sets the tag and calls sleep / wake.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>
#include <sys/types.h>

#include <map>
#include <mutex>

#include "tw_host.h"

namespace tw {
namespace {

struct Vmm {
  CUresult (*memGetAllocationGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags);
  CUresult (*memCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long);
  CUresult (*memRelease)(CUmemGenericAllocationHandle);
  CUresult (*memAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long);
  CUresult (*memAddressFree)(CUdeviceptr, size_t);
  CUresult (*memMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long);
  CUresult (*memUnmap)(CUdeviceptr, size_t);
  CUresult (*memSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t);
  bool ok;
};

template <typename F>
bool resolve(const char* name, F* out) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess ||
      p == nullptr) {
    set_last_error("driver entry point %s is not available", name);
    return false;
  }
  *out = reinterpret_cast<F>(p);
  return true;
}

Vmm* vmm() {
  static Vmm v;
  static std::once_flag once;
  std::call_once(once, []() {
    v.ok = resolve("cuMemGetAllocationGranularity", &v.memGetAllocationGranularity) &&
           resolve("cuMemCreate", &v.memCreate) && resolve("cuMemRelease", &v.memRelease) &&
           resolve("cuMemAddressReserve", &v.memAddressReserve) && resolve("cuMemAddressFree", &v.memAddressFree) &&
           resolve("cuMemMap", &v.memMap) && resolve("cuMemUnmap", &v.memUnmap) &&
           resolve("cuMemSetAccess", &v.memSetAccess);
  });
  return v.ok ? &v : nullptr;
}

struct Block {
  size_t size;        // mapped size (a multiple of the granularity)
  int device;
  int tag;
  bool mapped;
  CUmemGenericAllocationHandle handle;
  void* host_copy;    // pinned host copy while asleep (or null: contents discarded)
};

std::mutex g_mu;
std::map<CUdeviceptr, Block> g_blocks;
int g_tag = 0;

CUmemAllocationProp prop_for(int device) {
  CUmemAllocationProp p;
  memset(&p, 0, sizeof(p));
  p.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  p.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  p.location.id = device;
  return p;
}

bool fail(CUresult r, const char* what) {
  if (r == CUDA_SUCCESS) return false;
  set_last_error("%s failed with CUresult %d", what, static_cast<int>(r));
  return true;
}

// Physical memory behind [va, va + size) on `device`, readable and writable from it.
bool back_with_memory(Vmm* v, CUdeviceptr va, size_t size, int device, CUmemGenericAllocationHandle* h) {
  CUmemAllocationProp p = prop_for(device);
  if (fail(v->memCreate(h, size, &p, 0), "cuMemCreate")) return false;
  if (fail(v->memMap(va, size, 0, *h, 0), "cuMemMap")) {
    v->memRelease(*h);
    return false;
  }
  CUmemAccessDesc acc;
  memset(&acc, 0, sizeof(acc));
  acc.location = p.location;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  if (fail(v->memSetAccess(va, size, &acc, 1), "cuMemSetAccess")) {
    v->memUnmap(va, size);
    v->memRelease(*h);
    return false;
  }
  return true;
}

}  // namespace
}  // namespace tw

using namespace tw;

// Allocation hook with the signature torch's CUDAPluggableAllocator expects.
extern "C" void* tw_vmm_malloc(ssize_t size, int device, cudaStream_t /*stream*/) {
  Vmm* v = vmm();
  if (v == nullptr || size <= 0) return nullptr;
  cudaSetDevice(device);
  cudaFree(nullptr);   // make sure the primary context exists before driver calls
  CUmemAllocationProp p = prop_for(device);
  size_t gran = 0;
  if (fail(v->memGetAllocationGranularity(&gran, &p, CU_MEM_ALLOC_GRANULARITY_MINIMUM), "cuMemGetAllocationGranularity"))
    return nullptr;
  const size_t bytes = (static_cast<size_t>(size) + gran - 1) / gran * gran;
  CUdeviceptr va = 0;
  if (fail(v->memAddressReserve(&va, bytes, 0, 0, 0), "cuMemAddressReserve")) return nullptr;
  CUmemGenericAllocationHandle h;
  if (!back_with_memory(v, va, bytes, device, &h)) {
    v->memAddressFree(va, bytes);
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(g_mu);
  g_blocks[va] = Block{bytes, device, g_tag, true, h, nullptr};
  return reinterpret_cast<void*>(va);
}

extern "C" void tw_vmm_free(void* ptr, ssize_t /*size*/, int /*device*/, cudaStream_t /*stream*/) {
  Vmm* v = vmm();
  if (v == nullptr || ptr == nullptr) return;
  const CUdeviceptr va = reinterpret_cast<CUdeviceptr>(ptr);
  Block b;
  {
    std::lock_guard<std::mutex> lock(g_mu);
    auto it = g_blocks.find(va);
    if (it == g_blocks.end()) return;
    b = it->second;
    g_blocks.erase(it);
  }
  if (b.mapped) {
    v->memUnmap(va, b.size);
    v->memRelease(b.handle);
  }
  if (b.host_copy != nullptr) cudaFreeHost(b.host_copy);
  v->memAddressFree(va, b.size);
}

// Tag given to allocations made from now on (e.g. 1 = weights, 2 = KV cache).
extern "C" int tw_vmm_set_tag(int tag) {
  std::lock_guard<std::mutex> lock(g_mu);
  g_tag = tag;
  return 0;
}

// Releases the physical memory of every mapped block. Blocks whose tag has its bit set in
// `offload_tag_mask` (bit t for tag t) are saved to pinned host memory first; the others lose their contents.
// The caller synchronises the device beforehand; copies here are synchronous.
extern "C" int tw_vmm_sleep(unsigned int offload_tag_mask) {
  Vmm* v = vmm();
  if (v == nullptr) return 1;
  std::lock_guard<std::mutex> lock(g_mu);
  for (auto& kv : g_blocks) {
    Block& b = kv.second;
    if (!b.mapped) continue;
    cudaSetDevice(b.device);
    if (b.tag >= 0 && b.tag < 32 && ((offload_tag_mask >> b.tag) & 1u)) {
      if (cudaMallocHost(&b.host_copy, b.size) != cudaSuccess) {
        b.host_copy = nullptr;
        set_last_error("vmm_sleep: no pinned host memory for %zu bytes", b.size);
        return 1;
      }
      if (cudaMemcpy(b.host_copy, reinterpret_cast<void*>(kv.first), b.size, cudaMemcpyDeviceToHost) != cudaSuccess) {
        set_last_error("vmm_sleep: device-to-host copy failed");
        return 1;
      }
    }
    if (fail(v->memUnmap(kv.first, b.size), "cuMemUnmap")) return 1;
    if (fail(v->memRelease(b.handle), "cuMemRelease")) return 1;
    b.mapped = false;
  }
  return 0;
}

// Maps fresh physical memory behind every sleeping block whose tag is selected (all tags: 0xffffffff) and
// restores saved contents.
extern "C" int tw_vmm_wake(unsigned int tag_mask) {
  Vmm* v = vmm();
  if (v == nullptr) return 1;
  std::lock_guard<std::mutex> lock(g_mu);
  for (auto& kv : g_blocks) {
    Block& b = kv.second;
    if (b.mapped) continue;
    if (!(b.tag >= 0 && b.tag < 32 && ((tag_mask >> b.tag) & 1u))) continue;
    cudaSetDevice(b.device);
    if (!back_with_memory(v, kv.first, b.size, b.device, &b.handle)) return 1;
    b.mapped = true;
    if (b.host_copy != nullptr) {
      if (cudaMemcpy(reinterpret_cast<void*>(kv.first), b.host_copy, b.size, cudaMemcpyHostToDevice) != cudaSuccess) {
        set_last_error("vmm_wake: host-to-device copy failed");
        return 1;
      }
      cudaFreeHost(b.host_copy);
      b.host_copy = nullptr;
    }
  }
  return 0;
}

// which: 0 bytes currently backed by device memory, 1 bytes reserved in total, 2 bytes held in host copies.
extern "C" long long tw_vmm_bytes(int which) {
  std::lock_guard<std::mutex> lock(g_mu);
  long long n = 0;
  for (const auto& kv : g_blocks) {
    const Block& b = kv.second;
    if (which == 0 && b.mapped) n += static_cast<long long>(b.size);
    if (which == 1) n += static_cast<long long>(b.size);
    if (which == 2 && b.host_copy != nullptr) n += static_cast<long long>(b.size);
  }
  return n;
}
