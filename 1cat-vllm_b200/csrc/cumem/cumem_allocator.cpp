// Sleep-mode allocator: device memory whose physical pages can be given back to the driver and brought back at the same
// virtual address, so tensors (weights, KV cache, captured CUDA graphs that point into them) stay valid across a sleep.
//
// Every allocation reserves a virtual range (cuMemAddressReserve), creates physical memory (cuMemCreate) and maps it
// (cuMemMap + cuMemSetAccess). Allocations carry the tag that was current when they were made ("weights", "kv_cache", ...).
// sleep(offload_mask, discard_mask): allocations whose tag is in offload_mask are copied to pinned host memory first; those in
// either mask are unmapped and their physical memory released; the virtual range stays reserved. wake(mask) creates and maps new
// physical memory at the same addresses and copies the host backups back.
//
// The entry points `onecat_cumem_malloc` / `onecat_cumem_free` have the signature torch.cuda.memory.CUDAPluggableAllocator
// expects; everything else is called through ctypes. The CUDA driver is loaded with dlopen at first use (no link-time
// dependency; ONECAT_CUMEM_DRIVER names a stand-in library for tests on machines without a GPU).
// (reference: csrc/cumem_allocator.cpp; vllm/device_allocator/cumem.py:93 CuMemAllocator, sleep :241, wake_up :307)
#include <cuda.h>
#include <dlfcn.h>
#include <stddef.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/types.h>

#include <mutex>
#include <string>
#include <unordered_map>

namespace {

typedef CUresult CUresult_;
typedef CUdeviceptr CUdeviceptr_;
typedef CUmemGenericAllocationHandle CUhandle_;
typedef CUmemAllocationProp AllocProp;
typedef CUmemAccessDesc AccessDesc;

struct Driver {
  void* lib = nullptr;
  CUresult_ (*init)(unsigned) = nullptr;
  CUresult_ (*granularity)(size_t*, const AllocProp*, CUmemAllocationGranularity_flags) = nullptr;
  CUresult_ (*reserve)(CUdeviceptr_*, size_t, size_t, CUdeviceptr_, unsigned long long) = nullptr;
  CUresult_ (*addr_free)(CUdeviceptr_, size_t) = nullptr;
  CUresult_ (*create)(CUhandle_*, size_t, const AllocProp*, unsigned long long) = nullptr;
  CUresult_ (*release)(CUhandle_) = nullptr;
  CUresult_ (*map)(CUdeviceptr_, size_t, size_t, CUhandle_, unsigned long long) = nullptr;
  CUresult_ (*unmap)(CUdeviceptr_, size_t) = nullptr;
  CUresult_ (*set_access)(CUdeviceptr_, size_t, const AccessDesc*, size_t) = nullptr;
  CUresult_ (*d2h)(void*, CUdeviceptr_, size_t) = nullptr;
  CUresult_ (*h2d)(CUdeviceptr_, const void*, size_t) = nullptr;
  CUresult_ (*host_alloc)(void**, size_t, unsigned) = nullptr;
  CUresult_ (*host_free)(void*) = nullptr;
  CUresult_ (*ctx_sync)() = nullptr;
  CUresult_ (*err_string)(CUresult_, const char**) = nullptr;
};

struct Block {
  size_t size = 0;        // mapped size (multiple of the granularity)
  int device = 0, tag = 0;
  CUhandle_ handle = 0;
  bool mapped = false;
  void* host = nullptr;   // pinned backup while asleep
};

std::mutex g_mu;
Driver g_drv;
std::unordered_map<CUdeviceptr_, Block> g_blocks;
int g_tag = 0;
std::string g_err;

template <typename F>
bool sym(F& f, const char* name) {
  f = reinterpret_cast<F>(dlsym(g_drv.lib, name));
  if (!f) g_err = std::string("driver symbol missing: ") + name;
  return f != nullptr;
}

bool load_driver() {
  if (g_drv.lib) return true;
  const char* path = getenv("ONECAT_CUMEM_DRIVER");
  g_drv.lib = dlopen(path && *path ? path : "libcuda.so.1", RTLD_NOW | RTLD_GLOBAL);
  if (!g_drv.lib) {
    g_err = std::string("cannot load the CUDA driver: ") + dlerror();
    return false;
  }
  bool ok = sym(g_drv.init, "cuInit") && sym(g_drv.granularity, "cuMemGetAllocationGranularity") && sym(g_drv.reserve, "cuMemAddressReserve") &&
            sym(g_drv.addr_free, "cuMemAddressFree") && sym(g_drv.create, "cuMemCreate") && sym(g_drv.release, "cuMemRelease") &&
            sym(g_drv.map, "cuMemMap") && sym(g_drv.unmap, "cuMemUnmap") && sym(g_drv.set_access, "cuMemSetAccess") &&
            sym(g_drv.d2h, "cuMemcpyDtoH_v2") && sym(g_drv.h2d, "cuMemcpyHtoD_v2") && sym(g_drv.host_alloc, "cuMemHostAlloc") &&
            sym(g_drv.host_free, "cuMemFreeHost") && sym(g_drv.ctx_sync, "cuCtxSynchronize") && sym(g_drv.err_string, "cuGetErrorString");
  if (!ok) {
    dlclose(g_drv.lib);
    g_drv.lib = nullptr;
    return false;
  }
  g_drv.init(0);
  return true;
}

bool check(CUresult_ r, const char* what) {
  if (r == CUDA_SUCCESS) return true;
  const char* s = nullptr;
  if (g_drv.err_string) g_drv.err_string(r, &s);
  g_err = std::string(what) + " failed: " + (s ? s : "unknown") + " (" + std::to_string((int)r) + ")";
  return false;
}

AllocProp prop_for(int device) {
  AllocProp p;
  memset(&p, 0, sizeof(p));
  p.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  p.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  p.location.id = device;
  return p;
}

bool map_block(CUdeviceptr_ va, Block& b) {
  AllocProp prop = prop_for(b.device);
  if (!check(g_drv.create(&b.handle, b.size, &prop, 0), "cuMemCreate")) return false;
  if (!check(g_drv.map(va, b.size, 0, b.handle, 0), "cuMemMap")) {
    g_drv.release(b.handle);
    return false;
  }
  AccessDesc acc;
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = b.device;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  if (!check(g_drv.set_access(va, b.size, &acc, 1), "cuMemSetAccess")) {
    g_drv.unmap(va, b.size);
    g_drv.release(b.handle);
    return false;
  }
  b.mapped = true;
  return true;
}

bool unmap_block(CUdeviceptr_ va, Block& b) {
  if (!b.mapped) return true;
  if (!check(g_drv.unmap(va, b.size), "cuMemUnmap")) return false;
  if (!check(g_drv.release(b.handle), "cuMemRelease")) return false;
  b.mapped = false;
  b.handle = 0;
  return true;
}

}  // namespace

extern "C" {

__attribute__((visibility("default"))) void* onecat_cumem_malloc(ssize_t size, int device, void* /*stream*/) {
  std::lock_guard<std::mutex> lock(g_mu);
  if (size <= 0 || !load_driver()) return nullptr;
  AllocProp prop = prop_for(device);
  size_t gran = 0;
  if (!check(g_drv.granularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_MINIMUM), "cuMemGetAllocationGranularity") || gran == 0) return nullptr;
  Block b;
  b.size = ((size_t)size + gran - 1) / gran * gran;
  b.device = device;
  b.tag = g_tag;
  CUdeviceptr_ va = 0;
  if (!check(g_drv.reserve(&va, b.size, gran, 0, 0), "cuMemAddressReserve")) return nullptr;
  if (!map_block(va, b)) {
    g_drv.addr_free(va, b.size);
    return nullptr;
  }
  g_blocks[va] = b;
  return reinterpret_cast<void*>(va);
}

__attribute__((visibility("default"))) void onecat_cumem_free(void* ptr, ssize_t /*size*/, int /*device*/, void* /*stream*/) {
  std::lock_guard<std::mutex> lock(g_mu);
  auto it = g_blocks.find(reinterpret_cast<CUdeviceptr_>(ptr));
  if (it == g_blocks.end()) return;
  Block& b = it->second;
  unmap_block(it->first, b);
  if (b.host) g_drv.host_free(b.host);
  g_drv.addr_free(it->first, b.size);
  g_blocks.erase(it);
}

// Allocations made from now on carry this tag (bit index 0..30 of the masks below).
__attribute__((visibility("default"))) void onecat_cumem_set_tag(int tag) {
  std::lock_guard<std::mutex> lock(g_mu);
  g_tag = tag;
}

// Returns the number of bytes released, or -1 on error (see onecat_cumem_last_error).
__attribute__((visibility("default"))) long long onecat_cumem_sleep(unsigned offload_mask, unsigned discard_mask) {
  std::lock_guard<std::mutex> lock(g_mu);
  if (!g_drv.lib) return 0;
  if (!check(g_drv.ctx_sync(), "cuCtxSynchronize")) return -1;
  long long freed = 0;
  for (auto& kv : g_blocks) {
    Block& b = kv.second;
    const unsigned bit = 1u << b.tag;
    if (!b.mapped || !((offload_mask | discard_mask) & bit)) continue;
    if (offload_mask & bit) {
      if (!b.host && !check(g_drv.host_alloc(&b.host, b.size, 0), "cuMemHostAlloc")) return -1;
      if (!check(g_drv.d2h(b.host, kv.first, b.size), "cuMemcpyDtoH")) return -1;
    }
    if (!unmap_block(kv.first, b)) return -1;
    freed += (long long)b.size;
  }
  return freed;
}

// Maps fresh physical memory under every sleeping allocation whose tag is in the mask and restores offloaded contents.
__attribute__((visibility("default"))) long long onecat_cumem_wake(unsigned mask) {
  std::lock_guard<std::mutex> lock(g_mu);
  if (!g_drv.lib) return 0;
  long long mapped = 0;
  for (auto& kv : g_blocks) {
    Block& b = kv.second;
    if (b.mapped || !(mask & (1u << b.tag))) continue;
    if (!map_block(kv.first, b)) return -1;
    if (b.host) {
      if (!check(g_drv.h2d(kv.first, b.host, b.size), "cuMemcpyHtoD")) return -1;
      g_drv.host_free(b.host);
      b.host = nullptr;
    }
    mapped += (long long)b.size;
  }
  return mapped;
}

// what: 0 bytes mapped, 1 bytes asleep (virtual range kept, no physical memory), 2 bytes of host backups, 3 live allocations
__attribute__((visibility("default"))) long long onecat_cumem_stat(int what, unsigned mask) {
  std::lock_guard<std::mutex> lock(g_mu);
  long long v = 0;
  for (auto& kv : g_blocks) {
    const Block& b = kv.second;
    if (!(mask & (1u << b.tag))) continue;
    if (what == 0 && b.mapped) v += (long long)b.size;
    if (what == 1 && !b.mapped) v += (long long)b.size;
    if (what == 2 && b.host) v += (long long)b.size;
    if (what == 3) v += 1;
  }
  return v;
}

__attribute__((visibility("default"))) const char* onecat_cumem_last_error() {
  static std::string copy;
  std::lock_guard<std::mutex> lock(g_mu);
  copy = g_err;
  return copy.c_str();
}

}  // extern "C"
