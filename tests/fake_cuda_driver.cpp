// Stand-in for the CUDA driver's virtual-memory API on machines without a GPU: "physical" allocations are host buffers,
// "virtual" ranges are numbers, a mapping ties one to the other. Lets the sleep-mode allocator's bookkeeping run on CPU.
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <map>

namespace {
struct Phys { unsigned char* buf; size_t size; };
std::map<unsigned long long, Phys> g_phys;                 // handle -> buffer
std::map<unsigned long long, unsigned long long> g_map;    // va -> handle
std::map<unsigned long long, size_t> g_reserved;           // va -> size
unsigned long long g_next_va = 0x100000000ull, g_next_handle = 1;
long long g_live_phys_bytes = 0, g_host_bytes = 0;
}  // namespace

extern "C" {
int cuInit(unsigned) { return 0; }
int cuGetErrorString(int, const char** s) { *s = "fake driver error"; return 0; }
int cuCtxSynchronize() { return 0; }
int cuMemGetAllocationGranularity(size_t* g, const void*, int) { *g = 2u << 20; return 0; }
int cuMemAddressReserve(unsigned long long* va, size_t size, size_t, unsigned long long, unsigned long long) {
  *va = g_next_va;
  g_next_va += (size + (2u << 20)) & ~((2ull << 20) - 1);
  g_reserved[*va] = size;
  return 0;
}
int cuMemAddressFree(unsigned long long va, size_t) { return g_reserved.erase(va) ? 0 : 1; }
int cuMemCreate(unsigned long long* h, size_t size, const void*, unsigned long long) {
  Phys p{static_cast<unsigned char*>(malloc(size)), size};
  if (!p.buf) return 2;
  memset(p.buf, 0xCD, size);  // fresh physical memory holds garbage
  *h = g_next_handle++;
  g_phys[*h] = p;
  g_live_phys_bytes += (long long)size;
  return 0;
}
int cuMemRelease(unsigned long long h) {
  auto it = g_phys.find(h);
  if (it == g_phys.end()) return 1;
  g_live_phys_bytes -= (long long)it->second.size;
  free(it->second.buf);
  g_phys.erase(it);
  return 0;
}
int cuMemMap(unsigned long long va, size_t, size_t, unsigned long long h, unsigned long long) {
  if (!g_reserved.count(va) || !g_phys.count(h) || g_map.count(va)) return 1;
  g_map[va] = h;
  return 0;
}
int cuMemUnmap(unsigned long long va, size_t) { return g_map.erase(va) ? 0 : 1; }
int cuMemSetAccess(unsigned long long va, size_t, const void*, size_t) { return g_map.count(va) ? 0 : 1; }
static unsigned char* resolve(unsigned long long addr, size_t n) {
  auto it = g_map.upper_bound(addr);
  if (it == g_map.begin()) return nullptr;
  --it;
  Phys& p = g_phys[it->second];
  if (addr + n > it->first + p.size) return nullptr;
  return p.buf + (addr - it->first);
}
int cuMemcpyDtoH_v2(void* dst, unsigned long long src, size_t n) {
  unsigned char* s = resolve(src, n);
  if (!s) return 700;  // an unmapped address: what a real device would fault on
  memcpy(dst, s, n);
  return 0;
}
int cuMemcpyHtoD_v2(unsigned long long dst, const void* src, size_t n) {
  unsigned char* d = resolve(dst, n);
  if (!d) return 700;
  memcpy(d, src, n);
  return 0;
}
int cuMemHostAlloc(void** p, size_t n, unsigned) { *p = malloc(n); g_host_bytes += (long long)n; return *p ? 0 : 2; }
int cuMemFreeHost(void* p) { free(p); return 0; }
long long fake_live_phys_bytes() { return g_live_phys_bytes; }
}
