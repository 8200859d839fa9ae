// Expert-parallel token exchange over NVLink peer memory: each rank routes its own tokens, stores every (token, expert) row
// straight into the recv buffer of the rank that owns the expert, runs the grouped GEMMs over what it received, and stores each
// expert output row straight back into the sender's return buffer, where the sender forms the weighted sum per token.
//
// The recv buffer needs no second pass: its layout is fixed before a single row moves. Every rank publishes how many pairs it
// routes to every expert (one [E] row of a [ranks][E] table in each peer's slab); from the complete table every rank derives,
// identically, where its rows for expert e begin on the owner:
//     base(owner, e) = sum of totals of the owner's experts before e          (experts are contiguous, so GEMM tiles are too)
//     mine(e)        = base + rows of lower-numbered ranks for e
// so the owner's buffer is already expert-major "slot" order and the grouped GEMM consumes it as it lies.
//
// Synchronisation: one int32 per (stage, source rank) in every slab, written with st.release.sys after a system fence and polled
// with ld.acquire.sys under a time limit; values are a sequence number kept in device memory, so replays inside a CUDA graph need
// no reset. A wait that runs out raises the status word and the kernel returns; later stages then find their flags missing and
// give up the same way. Stages: 0 counts published, 1 rows dispatched, 2 outputs returned, 3 combined rows gathered.
// Rows written by a peer are read with ld.global.cg (L2), never through L1, in the kernel that waited for them.
// (reference: distributed/device_communicators/all2all.py:84-137 AgRs / DeepEP managers; layers/fused_moe/modular_kernel.py:1036-1684
//  prepare / finalize; csrc/moe/moe_permute_unpermute_op.cu:240)
#include "comm.h"
#include "common.cuh"

namespace oc {
namespace {

__device__ __forceinline__ void st_flag_release(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_flag_acquire(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ bool wait_flag(const int* p, int want, uint64_t limit_ns) {
  uint64_t t0 = 0;
  uint32_t spins = 0;
  while (ld_flag_acquire(p) - want < 0) {
    if ((++spins & 255u) == 0) {
      const uint64_t now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > limit_ns) return false;
    }
  }
  return true;
}

__device__ __forceinline__ int* flag_of(const EpParams& p, int rank, int stage, int src) {
  return reinterpret_cast<int*>(p.slab[rank] + p.off_flags) + stage * kMaxRanks + src;
}

// Threads 0..n-1 of the CTA wait for stage `stage` of every source; the result is the same for the whole CTA.
__device__ __forceinline__ bool cta_wait_stage(const EpParams& p, int stage, int seq, int* s_ok) {
  if (threadIdx.x == 0) *s_ok = 1;
  __syncthreads();
  if (threadIdx.x < p.n && !wait_flag(flag_of(p, p.me, stage, threadIdx.x), seq, p.wait_ns)) {
    *s_ok = 0;
    atomicOr(&g_status, ST_PEER_TIMEOUT);
  }
  __syncthreads();
  return *s_ok != 0;
}

// After a kernel's peer stores: the last CTA to finish tells every rank that this rank's part of `stage` is complete.
__device__ __forceinline__ void grid_signal_stage(const EpParams& p, int stage, int seq, int* done) {
  __threadfence_system();
  __syncthreads();
  __shared__ int s_last;
  if (threadIdx.x == 0) s_last = (atomicAdd(done, 1) == (int)gridDim.x - 1);
  __syncthreads();
  if (!s_last) return;
  __threadfence_system();
  if (threadIdx.x < p.n) st_flag_release(flag_of(p, threadIdx.x, stage, p.me), seq);
  if (threadIdx.x == 0) *done = 0;
}

// ---- stage 0: histogram of this rank's pairs, exchange of the rows of the count table, layout of every destination ------------
__global__ void __launch_bounds__(1024) ep_count_exchange_kernel(const EpParams p) {
  __shared__ int hist[1024], tot[1024], before[1024], base[1024];
  __shared__ int s_seq, s_ok;
  const int E = p.E, n = p.n, El = p.E_local;
  if (threadIdx.x == 0) {
    s_seq = p.seq[0] + 1;
    p.seq[0] = s_seq;
    p.done[0] = p.done[1] = p.done[2] = 0;
  }
  for (int e = threadIdx.x; e < 1024; e += blockDim.x) hist[e] = 0;
  __syncthreads();
  const int seq = s_seq;
  for (int i = threadIdx.x; i < p.n_pairs; i += blockDim.x) {
    const int e = p.ids[i];
    // ids outside the expert range are skipped here and in every later stage: padded rows of a captured batch carry whatever
    // their (unused) hidden state routes to
    if (e >= 0 && e < E) atomicAdd(&hist[e], 1);
  }
  __syncthreads();
  for (int r = 0; r < n; ++r) {
    int* dst = reinterpret_cast<int*>(p.slab[r] + p.off_counts) + (size_t)p.me * E;
    for (int e = threadIdx.x; e < E; e += blockDim.x) dst[e] = hist[e];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < n) st_flag_release(flag_of(p, threadIdx.x, 0, p.me), seq);
  const bool ok = cta_wait_stage(p, 0, seq, &s_ok);
  const int* table = reinterpret_cast<const int*>(p.slab[p.me] + p.off_counts);
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int t = 0, b = 0;
    for (int s = 0; s < n; ++s) {
      const int c = ok ? __ldcg(table + (size_t)s * E + e) : 0;
      if (s < p.me) b += c;
      t += c;
    }
    tot[e] = t;
    before[e] = b;
  }
  __syncthreads();
  if (threadIdx.x < n) {  // exclusive scan inside each owner's contiguous expert range
    int acc = 0;
    for (int el = 0; el < El; ++el) {
      const int e = threadIdx.x * El + el;
      base[e] = acc;
      acc += tot[e];
    }
    if (threadIdx.x == p.me && acc > p.cap) {  // cannot happen when cap covers every pair of every rank; checked all the same
      atomicOr(&g_status, ST_BOUNDS);
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    p.send_base[e] = ok ? base[e] + before[e] : -1;
    p.cursor[e] = 0;
  }
  for (int el = threadIdx.x; el < El; el += blockDim.x) p.counts_local[el] = ok ? tot[p.me * El + el] : 0;
}

// ---- stage 1: one warp per pair stores the token's row (and where it came from) into the owner's recv buffer -------------------
__global__ void __launch_bounds__(256) ep_dispatch_kernel(const EpParams p) {
  const int lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
  const int seq = p.seq[0];
  for (int pair = blockIdx.x * wpb + (threadIdx.x >> 5); pair < p.n_pairs; pair += gridDim.x * wpb) {
    const int e = p.ids[pair];
    if (e < 0 || e >= p.E) continue;
    const int sb = p.send_base[e];
    if (sb < 0) continue;
    int slot = 0;
    if (lane == 0) slot = sb + atomicAdd(&p.cursor[e], 1);
    slot = __shfl_sync(0xffffffffu, slot, 0);
    if (slot >= p.cap) continue;
    const int owner = e / p.E_local;
    const uint4* src = reinterpret_cast<const uint4*>(p.x + (size_t)(pair / p.k) * p.ldx);
    uint4* dst = reinterpret_cast<uint4*>(p.slab[owner] + p.off_recv_x) + (size_t)slot * (p.H / 8);
    for (int i = lane; i < p.H / 8; i += 32) dst[i] = src[i];
    if (lane == 0) reinterpret_cast<int*>(p.slab[owner] + p.off_recv_meta)[slot] = (p.me << 24) | pair;
  }
  grid_signal_stage(p, 1, seq, p.done + 0);
}

// One CTA: returns once every source has finished `stage` (placed in the stream before a consumer that cannot wait itself).
__global__ void __launch_bounds__(32) ep_wait_kernel(const EpParams p, int stage) {
  __shared__ int s_ok;
  cta_wait_stage(p, stage, p.seq[0], &s_ok);
}

// ---- stage 2: one warp per received slot stores the expert output row back to the rank and pair it came from -------------------
__global__ void __launch_bounds__(256) ep_return_kernel(const EpParams p, const __nv_bfloat16* __restrict__ a2) {
  const int lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
  const int seq = p.seq[0];
  const int total = min(p.total_slots[0], p.cap);
  const int* meta = reinterpret_cast<const int*>(p.slab[p.me] + p.off_recv_meta);
  for (int slot = blockIdx.x * wpb + (threadIdx.x >> 5); slot < total; slot += gridDim.x * wpb) {
    const int m = __ldcg(meta + slot);
    const int src = (m >> 24) & 0xff, pair = m & 0xffffff;
    if (src >= p.n || pair >= p.ret_rows) {
      atomicOr(&g_status, ST_BOUNDS);
      continue;
    }
    const uint4* from = reinterpret_cast<const uint4*>(a2 + (size_t)slot * p.H);
    uint4* to = reinterpret_cast<uint4*>(p.slab[src] + p.off_ret) + (size_t)pair * (p.H / 8);
    for (int i = lane; i < p.H / 8; i += 32) to[i] = from[i];
  }
  grid_signal_stage(p, 2, seq, p.done + 1);
}

// ---- stage 3: weighted sum over each token's k returned rows; optionally stored into every rank's gather buffer ---------------
__global__ void __launch_bounds__(128) ep_combine_kernel(const EpParams p, const float* __restrict__ w, __nv_bfloat16* __restrict__ y) {
  __shared__ int s_ok;
  const int seq = p.seq[0];
  const bool ok = cta_wait_stage(p, 2, seq, &s_ok);
  const __nv_bfloat16* ret = reinterpret_cast<const __nv_bfloat16*>(p.slab[p.me] + p.off_ret);
  const int cols = p.H / 8;
  if (ok) {
    for (int t = blockIdx.x; t < p.T; t += gridDim.x) {
      for (int cv = threadIdx.x; cv < cols; cv += blockDim.x) {
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int j = 0; j < p.k; ++j) {
          const int e = p.ids[t * p.k + j];
          if (e < 0 || e >= p.E) continue;
          const float wj = w[t * p.k + j];
          const uint4 v = __ldcg(reinterpret_cast<const uint4*>(ret + (size_t)(t * p.k + j) * p.H) + cv);
          const __nv_bfloat16* vp = reinterpret_cast<const __nv_bfloat16*>(&v);
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[i] += wj * __bfloat162float(vp[i]);
        }
        uint4 o;
        __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(&o);
#pragma unroll
        for (int i = 0; i < 8; ++i) op[i] = __float2bfloat16(acc[i]);
        if (y != nullptr) reinterpret_cast<uint4*>(y + (size_t)t * p.H)[cv] = o;
        if (p.gather)
          for (int r = 0; r < p.n; ++r) (reinterpret_cast<uint4*>(p.slab[r] + p.off_gather) + (size_t)(p.t_off + t) * cols)[cv] = o;
      }
    }
  }
  if (p.gather) grid_signal_stage(p, 3, seq, p.done + 2);
}

}  // namespace

int ep_count_exchange_launch(const EpParams& p, cudaStream_t st) {
  if (p.E > 1024 || p.n > kMaxRanks || p.E_local * p.n != p.E || p.H % 8 || p.n_pairs >= (1 << 24)) return -1;
  ep_count_exchange_kernel<<<1, 1024, 0, st>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
int ep_dispatch_launch(const EpParams& p, int sms, cudaStream_t st) {
  const int grid = max(1, min((p.n_pairs + 7) / 8, sms * 8));
  ep_dispatch_kernel<<<grid, 256, 0, st>>>(p);
  ep_wait_kernel<<<1, 32, 0, st>>>(p, 1);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
int ep_return_launch(const EpParams& p, const void* a2, int sms, cudaStream_t st) {
  const int grid = max(1, min((p.cap + 7) / 8, sms * 8));
  ep_return_kernel<<<grid, 256, 0, st>>>(p, (const __nv_bfloat16*)a2);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
int ep_combine_launch(const EpParams& p, const float* w, void* y, int sms, cudaStream_t st) {
  const int grid = max(1, min(p.T, sms * 8));
  ep_combine_kernel<<<grid, 128, 0, st>>>(p, w, (__nv_bfloat16*)y);
  if (p.gather) ep_wait_kernel<<<1, 32, 0, st>>>(p, 3);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
unsigned int ep_read_status(bool clear) { return read_status_tu(clear); }
void ep_read_status_async(unsigned int* dst, cudaStream_t st) { read_status_tu_async(dst, st); }

}  // namespace oc
