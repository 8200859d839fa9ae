// Tensor-parallel reductions over NVLink peer memory, fused with the residual add and RMSNorm that follow them.
//
// Every rank owns a slab ("symmetric heap") obtained with cudaMalloc and mapped into all other ranks through CUDA IPC
// handles, so a kernel can load a peer's partial sums with plain ld.global and store into a peer with st.global; NVSwitch
// gives each pair full bandwidth. Synchronisation is a flag per (source rank, CTA) written with st.release.sys into the
// consumer's slab and polled locally with ld.acquire.sys. Flags carry a per-CTA sequence number kept in device memory, so
// the protocol needs no resets and replays unchanged inside CUDA graphs. All polls are bounded: on expiry the kernel raises
// the status word, skips its work and returns.
//   mode ONE_SHOT  (decode-sized T): every rank sums all ranks' partial rows itself  -> replicated residual and output.
//   mode TWO_SHOT  (prefill-sized T): reduce-scatter + all-gather in one kernel: a rank reduces the rows it owns, normalises
//                  them and pushes the normalised rows into every peer's gather buffer; the residual stays row-sharded.
// Sums run in rank order 0..tp-1 on every rank, so all ranks obtain bit-identical results.
// (reference: csrc/custom_all_reduce.cuh:414 one-stage, :770 two-stage, :436 fused all-reduce + Gemma RMSNorm;
//  compilation/passes/fusion/allreduce_rms_fusion.py:199)
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
// waits until *p >= want; false on timeout
__device__ __forceinline__ bool wait_flag(const int* p, int want, uint64_t limit_ns) {
  uint64_t t0 = 0;
  uint32_t spins = 0;
  while (ld_flag_acquire(p) - want < 0) {
    if ((++spins & 255u) == 0) {  // the clock is slow to read: look at it once per 256 polls
      const uint64_t now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > limit_ns) return false;
    }
  }
  return true;
}

__device__ __forceinline__ float block_sum256(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (threadIdx.x < 8) ? red[threadIdx.x] : 0.f;
  if (warp == 0) {
    t = warp_sum(t);
    if (lane == 0) red[8] = t;
  }
  __syncthreads();
  return red[8];
}

template <int VEC_ITERS>
__global__ void __launch_bounds__(256) tp_reduce_norm_kernel(const CommParams p) {
  __shared__ float red[9];
  __shared__ int s_seq, s_ok;
  const int b = blockIdx.x;
  const int tp = p.tp, me = p.rank;
  pdl_trigger();
  // ---- phase 0: tell every rank that this rank's partial sums are complete (the producing GEMM ran earlier on this stream)
  if (threadIdx.x == 0) {
    int seq = p.seq_local[b] + 1;
    p.seq_local[b] = seq;
    s_seq = seq;
    s_ok = 1;
    __threadfence_system();
  }
  __syncthreads();
  const int seq = s_seq;
  if (threadIdx.x < tp) st_flag_release(p.flags[threadIdx.x] + (size_t)(p.phase * 2 * tp + me) * kMaxCommBlocks + b, seq);
  if (threadIdx.x < tp) {
    if (!wait_flag(p.flags[me] + (size_t)(p.phase * 2 * tp + threadIdx.x) * kMaxCommBlocks + b, seq, p.wait_ns)) {
      s_ok = 0;
      atomicOr(&g_status, ST_PEER_TIMEOUT);
    }
  }
  __syncthreads();
  const bool ok = s_ok != 0;

  // ---- phase 1: rows of this CTA
  int row_lo, row_hi;
  if (p.mode == COMM_ONE_SHOT) {
    row_lo = 0;
    row_hi = p.T;
  } else {
    const int per = (p.T + tp - 1) / tp;
    row_lo = min(me * per, p.T);
    row_hi = min(row_lo + per, p.T);
  }
  if (ok) {
    for (int t = row_lo + b; t < row_hi; t += gridDim.x) {
      float v[VEC_ITERS][8];
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < VEC_ITERS; ++i) {
        const int c = (i * 256 + threadIdx.x) * 8;
        if (c < p.H) {
          float acc[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] = 0.f;
          for (int r = 0; r < tp; ++r) {
            const uint4 a = *reinterpret_cast<const uint4*>(p.part[r] + (size_t)t * p.H + c);
            const __nv_bfloat16* ap = reinterpret_cast<const __nv_bfloat16*>(&a);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] += __bfloat162float(ap[j]);
          }
          if (p.residual_in != nullptr) {
            const uint4 rr = *reinterpret_cast<const uint4*>(p.residual_in + (size_t)t * p.H + c);
            const __nv_bfloat16* rp = reinterpret_cast<const __nv_bfloat16*>(&rr);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] += __bfloat162float(rp[j]);
          }
          uint4 o;
          __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(&o);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            op[j] = __float2bfloat16(acc[j]);
            v[i][j] = __bfloat162float(op[j]);
            ss += v[i][j] * v[i][j];
          }
          if (p.residual_out != nullptr) *reinterpret_cast<uint4*>(p.residual_out + (size_t)t * p.H + c) = o;
        }
      }
      float inv = 1.f;
      if (p.w != nullptr) {
        const float tot = block_sum256(ss, red);
        inv = rsqrtf(tot / (float)p.H + p.eps);
      }
#pragma unroll
      for (int i = 0; i < VEC_ITERS; ++i) {
        const int c = (i * 256 + threadIdx.x) * 8;
        if (c < p.H) {
          uint4 o;
          __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(&o);
          if (p.w != nullptr) {
            const uint4 ww = *reinterpret_cast<const uint4*>(p.w + c);
            const __nv_bfloat16* wp = reinterpret_cast<const __nv_bfloat16*>(&ww);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float g = __bfloat162float(wp[j]);
              op[j] = __float2bfloat16(v[i][j] * inv * (p.gemma ? 1.f + g : g));
            }
          } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) op[j] = __float2bfloat16(v[i][j]);
          }
          if (p.mode == COMM_ONE_SHOT) {
            *reinterpret_cast<uint4*>(p.x_out[me] + (size_t)t * p.H + c) = o;
          } else {
            for (int r = 0; r < tp; ++r) *reinterpret_cast<uint4*>(p.x_out[(me + r) % tp] + (size_t)t * p.H + c) = o;
          }
        }
      }
    }
  }
  if (p.mode != COMM_TWO_SHOT) return;
  // ---- phase 2 (two-shot): publish "my rows are in your gather buffer", then wait for everybody's rows
  __syncthreads();
  if (threadIdx.x == 0) __threadfence_system();
  __syncthreads();
  if (threadIdx.x < tp) st_flag_release(p.flags[threadIdx.x] + (size_t)((p.phase * 2 + 1) * tp + me) * kMaxCommBlocks + b, seq);
  if (threadIdx.x < tp) {
    if (!wait_flag(p.flags[me] + (size_t)((p.phase * 2 + 1) * tp + threadIdx.x) * kMaxCommBlocks + b, seq, p.wait_ns))
      atomicOr(&g_status, ST_PEER_TIMEOUT);
  }
}


// ---- one-shot reduction without flags (COMM_LAMPORT) -----------------------------------------------------------------
// The data is its own arrival signal: a slot holds bf16 -0.0 (0x8000) until the source's value lands, and sources turn a
// genuine -0.0 into +0.0 before sending. A reader polls each 16-byte vector until none of its eight values is the marker,
// takes it and puts the marker back, so a buffer is clean again the moment it has been read; three buffers rotate (index kept
// in device memory, advanced by the last CTA of each launch) so that a source that is one reduction ahead never meets a
// buffer that is still being read. There is no handshake and no separate flag traffic: the latency of a reduction is one
// NVLink store plus the local poll. Sums run in rank order on every rank, so all ranks obtain bit-identical results.
// (reference: the Lamport one-shot protocol behind FlashInfer's allreduce_fusion, compilation/passes/fusion/allreduce_rms_fusion.py:199;
//  csrc/minimax_reduce_rms_kernel.cu:235)
__device__ __forceinline__ uint4 ld_volatile_v4(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ bool has_marker(uint32_t w) { return (w & 0xffffu) == 0x8000u || (w >> 16) == 0x8000u; }
__device__ __forceinline__ uint32_t strip_marker(uint32_t w) {
  if ((w & 0xffffu) == 0x8000u) w &= 0xffff0000u;
  if ((w >> 16) == 0x8000u) w &= 0x0000ffffu;
  return w;
}

template <int VEC_ITERS>
__global__ void __launch_bounds__(256) tp_lamport_kernel(const CommParams p) {
  __shared__ float red[9];
  __shared__ int s_buf;
  pdl_trigger();
  pdl_wait();
  const int tp = p.tp, me = p.rank;
  if (threadIdx.x == 0) s_buf = *reinterpret_cast<volatile int*>(p.lam_ctr);
  __syncthreads();
  const size_t boff = (size_t)s_buf * (size_t)p.lam_buf_stride;
  const uint4 marker = make_uint4(0x80008000u, 0x80008000u, 0x80008000u, 0x80008000u);
  bool timed_out = false;
  for (int t = blockIdx.x; t < p.T; t += gridDim.x) {
    uint4 mine[VEC_ITERS];
    // ---- send this rank's row to every peer (skipped when the GEMM epilogue already stored it there)
#pragma unroll
    for (int i = 0; i < VEC_ITERS; ++i) {
      const int c = (i * 256 + threadIdx.x) * 8;
      if (c < p.H && !p.lam_pushed) {
        uint4 a = *reinterpret_cast<const uint4*>(p.part[me] + (size_t)t * p.H + c);
        a.x = strip_marker(a.x); a.y = strip_marker(a.y); a.z = strip_marker(a.z); a.w = strip_marker(a.w);
        mine[i] = a;
        const size_t off = boff + (size_t)me * (size_t)p.lam_src_stride + (size_t)t * p.H + c;
        for (int r = 1; r < tp; ++r) *reinterpret_cast<uint4*>(p.lam[(me + r) % tp] + off) = a;
      }
    }
    // ---- gather: poll, take, clean
    float v[VEC_ITERS][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VEC_ITERS; ++i) {
      const int c = (i * 256 + threadIdx.x) * 8;
      if (c < p.H) {
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
        // all sources' vectors are requested at once (one L2 round trip instead of one per source: at eight ranks the serial form
        // spent most of the kernel in 7 x VEC_ITERS dependent loads); a slot that still holds the marker is then polled on its own
        uint4 a[kMaxRanks];
        __nv_bfloat16* const base = p.lam[me] + boff + (size_t)t * p.H + c;
#pragma unroll
        for (int r = 0; r < kMaxRanks; ++r)
          if (r < tp && !(r == me && !p.lam_pushed)) a[r] = ld_volatile_v4(base + (size_t)r * (size_t)p.lam_src_stride);
#pragma unroll
        for (int r = 0; r < kMaxRanks; ++r) {
          if (r >= tp) continue;
          if (r == me && !p.lam_pushed) {
            a[r] = mine[i];
          } else {
            __nv_bfloat16* slot = base + (size_t)r * (size_t)p.lam_src_stride;
            uint64_t t0 = 0;
            uint32_t spins = 0;
            while (has_marker(a[r].x) || has_marker(a[r].y) || has_marker(a[r].z) || has_marker(a[r].w)) {
              if (timed_out) break;
              if ((++spins & 255u) == 0) {
                const uint64_t now = globaltimer_ns();
                if (t0 == 0) t0 = now;
                else if (now - t0 > p.wait_ns) { timed_out = true; break; }
              }
              a[r] = ld_volatile_v4(slot);
            }
            *reinterpret_cast<uint4*>(slot) = marker;
          }
          const __nv_bfloat16* ap = reinterpret_cast<const __nv_bfloat16*>(&a[r]);
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] += __bfloat162float(ap[j]);
        }
        if (p.residual_in != nullptr) {
          const uint4 rr = *reinterpret_cast<const uint4*>(p.residual_in + (size_t)t * p.H + c);
          const __nv_bfloat16* rp = reinterpret_cast<const __nv_bfloat16*>(&rr);
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] += __bfloat162float(rp[j]);
        }
        uint4 o;
        __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(&o);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          op[j] = __float2bfloat16(acc[j]);
          v[i][j] = __bfloat162float(op[j]);
          ss += v[i][j] * v[i][j];
        }
        if (p.residual_out != nullptr) *reinterpret_cast<uint4*>(p.residual_out + (size_t)t * p.H + c) = o;
      }
    }
    float inv = 1.f;
    if (p.w != nullptr) {
      const float tot = block_sum256(ss, red);
      inv = rsqrtf(tot / (float)p.H + p.eps);
    }
#pragma unroll
    for (int i = 0; i < VEC_ITERS; ++i) {
      const int c = (i * 256 + threadIdx.x) * 8;
      if (c < p.H) {
        uint4 o;
        __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(&o);
        if (p.w != nullptr) {
          const uint4 ww = *reinterpret_cast<const uint4*>(p.w + c);
          const __nv_bfloat16* wp = reinterpret_cast<const __nv_bfloat16*>(&ww);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float g = __bfloat162float(wp[j]);
            op[j] = __float2bfloat16(v[i][j] * inv * (p.gemma ? 1.f + g : g));
          }
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) op[j] = __float2bfloat16(v[i][j]);
        }
        *reinterpret_cast<uint4*>(p.x_out[me] + (size_t)t * p.H + c) = o;
      }
    }
  }
  if (timed_out) atomicOr(&g_status, ST_PEER_TIMEOUT);
  // the last CTA to finish moves this rank on to the next buffer (launches on one stream do not overlap)
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(p.lam_ctr + 1, 1) == (int)gridDim.x - 1) {
      p.lam_ctr[1] = 0;
      p.lam_ctr[0] = (s_buf + 1) % kLamportBuffers;
    }
  }
}

}  // namespace

// ---- two-shot reduction through the switch (COMM_NVLS) ---------------------------------------------------------------
// The partial sums and the output live in a symmetric buffer that is also mapped at a multicast address (NVLink SHARP): one
// multimem.ld_reduce at that address returns the sum over all ranks' copies, added inside the switch with fp32 accumulation, and
// one multimem.st writes a value into every rank's copy. A rank therefore reduces only the rows it owns (one round trip to the
// switch instead of tp - 1 peer transfers), adds the residual, normalises and broadcasts the normalised rows. Flags (unicast peer stores, bounded polls) order the phases: nobody reads before
// every rank's partial is complete, nobody leaves before every rank's rows have been broadcast. The switch returns each sum to
// exactly one rank, which broadcasts what it derived from it, so all ranks hold bit-identical outputs.
// The new residual rows are broadcast as well, so every rank ends with the whole residual, as after the one-shot kernels.
//   p.part[0]  multicast address of the partial sums [T, H];  p.x_out[0]  multicast address of the output [T, H];
//   p.x_out[1] multicast address of the residual output [T, H] (or null)
// (reference: distributed/device_communicators/symm_mem.py:149-153 multimem all-reduce; NCCL's NVLS algorithms)
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st_v4(void* mc, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// Polls with relaxed loads: what the flag guards is read through the switch (phase 0) or by later kernels (phase 2), never through
// this SM's L1 in this kernel, so the poll itself needs no acquire.
__device__ __forceinline__ bool wait_flag_relaxed(const int* p, int want, uint64_t limit_ns) {
  uint64_t t0 = 0;
  uint32_t spins = 0;
  while (true) {
    int v;
    asm volatile("ld.relaxed.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    if (v - want >= 0) return true;
    if ((++spins & 255u) == 0) {
      const uint64_t now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > limit_ns) return false;
    }
  }
}

template <int VEC_ITERS>
__global__ void __launch_bounds__(256) tp_nvls_kernel(const CommParams p) {
  __shared__ float red[9];
  __shared__ int s_seq, s_ok;
  const int b = blockIdx.x;
  const int tp = p.tp, me = p.rank;
  pdl_trigger();
  pdl_wait();
  // ---- phase 0: this rank's partial sums are complete (the producing GEMM ran earlier on this stream); wait for everybody's
  if (threadIdx.x == 0) {
    int seq = p.seq_local[b] + 1;
    p.seq_local[b] = seq;
    s_seq = seq;
    s_ok = 1;   // no fence: the partial sums were written by the previous kernel, which has completed (pdl_wait above)
  }
  __syncthreads();
  const int seq = s_seq;
  if (threadIdx.x < tp) st_flag_release(p.flags[threadIdx.x] + (size_t)(p.phase * 2 * tp + me) * kMaxCommBlocks + b, seq);
  if (threadIdx.x < tp) {
    if (!wait_flag_relaxed(p.flags[me] + (size_t)(p.phase * 2 * tp + threadIdx.x) * kMaxCommBlocks + b, seq, p.wait_ns)) {
      s_ok = 0;
      atomicOr(&g_status, ST_PEER_TIMEOUT);
    }
  }
  __syncthreads();
  const bool ok = s_ok != 0;
  const int per = (p.T + tp - 1) / tp;
  const int row_lo = min(me * per, p.T), row_hi = min(row_lo + per, p.T);
  if (ok) {
    for (int t = row_lo + b; t < row_hi; t += gridDim.x) {
      float v[VEC_ITERS][8];
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < VEC_ITERS; ++i) {
        const int c = (i * 256 + threadIdx.x) * 8;
        if (c < p.H) {
          const uint4 a = multimem_ld_reduce_bf16x8(p.part[0] + (size_t)t * p.H + c);
          const __nv_bfloat16* ap = reinterpret_cast<const __nv_bfloat16*>(&a);
          float acc[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] = __bfloat162float(ap[j]);
          if (p.residual_in != nullptr) {
            const uint4 rr = *reinterpret_cast<const uint4*>(p.residual_in + (size_t)t * p.H + c);
            const __nv_bfloat16* rp = reinterpret_cast<const __nv_bfloat16*>(&rr);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] += __bfloat162float(rp[j]);
          }
          uint4 o;
          __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(&o);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            op[j] = __float2bfloat16(acc[j]);
            v[i][j] = __bfloat162float(op[j]);
            ss += v[i][j] * v[i][j];
          }
          if (p.x_out[1] != nullptr) multimem_st_v4(p.x_out[1] + (size_t)t * p.H + c, o);
        }
      }
      float inv = 1.f;
      if (p.w != nullptr) {
        const float tot = block_sum256(ss, red);
        inv = rsqrtf(tot / (float)p.H + p.eps);
      }
#pragma unroll
      for (int i = 0; i < VEC_ITERS; ++i) {
        const int c = (i * 256 + threadIdx.x) * 8;
        if (c < p.H) {
          uint4 o;
          __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(&o);
          if (p.w != nullptr) {
            const uint4 ww = *reinterpret_cast<const uint4*>(p.w + c);
            const __nv_bfloat16* wp = reinterpret_cast<const __nv_bfloat16*>(&ww);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float g = __bfloat162float(wp[j]);
              op[j] = __float2bfloat16(v[i][j] * inv * (p.gemma ? 1.f + g : g));
            }
          } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) op[j] = __float2bfloat16(v[i][j]);
          }
          multimem_st_v4(p.x_out[0] + (size_t)t * p.H + c, o);
        }
      }
    }
  }
  // ---- phase 2: "my rows are in your output buffer", then wait for everybody's rows
  __syncthreads();
  if (threadIdx.x == 0) __threadfence_system();
  __syncthreads();
  if (threadIdx.x < tp) st_flag_release(p.flags[threadIdx.x] + (size_t)((p.phase * 2 + 1) * tp + me) * kMaxCommBlocks + b, seq);
  if (threadIdx.x < tp) {
    if (!wait_flag_relaxed(p.flags[me] + (size_t)((p.phase * 2 + 1) * tp + threadIdx.x) * kMaxCommBlocks + b, seq, p.wait_ns))
      atomicOr(&g_status, ST_PEER_TIMEOUT);
  }
}

int tp_reduce_norm_launch(const CommParams& p, int grid, cudaStream_t st) {
  if (p.H % 8 || p.H > 8192 || grid < 1 || grid > kMaxCommBlocks || p.tp > kMaxRanks) return -1;
  if (p.T == 0) return 0;
  const int iters = (p.H + 2047) / 2048;
  if (p.mode == COMM_LAMPORT) {
    if (p.lam_ctr == nullptr || p.lam_buf_stride <= 0 || (size_t)p.T * p.H > (size_t)p.lam_src_stride) return -3;
    switch (iters) {
      case 1: launch_k(tp_lamport_kernel<1>, dim3(grid), dim3(256), 0, st, true, p); break;
      case 2: launch_k(tp_lamport_kernel<2>, dim3(grid), dim3(256), 0, st, true, p); break;
      case 3: launch_k(tp_lamport_kernel<3>, dim3(grid), dim3(256), 0, st, true, p); break;
      default: launch_k(tp_lamport_kernel<4>, dim3(grid), dim3(256), 0, st, true, p); break;
    }
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
  }
  if (p.mode == COMM_NVLS) {
    if (p.part[0] == nullptr || p.x_out[0] == nullptr) return -4;
    switch (iters) {
      case 1: launch_k(tp_nvls_kernel<1>, dim3(grid), dim3(256), 0, st, true, p); break;
      case 2: launch_k(tp_nvls_kernel<2>, dim3(grid), dim3(256), 0, st, true, p); break;
      case 3: launch_k(tp_nvls_kernel<3>, dim3(grid), dim3(256), 0, st, true, p); break;
      default: launch_k(tp_nvls_kernel<4>, dim3(grid), dim3(256), 0, st, true, p); break;
    }
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
  }
  switch (iters) {
    case 1: tp_reduce_norm_kernel<1><<<grid, 256, 0, st>>>(p); break;
    case 2: tp_reduce_norm_kernel<2><<<grid, 256, 0, st>>>(p); break;
    case 3: tp_reduce_norm_kernel<3><<<grid, 256, 0, st>>>(p); break;
    default: tp_reduce_norm_kernel<4><<<grid, 256, 0, st>>>(p); break;
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// ---- slab management (host) ------------------------------------------------------------------------------------
int comm_alloc(size_t bytes, void** ptr) {
  if (cudaMalloc(ptr, bytes) != cudaSuccess) return -1;
  return cudaMemset(*ptr, 0, bytes) == cudaSuccess ? 0 : -2;
}
int comm_free(void* ptr) { return cudaFree(ptr) == cudaSuccess ? 0 : -1; }
int comm_export(void* ptr, void* handle_out64) {
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, ptr) != cudaSuccess) return -1;
  static_assert(sizeof(h) == 64, "unexpected IPC handle size");
  memcpy(handle_out64, &h, 64);
  return 0;
}
int comm_import(const void* handle64, void** ptr) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  return cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess) == cudaSuccess ? 0 : -1;
}
int comm_unimport(void* ptr) { return cudaIpcCloseMemHandle(ptr) == cudaSuccess ? 0 : -1; }

unsigned int comm_read_status(bool clear) { return read_status_tu(clear); }
void comm_read_status_async(unsigned int* dst, cudaStream_t st) { read_status_tu_async(dst, st); }

}  // namespace oc
