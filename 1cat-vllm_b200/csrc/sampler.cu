// Token sampler: temperature, min-p, top-k, top-p and the random draw for one row of logits per CTA, without sorting
// (reference: v1/sample/sampler.py:87-366; v1/sample/ops/topk_topp_sampler.py:22-438; csrc/sampler.cu, csrc/topk.cu).
//
// Every filter keeps an upper set of the row ("all logits >= some threshold"), so the kernel only has to find thresholds:
//   min-p : scaled logit >= max + log(min_p)
//   top-k : the k-th largest value, by a 4-pass radix select over the order-preserving 32-bit key of the scaled logit
//           (256-bin count histogram per pass)
//   top-p : the value at which the probability mass of the larger tokens first reaches p, by the same radix descent over
//           histograms of exp(logit - max) restricted to what min-p and top-k kept
// The draw is the Gumbel / exponential race over the kept tokens: argmax(logit/T - log(E_i)), E_i ~ Exp(1) from a counter-based
// generator keyed by (seed, token index), which is the distribution of softmax sampling. Rows with temperature ~ 0 take the arg-max.
// The row is read once per pass (max, 4 + 4 select passes at most, draw); it stays in L2 between passes.
#include "common.cuh"
#include "kernels.h"

namespace oc {
namespace {

constexpr int kThreads = 1024;
constexpr int kWarps = kThreads / 32;

__device__ __forceinline__ uint32_t order_key(float x) {
  uint32_t u = __float_as_uint(x);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ float uniform01(unsigned long long seed, unsigned long long idx) {
  // splitmix64 finaliser over (seed, idx): one independent 24-bit uniform per token
  unsigned long long z = seed + 0x9e3779b97f4a7c15ull * (idx + 1);
  z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
  z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
  z ^= z >> 31;
  return ((float)(z >> 40) + 0.5f) * (1.0f / 16777216.0f);
}

__device__ __forceinline__ float load_scaled(const float* row, int i, float inv_t) { return row[i] * inv_t; }
__device__ __forceinline__ float load_scaled(const __nv_bfloat16* row, int i, float inv_t) { return __bfloat162float(row[i]) * inv_t; }

// Visits every element of the row once: four independent loads are issued before any of them is used, so the L2 latency of one
// pass is paid once per four elements (the passes are latency-bound: long-scoreboard stalls dominated the first version).
template <typename T, typename F>
__device__ __forceinline__ void for_each_scaled(const T* row, int V, float inv_t, F&& f) {
  constexpr int U = 4;
  int i = threadIdx.x;
  for (; i + (U - 1) * kThreads < V; i += U * kThreads) {
    float x[U];
#pragma unroll
    for (int j = 0; j < U; ++j) x[j] = load_scaled(row, i + j * kThreads, inv_t);
#pragma unroll
    for (int j = 0; j < U; ++j) f(i + j * kThreads, x[j]);
  }
  for (; i < V; i += kThreads) f(i, load_scaled(row, i, inv_t));
}

__device__ float block_max(float v, float* sh) {
  v = warp_max(v);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = sh[0];
  for (int i = 1; i < kWarps; ++i) r = fmaxf(r, sh[i]);
  __syncthreads();
  return r;
}
__device__ float block_sum(float v, float* sh) {
  v = warp_sum(v);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = 0.f;
  for (int i = 0; i < kWarps; ++i) r += sh[i];  // fixed order: the same value in every thread
  __syncthreads();
  return r;
}

// Radix descent for the threshold key. Elements are the row's keys >= floor_key. With MASS = false an element weighs 1 and the
// result is the key of the element with fewer than `target` elements above it and at least `target` counting itself (the k-th
// largest). With MASS = true an element weighs exp(x - m) and the result is the key at which the mass of the strictly larger
// elements is still below `target` while including the key's own elements reaches it.
template <typename T, bool MASS>
__device__ uint32_t radix_threshold(const T* row, int V, float inv_t, float m, uint32_t floor_key, float target, float* hist /*[kWarps][256]*/,
                                    float* tot /*[256]*/, uint32_t* s_sel, float* s_above) {
  const int warp = threadIdx.x >> 5;
  uint32_t prefix = 0;   // the selected high bytes so far
  float above = 0.f;     // weight strictly above the current prefix range
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    for (int i = threadIdx.x; i < kWarps * 256; i += kThreads) hist[i] = 0.f;
    __syncthreads();
    for_each_scaled(row, V, inv_t, [&](int, float x) {
      const uint32_t k = order_key(x);
      if (k < floor_key) return;
      if (pass > 0 && (k >> (shift + 8)) != (prefix >> (shift + 8))) return;
      atomicAdd(&hist[warp * 256 + ((k >> shift) & 255u)], MASS ? __expf(x - m) : 1.f);
    });
    __syncthreads();
    if (threadIdx.x < 256) {
      float s = 0.f;
      for (int w = 0; w < kWarps; ++w) s += hist[w * 256 + threadIdx.x];
      tot[threadIdx.x] = s;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      float acc = above;
      int sel = -1, lowest = 0;
      for (int b = 255; b >= 0; --b) {
        const float w = tot[b];
        if (w <= 0.f) continue;
        lowest = b;
        if (acc + w >= target) { sel = b; break; }
        acc += w;
      }
      if (sel < 0) {  // rounding left the target just above the total: everything is kept
        sel = lowest;
        acc -= tot[lowest];
      }
      *s_sel = (uint32_t)sel;
      *s_above = acc;
    }
    __syncthreads();
    prefix |= (*s_sel) << shift;
    above = *s_above;
    __syncthreads();
  }
  return prefix;
}

template <typename T>
__global__ void __launch_bounds__(kThreads) sample_kernel(const SampleParams p) {
  extern __shared__ float dyn[];
  float* hist = dyn;                       // [kWarps][256]
  float* tot = hist + kWarps * 256;        // [256]
  __shared__ float red[kWarps];
  __shared__ int redi[kWarps];
  __shared__ uint32_t s_sel;
  __shared__ float s_above;
  const int row_i = blockIdx.x;
  const T* row = reinterpret_cast<const T*>(p.logits) + (size_t)row_i * p.ld;
  const int V = p.V;
  const float temp = p.temperature[row_i];
  const bool greedy = temp < 1e-5f;
  const float inv_t = greedy ? 1.f : 1.f / temp;

  float mx = -INFINITY;
  for_each_scaled(row, V, inv_t, [&](int, float x) { mx = fmaxf(mx, x); });
  const float m = block_max(mx, red);

  uint32_t floor_key = 0;
  if (!greedy) {
    const float min_p = p.min_p != nullptr ? p.min_p[row_i] : 0.f;
    if (min_p > 0.f) floor_key = max(floor_key, order_key(m + __logf(min_p)));
    const int top_k = p.top_k != nullptr ? p.top_k[row_i] : 0;
    if (top_k > 0 && top_k < V)
      floor_key = max(floor_key, radix_threshold<T, false>(row, V, inv_t, m, 0u, (float)top_k, hist, tot, &s_sel, &s_above));
    const float top_p = p.top_p != nullptr ? p.top_p[row_i] : 1.f;
    if (top_p < 1.f) {
      float s = 0.f;
      for_each_scaled(row, V, inv_t, [&](int, float x) {
        if (order_key(x) >= floor_key) s += __expf(x - m);
      });
      const float total = block_sum(s, red);
      floor_key = max(floor_key, radix_threshold<T, true>(row, V, inv_t, m, floor_key, top_p * total, hist, tot, &s_sel, &s_above));
    }
  }
  if (p.kept != nullptr) {  // test hook: which tokens survived the filters
    for (int i = threadIdx.x; i < V; i += kThreads)
      p.kept[(size_t)row_i * V + i] = order_key(load_scaled(row, i, inv_t)) >= floor_key ? 1 : 0;
  }

  // the draw (or the arg-max): best score, lowest index on ties
  const unsigned long long seed = p.seeds[row_i];
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for_each_scaled(row, V, inv_t, [&](int i, float x) {
    if (order_key(x) < floor_key) return;
    float sc = x;
    if (!greedy) sc = x - m - __logf(-__logf(uniform01(seed, (unsigned long long)i)));
    if (sc > best || (sc == best && i < bi)) { best = sc; bi = i; }
  });
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  if ((threadIdx.x & 31) == 0) { red[threadIdx.x >> 5] = best; redi[threadIdx.x >> 5] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < kWarps; ++w)
      if (red[w] > best || (red[w] == best && redi[w] < bi)) { best = red[w]; bi = redi[w]; }
    p.out[row_i] = bi == 0x7fffffff ? 0 : bi;
  }
}

}  // namespace

int sample_launch(const SampleParams& p, cudaStream_t st) {
  if (p.B == 0) return 0;
  if (p.V <= 0) return -1;
  const int smem = (kWarps * 256 + 256) * (int)sizeof(float);
  if (p.is_fp32) sample_kernel<float><<<p.B, kThreads, smem, st>>>(p);
  else sample_kernel<__nv_bfloat16><<<p.B, kThreads, smem, st>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

}  // namespace oc
