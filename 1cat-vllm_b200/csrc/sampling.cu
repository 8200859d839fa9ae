// Speculative-decoding verifier (rejection sampler) and MoE routing kernels.
//
// Verification runs in two launches. `verify_rows_kernel` makes one pass over the vocabulary for every (request, draft
// position): running max and sum of exp (the softmax normaliser at the request's temperature), the target probability of the
// draft token, the arg-max of the row, and the "recovered" token arg-max_{v != draft}(logit_v / T + Gumbel noise_v), which is a
// sample from the residual distribution max(p - q, 0) when the draft is a point mass (no draft probabilities), using a counter
// based generator so that results depend only on (seed, step, row, v). `accept_kernel` then walks each request's drafts in order:
// greedy rows accept while draft == arg-max; random rows accept iff p_target(draft) >= u; in synthetic mode acceptance is
// u < rate[pos]. The first rejection emits the recovered token (arg-max for greedy rows); full acceptance appends the bonus token.
// (reference: vllm/v1/sample/rejection_sampler.py:896-1026 and Triton kernels :1292,1346,1438; csrc/cpu/spec_decode_utils.cpp:211-409)
//
// Routing: softmax top-k with renormalisation (Qwen MoE) and sigmoid scoring with bias-corrected grouped top-k (DeepSeek-V3), one warp
// per token (reference: csrc/moe/topk_softmax_kernels.cu:75-269, grouped_topk_kernels.cu:516,675).
#include "common.cuh"
#include "kernels.h"

namespace oc {
namespace {

__device__ __forceinline__ uint32_t hash32(uint32_t x) {
  x ^= x >> 16; x *= 0x7feb352du; x ^= x >> 15; x *= 0x846ca68bu; x ^= x >> 16;
  return x;
}
__device__ __forceinline__ float uniform01(uint64_t seed, uint32_t row, uint32_t v) {
  uint32_t h = hash32((uint32_t)seed ^ hash32(row * 0x9e3779b9u + (uint32_t)(seed >> 32)) ^ hash32(v + 0x85ebca6bu));
  return ((h >> 8) + 0.5f) * (1.0f / 16777216.0f);
}

template <typename T>
__global__ void __launch_bounds__(512) verify_rows_kernel(const T* __restrict__ logits, const long long* __restrict__ draft_ids,
                                                          const float* __restrict__ temperature, RowStats* __restrict__ stats, int k, int V,
                                                          long long ld_b, long long ld_pos, uint64_t seed, int use_noise) {
  const int row = blockIdx.x;  // b * k + pos
  const int b = row / k, pos = row % k;
  const T* x = logits + (size_t)b * ld_b + (size_t)pos * ld_pos;
  const int d = (int)draft_ids[row];
  float temp = temperature != nullptr ? temperature[b] : 0.f;
  const bool greedy = temp < 1e-5f;
  const float inv_t = greedy ? 1.f : 1.f / temp;
  float m = -INFINITY, s = 0.f, best_all = -INFINITY, best_ex = -INFINITY;
  int arg_all = 0x7fffffff, arg_ex = 0x7fffffff;
  for (int v = threadIdx.x; v < V; v += blockDim.x) {
    const float raw = (float)x[v];
    const float z = raw * inv_t;
    if (z > m) { s = s * __expf(m - z) + 1.f; m = z; } else { s += __expf(z - m); }
    if (raw > best_all || (raw == best_all && v < arg_all)) { best_all = raw; arg_all = v; }
    if (v != d) {
      float sc = z;
      if (use_noise && !greedy) { const float u = uniform01(seed, (uint32_t)row, (uint32_t)v); sc = z - __logf(-__logf(u)); }
      if (sc > best_ex || (sc == best_ex && v < arg_ex)) { best_ex = sc; arg_ex = v; }
    }
  }
  __shared__ float sm[16], ss[16], sa[16], se[16];
  __shared__ int ia[16], ie[16];
  // warp-level merge, then across warps
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float om = __shfl_xor_sync(0xffffffffu, m, o), os = __shfl_xor_sync(0xffffffffu, s, o);
    const float nm = fmaxf(m, om);
    s = (m == -INFINITY ? 0.f : s * __expf(m - nm)) + (om == -INFINITY ? 0.f : os * __expf(om - nm));
    m = nm;
    const float oa = __shfl_xor_sync(0xffffffffu, best_all, o); const int oia = __shfl_xor_sync(0xffffffffu, arg_all, o);
    if (oa > best_all || (oa == best_all && oia < arg_all)) { best_all = oa; arg_all = oia; }
    const float oe = __shfl_xor_sync(0xffffffffu, best_ex, o); const int oie = __shfl_xor_sync(0xffffffffu, arg_ex, o);
    if (oe > best_ex || (oe == best_ex && oie < arg_ex)) { best_ex = oe; arg_ex = oie; }
  }
  const int w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  if ((threadIdx.x & 31) == 0) { sm[w] = m; ss[w] = s; sa[w] = best_all; ia[w] = arg_all; se[w] = best_ex; ie[w] = arg_ex; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < nw; ++i) {
      const float nm = fmaxf(m, sm[i]);
      s = (m == -INFINITY ? 0.f : s * __expf(m - nm)) + (sm[i] == -INFINITY ? 0.f : ss[i] * __expf(sm[i] - nm));
      m = nm;
      if (sa[i] > best_all || (sa[i] == best_all && ia[i] < arg_all)) { best_all = sa[i]; arg_all = ia[i]; }
      if (se[i] > best_ex || (se[i] == best_ex && ie[i] < arg_ex)) { best_ex = se[i]; arg_ex = ie[i]; }
    }
    RowStats r;
    const float zd = (d >= 0 && d < V) ? (float)x[d] * inv_t : -INFINITY;
    r.p_draft = greedy ? 0.f : __expf(zd - m) / s;
    r.arg_all = arg_all;
    r.arg_ex = arg_ex == 0x7fffffff ? arg_all : arg_ex;
    stats[row] = r;
  }
}

__global__ void accept_kernel(const RowStats* __restrict__ stats, const long long* __restrict__ draft_ids, const long long* __restrict__ num_draft,
                              const long long* __restrict__ bonus, const double* __restrict__ uniforms, const float* __restrict__ temperature,
                              const float* __restrict__ synth_rates, long long* __restrict__ out, int B, int k) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  const int n = (int)num_draft[b];
  const bool greedy = temperature == nullptr || temperature[b] < 1e-5f;
  long long* o = out + (size_t)b * (k + 1);
  for (int i = 0; i <= k; ++i) o[i] = -1;
  for (int i = 0; i < n; ++i) {
    const RowStats r = stats[b * k + i];
    const long long d = draft_ids[b * k + i];
    bool accept;
    if (synth_rates != nullptr) accept = uniforms[b * k + i] < (double)synth_rates[i];
    else if (greedy) accept = d == r.arg_all;
    else accept = (double)r.p_draft >= uniforms[b * k + i];  // the draft is a point mass: q(d) = 1
    if (accept) { o[i] = d; continue; }
    o[i] = (greedy && synth_rates == nullptr) ? r.arg_all : r.arg_ex;
    return;
  }
  o[n] = bonus[b];
}

// ---- routing: one warp per token, E <= 512 experts (E / 32 scores per lane)
__global__ void route_kernel(const RouteParams p) {
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= p.T) return;
  const int lane = threadIdx.x & 31;
  const int per = p.E / 32;  // host guarantees E % 32 == 0 and per <= 16
  float sc[16], sel[16];
  const __nv_bfloat16* x = p.logits + (size_t)t * p.ld;
  float mx = -INFINITY;
  for (int i = 0; i < per; ++i) { sc[i] = __bfloat162float(x[lane * per + i]); mx = fmaxf(mx, sc[i]); }
  if (p.sigmoid) {
    for (int i = 0; i < per; ++i) sc[i] = 1.f / (1.f + __expf(-sc[i]));
  } else {
    mx = warp_max(mx);
    float sum = 0.f;
    for (int i = 0; i < per; ++i) { sc[i] = __expf(sc[i] - mx); sum += sc[i]; }
    sum = warp_sum(sum);
    for (int i = 0; i < per; ++i) sc[i] /= sum;
  }
  for (int i = 0; i < per; ++i) sel[i] = sc[i] + (p.bias != nullptr ? p.bias[lane * per + i] : 0.f);
  if (p.n_group > 1) {
    // group score = sum of the two best biased scores in the group (max without bias); keep the topk_group best groups
    const int gsz = p.E / p.n_group;            // experts per group; a group spans gsz / per lanes
    const int lanes_per_group = gsz / per;      // host guarantees gsz % per == 0 and lanes_per_group is a power of two <= 32
    float b1 = -INFINITY, b2 = -INFINITY;
    for (int i = 0; i < per; ++i) { if (sel[i] > b1) { b2 = b1; b1 = sel[i]; } else if (sel[i] > b2) b2 = sel[i]; }
    for (int o = 1; o < lanes_per_group; o <<= 1) {
      const float o1 = __shfl_xor_sync(0xffffffffu, b1, o), o2 = __shfl_xor_sync(0xffffffffu, b2, o);
      const float n1 = fmaxf(b1, o1);
      const float n2 = fmaxf(fminf(b1, o1), fmaxf(b2, o2));
      b1 = n1; b2 = n2;
    }
    const float gscore = p.bias != nullptr ? b1 + b2 : b1;
    const int my_group = lane / lanes_per_group;
    int rank = 0;  // how many groups beat mine (ties: lower index wins)
    for (int g = 0; g < p.n_group; ++g) {
      const float og = __shfl_sync(0xffffffffu, gscore, g * lanes_per_group);
      if (og > gscore || (og == gscore && g < my_group)) ++rank;
    }
    if (rank >= p.topk_group)
      for (int i = 0; i < per; ++i) sel[i] = -INFINITY;
  }
  float wsum = 0.f;
  float wk[16];
  int ik[16];
  for (int kk = 0; kk < p.k; ++kk) {
    float bv = -INFINITY; int bi = 0x7fffffff; float bw = 0.f;
    for (int i = 0; i < per; ++i)
      if (sel[i] > bv) { bv = sel[i]; bi = lane * per + i; bw = sc[i]; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o); const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      const float ow = __shfl_xor_sync(0xffffffffu, bw, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; bw = ow; }
    }
    if (bi / per == lane) sel[bi % per] = -INFINITY;
    wk[kk] = bw; ik[kk] = bi; wsum += bw;
  }
  if (lane == 0) {
    const float norm = p.renormalize ? 1.f / (wsum + 1e-20f) : 1.f;
    for (int kk = 0; kk < p.k; ++kk) {
      p.topk_w[(size_t)t * p.k + kk] = wk[kk] * norm * p.scaling;
      p.topk_ids[(size_t)t * p.k + kk] = ik[kk];
    }
  }
}

}  // namespace

int rejection_launch(const void* logits, int is_fp32, const long long* draft_ids, const long long* num_draft, const long long* bonus,
                     const double* uniforms, const float* temperature, const float* synth_rates, RowStats* stats, long long* out, int B, int k, int V,
                     long long ld_b, long long ld_pos, unsigned long long seed, int use_noise, cudaStream_t st) {
  if (B == 0) return 0;
  if (k > 0) {
    if (is_fp32) verify_rows_kernel<float><<<B * k, 512, 0, st>>>((const float*)logits, draft_ids, temperature, stats, k, V, ld_b, ld_pos, seed, use_noise);
    else verify_rows_kernel<__nv_bfloat16><<<B * k, 512, 0, st>>>((const __nv_bfloat16*)logits, draft_ids, temperature, stats, k, V, ld_b, ld_pos, seed, use_noise);
  }
  accept_kernel<<<(B + 127) / 128, 128, 0, st>>>(stats, draft_ids, num_draft, bonus, uniforms, temperature, synth_rates, out, B, k);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int route_launch(const RouteParams& p, cudaStream_t st) {
  if (p.T == 0) return 0;
  if (p.E % 32 || p.E / 32 > 16 || p.k > 16 || p.k > p.E) return -1;
  if (p.n_group > 1) {
    const int per = p.E / 32, gsz = p.E / p.n_group;
    if (p.E % p.n_group || gsz % per) return -1;
    const int lpg = gsz / per;
    if (lpg < 1 || (lpg & (lpg - 1)) || lpg > 32) return -1;
  }
  route_kernel<<<(p.T + 7) / 8, 256, 0, st>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

unsigned int sampling_read_status(bool clear) { return read_status_tu(clear); }
void sampling_read_status_async(unsigned int* dst, cudaStream_t st) { read_status_tu_async(dst, st); }

}  // namespace oc
