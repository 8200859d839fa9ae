// Mixture-of-experts plumbing around the grouped tcgen05 GEMM: count tokens per local expert, lay the (token, expert) pairs out
// expert-major ("slots"), build the GEMM work lists on the device, gather activations into slot order, and combine the expert
// outputs back per token with the routing weights. Nothing here needs the host to know how tokens were routed, so a whole MoE
// layer is a fixed sequence of launches (CUDA-graph friendly).
//   count -> plan (1 CTA: prefix sum + work lists for both GEMMs) -> scatter (slot assignment + gather of X rows)
//   -> grouped GEMM w13 with SiLU*mul epilogue -> grouped GEMM w2 -> combine (weighted sum over each token's experts)
// With expert parallelism a rank owns experts [e_off, e_off + E_local); pairs routed elsewhere get slot -1 and contribute nothing,
// so the layer output is a partial sum that the tensor-parallel reduction completes.
// (reference: csrc/moe/moe_align_sum_kernels.cu:22-456, moe_permute_unpermute_op.cu:240; layers/fused_moe/modular_kernel.py:1236-1461)
#include "common.cuh"
#include "kernels.h"

namespace oc {
namespace {

__global__ void moe_count_kernel(const int* __restrict__ ids, int n_pairs, int e_off, int E, int* __restrict__ counts) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_pairs) return;
  const int e = ids[i] - e_off;
  if (e >= 0 && e < E) atomicAdd(&counts[e], 1);
}

// One CTA. offsets[e] = first slot of expert e; work lists for GEMM 1 (n1 row tiles per expert) and GEMM 2 (n2 row tiles).
__global__ void __launch_bounds__(1024) moe_plan_kernel(MoePlanParams p) {
  __shared__ int s_off[1025];
  const int E = p.E;
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < E; ++e) { s_off[e] = acc; acc += p.counts[e]; }
    s_off[E] = acc;
    p.total_slots[0] = acc;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= E; e += blockDim.x) p.offsets[e] = s_off[e];
  for (int e = threadIdx.x; e < E; e += blockDim.x) p.cursor[e] = 0;
  // item base per expert for both lists (sequential scan by thread 0; E <= 1024)
  __shared__ int s_tiles[1025];
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < E; ++e) { s_tiles[e] = acc; acc += (p.counts[e] + p.tn - 1) / p.tn; }
    s_tiles[E] = acc;
    p.work_count[0] = acc * p.n1;
    p.work_count[1] = acc * p.n2;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    const int cnt = p.counts[e], tt0 = s_tiles[e], ntt = s_tiles[e + 1] - tt0;
    for (int tt = 0; tt < ntt; ++tt) {
      const int t0 = s_off[e] + tt * p.tn, rows = min(p.tn, cnt - tt * p.tn);
      for (int n = 0; n < p.n1; ++n) p.work1[(size_t)(tt0 + tt) * p.n1 + n] = make_int4(e * p.n1 + n, t0, rows, n * 128);
      for (int n = 0; n < p.n2; ++n) p.work2[(size_t)(tt0 + tt) * p.n2 + n] = make_int4(e * p.n2 + n, t0, rows, n * 128);
    }
  }
}

// One warp per (token, j) pair: claim a slot in the pair's expert, remember it, copy the token's activation row there.
__global__ void moe_scatter_kernel(const int* __restrict__ ids, int n_pairs, int k, int e_off, int E, const int* __restrict__ offsets,
                                   int* __restrict__ cursor, int* __restrict__ slot_of, const __nv_bfloat16* __restrict__ x, long long ldx,
                                   __nv_bfloat16* __restrict__ xs, int H) {
  const int pair = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (pair >= n_pairs) return;
  const int lane = threadIdx.x & 31;
  const int e = ids[pair] - e_off;
  int slot = -1;
  if (e >= 0 && e < E) {
    if (lane == 0) slot = offsets[e] + atomicAdd(&cursor[e], 1);
    slot = __shfl_sync(0xffffffffu, slot, 0);
  }
  if (lane == 0) slot_of[pair] = slot;
  if (slot < 0) return;
  const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)(pair / k) * ldx);
  uint4* dst = reinterpret_cast<uint4*>(xs + (size_t)slot * H);
  for (int i = lane; i < H / 8; i += 32) dst[i] = src[i];
}

// y[t] = sum_j w[t, j] * a2[slot_of[t, j]]   (fixed j order: bit-stable), 8 columns per thread
__global__ void moe_combine_kernel(const __nv_bfloat16* __restrict__ a2, const int* __restrict__ slot_of, const float* __restrict__ w,
                                   __nv_bfloat16* __restrict__ y, int T, int k, int H) {
  const int t = blockIdx.y;
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (c >= H) return;
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  for (int j = 0; j < k; ++j) {
    const int slot = slot_of[t * k + j];
    if (slot < 0) continue;
    const float wj = w[t * k + j];
    const uint4 v = *reinterpret_cast<const uint4*>(a2 + (size_t)slot * H + c);
    const __nv_bfloat16* vp = reinterpret_cast<const __nv_bfloat16*>(&v);
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] += wj * __bfloat162float(vp[i]);
  }
  uint4 o;
  __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(&o);
#pragma unroll
  for (int i = 0; i < 8; ++i) op[i] = __float2bfloat16(acc[i]);
  *reinterpret_cast<uint4*>(y + (size_t)t * H + c) = o;
}

}  // namespace

int moe_prepare_launch(const MoePlanParams& p, const int* ids, int n_pairs, int k, int e_off, int* slot_of, const void* x, long long ldx,
                       void* xs, int H, cudaStream_t st) {
  if (p.E > 1024 || H % 8) return -1;
  if (cudaMemsetAsync(p.counts, 0, sizeof(int) * p.E, st) != cudaSuccess) return -2;
  if (n_pairs > 0) moe_count_kernel<<<(n_pairs + 255) / 256, 256, 0, st>>>(ids, n_pairs, e_off, p.E, p.counts);
  moe_plan_kernel<<<1, 1024, 0, st>>>(p);
  if (n_pairs > 0)
    moe_scatter_kernel<<<(n_pairs + 7) / 8, 256, 0, st>>>(ids, n_pairs, k, e_off, p.E, p.offsets, p.cursor, slot_of, (const __nv_bfloat16*)x, ldx,
                                                           (__nv_bfloat16*)xs, H);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// Work lists only, from counts that are already on the device (expert-parallel exchange: the rows arrive in slot order).
int moe_plan_launch(const MoePlanParams& p, cudaStream_t st) {
  if (p.E > 1024) return -1;
  moe_plan_kernel<<<1, 1024, 0, st>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

int moe_combine_launch(const void* a2, const int* slot_of, const float* w, void* y, int T, int k, int H, cudaStream_t st) {
  if (T == 0) return 0;
  if (H % 8) return -1;
  dim3 grid((H / 8 + 127) / 128, T);
  moe_combine_kernel<<<grid, 128, 0, st>>>((const __nv_bfloat16*)a2, slot_of, w, (__nv_bfloat16*)y, T, k, H);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

unsigned int moe_read_status(bool clear) { return read_status_tu(clear); }
void moe_read_status_async(unsigned int* dst, cudaStream_t st) { read_status_tu_async(dst, st); }

}  // namespace oc
