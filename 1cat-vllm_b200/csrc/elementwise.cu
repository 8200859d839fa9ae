// Memory-bound helper kernels: fused residual-add + RMSNorm, gated RMSNorm, SiLU*mul, per-head norm + RoPE + paged
// KV insert, arg-max over the vocabulary. One pass over the data each, 16-byte accesses.
// (reference: csrc/libtorch_stable/layernorm_kernels.cu:21,99; pos_encoding_kernels.cu:77; fused_qknorm_rope_kernel.cu:104;
//  cache_kernels.cu reshape_and_cache_flash; activation_kernels.cu:78)
#include <cuda_fp8.h>

#include "common.cuh"
#include "kernels.h"

namespace oc {
namespace {

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (threadIdx.x < nw) ? red[threadIdx.x] : 0.f;
  if (warp == 0) {
    t = warp_sum(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}

// y = norm(x (+ residual)) * w ; residual_out = bf16(x + residual).  One CTA per token, values stay in registers.
template <int VEC_ITERS>
__global__ void __launch_bounds__(256) rms_norm_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res_in,
                                                       const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                                                       __nv_bfloat16* __restrict__ res_out, int H, int ldx, float eps, int gemma) {
  __shared__ float red[33];
  pdl_trigger();
  pdl_wait();
  const size_t t = blockIdx.x;
  const __nv_bfloat16* xr = x + t * ldx;
  float v[VEC_ITERS][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VEC_ITERS; ++i) {
    int c = (i * 256 + threadIdx.x) * 8;
    if (c < H) {
      uint4 a = *reinterpret_cast<const uint4*>(xr + c);
      const __nv_bfloat16* ap = reinterpret_cast<const __nv_bfloat16*>(&a);
      if (res_in != nullptr) {
        uint4 b = *reinterpret_cast<const uint4*>(res_in + t * H + c);
        const __nv_bfloat16* bp = reinterpret_cast<const __nv_bfloat16*>(&b);
        uint4 o;
        __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(&o);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          op[j] = __float2bfloat16(__bfloat162float(ap[j]) + __bfloat162float(bp[j]));
          v[i][j] = __bfloat162float(op[j]);
        }
        *reinterpret_cast<uint4*>(res_out + t * H + c) = o;
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[i][j] = __bfloat162float(ap[j]);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += v[i][j] * v[i][j];
    }
  }
  float tot = block_sum(ss, red);
  float inv = rsqrtf(tot / (float)H + eps);
#pragma unroll
  for (int i = 0; i < VEC_ITERS; ++i) {
    int c = (i * 256 + threadIdx.x) * 8;
    if (c < H) {
      uint4 ww = *reinterpret_cast<const uint4*>(w + c);
      const __nv_bfloat16* wp = reinterpret_cast<const __nv_bfloat16*>(&ww);
      uint4 o;
      __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(&o);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float g = __bfloat162float(wp[j]);
        op[j] = __float2bfloat16(v[i][j] * inv * (gemma ? 1.f + g : g));
      }
      *reinterpret_cast<uint4*>(y + t * H + c) = o;
    }
  }
}

// y = rmsnorm(x) * w * silu(z) over rows of D (64..256) elements; one warp per row.
__global__ void rms_norm_gated_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ z,
                                      const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y, int rows, int D,
                                      int ldx, int ldz, int heads, float eps) {
  int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  // rows are (token, head) pairs; x and z may be column slices of wider matrices
  const size_t tok = row / heads, hd = row % heads;
  const __nv_bfloat16* xr = x + tok * ldx + hd * D;
  const __nv_bfloat16* zr = z + tok * ldz + hd * D;
  float v[8];
  float ss = 0.f;
  int n = D / 32;
  for (int i = 0; i < n; ++i) {
    v[i] = __bfloat162float(xr[lane + 32 * i]);
    ss += v[i] * v[i];
  }
  ss = warp_sum(ss);
  float inv = rsqrtf(ss / (float)D + eps);
  for (int i = 0; i < n; ++i) {
    float g = __bfloat162float(zr[lane + 32 * i]);
    float o = v[i] * inv * __bfloat162float(w[lane + 32 * i]) * (g / (1.f + __expf(-g)));
    y[(size_t)row * D + lane + 32 * i] = __float2bfloat16(o);
  }
}

__global__ void silu_and_mul_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, int T, int I) {
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  size_t total = (size_t)T * I / 8;
  if (idx >= total) return;
  size_t t = idx / (I / 8), c = (idx % (I / 8)) * 8;
  uint4 g = *reinterpret_cast<const uint4*>(x + t * 2 * I + c);
  uint4 u = *reinterpret_cast<const uint4*>(x + t * 2 * I + I + c);
  const __nv_bfloat16 *gp = reinterpret_cast<const __nv_bfloat16*>(&g), *up = reinterpret_cast<const __nv_bfloat16*>(&u);
  uint4 o;
  __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(&o);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    float a = __bfloat162float(gp[j]);
    op[j] = __float2bfloat16(a / (1.f + __expf(-a)) * __bfloat162float(up[j]));
  }
  *reinterpret_cast<uint4*>(y + t * I + c) = o;
}

// One warp per (token, head): optional RMSNorm over the head, NeoX rotary on the first `rot` dims (q and k, in place),
// k and v rows copied into the paged cache [block][2][Hkv][bs][D] at slot_mapping[token].
__global__ void rope_cache_kernel(RopeCacheParams p) {
  extern __shared__ float sh[];
  pdl_trigger();
  pdl_wait();
  const int wpb = blockDim.x >> 5;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int heads = p.Hq + 2 * p.Hkv;
  const long long gw = (long long)blockIdx.x * wpb + warp;
  if (gw >= (long long)p.T * heads) return;
  const int t = (int)(gw / heads), hh = (int)(gw % heads);
  float* buf = sh + warp * p.D;
  const int D = p.D;
  __nv_bfloat16* src;
  const __nv_bfloat16* nw = nullptr;
  int kind;  // 0 q, 1 k, 2 v
  if (hh < p.Hq) { kind = 0; src = p.q + (size_t)t * p.q_st + (size_t)hh * p.q_sh; nw = p.q_norm; }
  else if (hh < p.Hq + p.Hkv) { kind = 1; src = p.k + (size_t)t * p.k_st + (size_t)(hh - p.Hq) * D; nw = p.k_norm; }
  else { kind = 2; src = p.v + (size_t)t * p.v_st + (size_t)(hh - p.Hq - p.Hkv) * D; }
  float ss = 0.f;
  for (int i = lane; i < D; i += 32) {
    float v = __bfloat162float(src[i]);
    buf[i] = v;
    ss += v * v;
  }
  if (kind != 2 && nw != nullptr) {
    ss = warp_sum(ss);
    float inv = rsqrtf(ss / (float)D + p.eps);
    for (int i = lane; i < D; i += 32) {
      float g = __bfloat162float(nw[i]);
      // the normalised value is rounded to bf16 before the rotation, like the separate-kernel formulation
      buf[i] = __bfloat162float(__float2bfloat16(buf[i] * inv * (p.gemma ? 1.f + g : g)));
    }
  }
  __syncwarp();
  const long long slot = (kind != 0 && p.kv_cache != nullptr) ? (long long)p.slot_mapping[t] : -1;
  __nv_bfloat16* cdst = nullptr;
  uint8_t* cdst8 = nullptr;  // fp8 cache: same element index, one byte each
  if (slot >= 0) {
    long long blk = slot / p.bs, off = slot % p.bs;
    int h = (kind == 1) ? hh - p.Hq : hh - p.Hq - p.Hkv;
    const size_t e = ((((size_t)blk * 2 + (kind - 1)) * p.Hkv + h) * p.bs + off) * D;
    if (p.kv_fp8) cdst8 = reinterpret_cast<uint8_t*>(p.kv_cache) + e;
    else cdst = p.kv_cache + e;
  }
  if (kind == 2) {
    if (cdst != nullptr)
      for (int i = lane; i < D; i += 32) cdst[i] = src[i];
    if (cdst8 != nullptr)
      for (int i = lane; i < D; i += 32)
        cdst8[i] = (uint8_t)__nv_cvt_float_to_fp8(buf[i] * p.v_scale_inv, __NV_SATFINITE, __NV_E4M3);
    return;
  }
  const int half = p.rot >> 1;
  const float* cs = p.cos_sin + (size_t)p.positions[t] * p.rot;
  const float *cs1 = cs, *cs2 = cs;
  if (p.mrope_s0 > 0) {  // the height and width components of the position
    cs1 = p.cos_sin + (size_t)p.positions[p.pos_stride + t] * p.rot;
    cs2 = p.cos_sin + (size_t)p.positions[2 * p.pos_stride + t] * p.rot;
  }
  for (int i = lane; i < D; i += 32) {
    float o;
    const int f = i < half ? i : i - half;
    const float* c = (p.mrope_s0 == 0 || f < p.mrope_s0) ? cs : (f < p.mrope_s1 ? cs1 : cs2);
    if (i < half) o = buf[i] * c[i] - buf[i + half] * c[half + i];
    else if (i < p.rot) o = buf[i] * c[i - half] + buf[i - half] * c[i];
    else o = buf[i];
    __nv_bfloat16 ob = __float2bfloat16(o);
    src[i] = ob;
    if (cdst != nullptr) cdst[i] = ob;
    if (cdst8 != nullptr) cdst8[i] = (uint8_t)__nv_cvt_float_to_fp8(__bfloat162float(ob) * p.k_scale_inv, __NV_SATFINITE, __NV_E4M3);
  }
}

// arg-max of each row of a [B, V] bf16/fp32 matrix; ties go to the lowest index (torch semantics). A row is split over gridDim.y
// CTAs; each folds its part into one 64-bit word per row with atomicMax: the high half is the value mapped to an order-preserving
// unsigned key, the low half is ~index, so the largest word is the largest value at its lowest index. A second tiny kernel unpacks.
__device__ __forceinline__ unsigned int float_order_key(float v) {
  unsigned int b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
template <typename T>
__global__ void __launch_bounds__(256) argmax_partial_kernel(const T* __restrict__ x, unsigned long long* __restrict__ packed, int V, long long ld, int vec) {
  __shared__ float sv[8];
  __shared__ int si[8];
  pdl_trigger();
  pdl_wait();
  const T* r = x + (size_t)blockIdx.x * ld;
  const int per = (((V + gridDim.y - 1) / gridDim.y) + 7) & ~7;
  const int lo = blockIdx.y * per, hi = min(lo + per, V);
  float best = -INFINITY;
  int bi = 0x7fffffff;
  auto take = [&](float v, int i) { if (v > best || (v == best && i < bi)) { best = v; bi = i; } };
  if (vec && sizeof(T) == 2) {  // 16-byte loads of eight bf16 (the caller checked the alignment of every row)
    for (int i = lo + threadIdx.x * 8; i < hi; i += blockDim.x * 8) {
      if (i + 8 <= hi) {
        const uint4 q = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(r) + i);
        const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&q);
#pragma unroll
        for (int j = 0; j < 8; ++j) take(__bfloat162float(e[j]), i + j);
      } else {
        for (int j = i; j < hi; ++j) take((float)r[j], j);
      }
    }
  } else {
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) take((float)r[i], i);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float ov = __shfl_xor_sync(0xffffffffu, best, o);
    int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = best; si[threadIdx.x >> 5] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w)
      if (sv[w] > best || (sv[w] == best && si[w] < bi)) { best = sv[w]; bi = si[w]; }
    if (bi != 0x7fffffff)
      atomicMax(&packed[blockIdx.x], ((unsigned long long)float_order_key(best) << 32) | (unsigned long long)(0xffffffffu - (unsigned int)bi));
  }
}
__global__ void argmax_unpack_kernel(const unsigned long long* __restrict__ packed, long long* __restrict__ out, int B) {
  pdl_trigger();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < B) out[i] = packed[i] == 0ull ? 0 : (long long)(0xffffffffu - (unsigned int)(packed[i] & 0xffffffffull));
}

}  // namespace

int rms_norm_launch(const void* x, const void* res_in, const void* w, void* y, void* res_out, int T, int H, int ldx, float eps,
                    int gemma, cudaStream_t st) {
  if (H % 8 || H > 256 * 8 * 4) return -1;
  const __nv_bfloat16 *xp = (const __nv_bfloat16*)x, *rp = (const __nv_bfloat16*)res_in, *wp = (const __nv_bfloat16*)w;
  __nv_bfloat16 *yp = (__nv_bfloat16*)y, *rop = (__nv_bfloat16*)res_out;
  int iters = (H + 2047) / 2048;
  if (T == 0) return 0;
  switch (iters) {
    case 1: launch_k(rms_norm_kernel<1>, dim3(T), dim3(256), 0, st, true, xp, rp, wp, yp, rop, H, ldx, eps, gemma); break;
    case 2: launch_k(rms_norm_kernel<2>, dim3(T), dim3(256), 0, st, true, xp, rp, wp, yp, rop, H, ldx, eps, gemma); break;
    case 3: launch_k(rms_norm_kernel<3>, dim3(T), dim3(256), 0, st, true, xp, rp, wp, yp, rop, H, ldx, eps, gemma); break;
    default: launch_k(rms_norm_kernel<4>, dim3(T), dim3(256), 0, st, true, xp, rp, wp, yp, rop, H, ldx, eps, gemma); break;
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int rms_norm_gated_launch(const void* x, const void* z, const void* w, void* y, int rows, int D, int ldx, int ldz, int heads,
                          float eps, cudaStream_t st) {
  if (D % 32 || D > 256) return -1;
  if (rows == 0) return 0;
  rms_norm_gated_kernel<<<(rows + 7) / 8, 256, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)z, (const __nv_bfloat16*)w,
                                                        (__nv_bfloat16*)y, rows, D, ldx, ldz, heads, eps);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int silu_and_mul_launch(const void* x, void* y, int T, int I, cudaStream_t st) {
  if (I % 8) return -1;
  size_t total = (size_t)T * I / 8;
  if (total == 0) return 0;
  silu_and_mul_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, T, I);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int rope_cache_launch(const RopeCacheParams& p, cudaStream_t st) {
  if (p.T == 0) return 0;
  if (p.D > 512 || p.rot > p.D || (p.rot & 1)) return -1;
  long long warps = (long long)p.T * (p.Hq + 2 * p.Hkv);
  int wpb = 8;
  launch_k(rope_cache_kernel, dim3((unsigned)((warps + wpb - 1) / wpb)), dim3(wpb * 32), wpb * p.D * sizeof(float), st, true, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// o = w1 o1 + w2 o2 with w_i = e^{lse_i - m} / (e^{lse1 - m} + e^{lse2 - m}), m = max(lse1, lse2); lse = m + log(sum): the merge of two
// attention results over disjoint key sets (split contexts, cascade prefixes, decode context parallel ranks). One warp per (token, head) row.
// (reference: csrc/attention/merge_attn_states.cu:19)
__global__ void merge_attn_states_kernel(const __nv_bfloat16* o1, const float* lse1, const __nv_bfloat16* o2, const float* lse2, __nv_bfloat16* out,
                                         float* lse_out, int rows, int D) {
  const int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (row >= rows) return;
  const float a = lse1[row], b = lse2[row];
  float m = fmaxf(a, b);
  if (isinf(m)) m = 0.f;  // both sides empty (or +inf): weights fall back to equal shares of zero outputs
  const float w1 = __expf(a - m), w2 = __expf(b - m);
  const float den = fmaxf(w1 + w2, 1e-30f);
  const float f1 = w1 / den, f2 = w2 / den;
  for (int c = lane * 2; c < D; c += 64) {
    const float2 x = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(o1 + (size_t)row * D + c));
    const float2 y = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(o2 + (size_t)row * D + c));
    *reinterpret_cast<__nv_bfloat162*>(out + (size_t)row * D + c) = __floats2bfloat162_rn(x.x * f1 + y.x * f2, x.y * f1 + y.y * f2);
  }
  if (lane == 0 && lse_out != nullptr) lse_out[row] = m + __logf(den);
}

int merge_attn_states_launch(const void* o1, const float* lse1, const void* o2, const float* lse2, void* out, float* lse_out, int rows, int D,
                             cudaStream_t st) {
  if (D % 2) return -1;
  if (rows == 0) return 0;
  merge_attn_states_kernel<<<(rows * 32 + 255) / 256, 256, 0, st>>>((const __nv_bfloat16*)o1, lse1, (const __nv_bfloat16*)o2, lse2, (__nv_bfloat16*)out,
                                                                   lse_out, rows, D);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// `packed` is B zeroed 64-bit words of scratch (zeroed by the caller before every call).
int argmax_launch(const void* x, int is_fp32, long long* out, unsigned long long* packed, int B, int V, long long ld, cudaStream_t st) {
  if (B == 0) return 0;
  int splits = V >= (1 << 15) ? (B >= 128 ? 4 : 16) : 1;
  const int vec = (!is_fp32 && ld % 8 == 0 && ((uintptr_t)x & 15) == 0) ? 1 : 0;
  dim3 grid((unsigned)B, (unsigned)splits);
  if (is_fp32) launch_k(argmax_partial_kernel<float>, grid, dim3(256), 0, st, true, (const float*)x, packed, V, ld, 0);
  else launch_k(argmax_partial_kernel<__nv_bfloat16>, grid, dim3(256), 0, st, true, (const __nv_bfloat16*)x, packed, V, ld, vec);
  launch_k(argmax_unpack_kernel, dim3((B + 255) / 256), dim3(256), 0, st, true, (const unsigned long long*)packed, out, B);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

unsigned int elementwise_read_status(bool clear) { return read_status_tu(clear); }
void elementwise_read_status_async(unsigned int* dst, cudaStream_t st) { read_status_tu_async(dst, st); }

}  // namespace oc
