// Gated-DeltaNet kernels: depthwise causal conv (k <= 4) + SiLU over variable-length batches with a rolling per-sequence
// state, and the gated delta rule itself with fused gating (g = -exp(A_log) * softplus(a + dt_bias), beta = sigmoid(b)),
// q/k L2 normalisation and fp32 state [K=128][V=128] per (sequence, value head).
//
// Recurrence kernel: one CTA per (sequence, value head), 128 threads; thread j keeps column j of the state in 128 registers,
// so the decay, the k-projection (S^T k), the rank-1 update and the output (S^T q) are thread-local FMAs with q and k
// broadcast from shared memory. Tokens of a sequence are consumed in order, which makes the same kernel serve single-token
// decode, multi-token verification (optionally recording the state after every token) and prefill chunks.
//   S <- e^g S ;  d = (v - S^T k) * beta ;  S <- S + k d^T ;  o = S^T q * K^-1/2
// (reference: flash_qla/ops/gated_delta_rule/chunk/sm70/csrc/gdn_forward.cu:131-215,243,399; gating
//  layers/mamba/gdn/qwen_gdn_linear_attn.py:6945-7013; conv layers/mamba/ops/causal_conv1d.py:16,746)
#include "common.cuh"
#include "kernels.h"

namespace oc {
namespace {

__device__ __forceinline__ int find_request(const int* qsl, int R, int t) {
  int lo = 0, hi = R;  // qsl[lo] <= t < qsl[hi]
  while (hi - lo > 1) {
    int mid = (lo + hi) >> 1;
    if (qsl[mid] <= t) lo = mid; else hi = mid;
  }
  return lo;
}

// y[t, c] = silu(sum_j w[c, j] * x[t - (kw-1) + j, c]) where rows before the sequence start come from conv_state[slot][c][*]
// (or zero without an initial state). One thread per (token, 8 channels): 16-byte loads of the kw input rows and one 16-byte store;
// VEC = 1 is the fallback for channel counts or pitches that are not multiples of 8.
template <int VEC>
__global__ void gdn_conv_kernel(const GdnConvParams p) {
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * VEC;
  const int t = blockIdx.y;
  __shared__ int s_r;
  if (threadIdx.x == 0) s_r = find_request(p.query_start_loc, p.R, t);
  __syncthreads();
  if (c >= p.C) return;
  const int r = s_r;
  const int t0 = p.query_start_loc[r];
  const int slot = p.state_slots[r];
  const bool has_init = p.has_initial_state[r] != 0;
  const int kw = p.kw;
  float acc[VEC];
#pragma unroll
  for (int e = 0; e < VEC; ++e) acc[e] = 0.f;
  // taps of this thread's channels: [channel][tap] is contiguous, so eight channels of a 4-tap filter are four 16-byte loads
  float wv[VEC][4];
  if (VEC == 8) {
    const uint4* wp = reinterpret_cast<const uint4*>(p.w + (size_t)c * 4);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint4 raw = wp[i];
      const __nv_bfloat16* rp = reinterpret_cast<const __nv_bfloat16*>(&raw);
#pragma unroll
      for (int e = 0; e < 8; ++e) wv[(i * 8 + e) >> 2][(i * 8 + e) & 3] = __bfloat162float(rp[e]);
    }
  }
  const int taps = VEC == 8 ? 4 : kw;  // a compile-time 4 on the vector path, so wv[][j] stays in registers
#pragma unroll
  for (int j = 0; j < taps; ++j) {
    const int tt = t - (kw - 1) + j;
    float xv[VEC];
    if (tt >= t0) {
      if (VEC == 8) {
        const uint4 raw = *reinterpret_cast<const uint4*>(p.x + (size_t)tt * p.ldx + c);
        const __nv_bfloat16* rp = reinterpret_cast<const __nv_bfloat16*>(&raw);
#pragma unroll
        for (int e = 0; e < VEC; ++e) xv[e] = __bfloat162float(rp[e]);
      } else {
        xv[0] = __bfloat162float(p.x[(size_t)tt * p.ldx + c]);
      }
    } else {
#pragma unroll
      for (int e = 0; e < VEC; ++e)
        xv[e] = has_init ? __bfloat162float(p.conv_state[((size_t)slot * p.C + c + e) * (kw - 1) + (kw - 1) + (tt - t0)]) : 0.f;
    }
#pragma unroll
    for (int e = 0; e < VEC; ++e) acc[e] += xv[e] * (VEC == 8 ? wv[e][j & 3] : __bfloat162float(p.w[(size_t)(c + e) * kw + j]));
  }
  if (VEC == 8) {
    uint4 o;
    __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(&o);
#pragma unroll
    for (int e = 0; e < VEC; ++e) op[e] = __float2bfloat16(acc[e] / (1.f + __expf(-acc[e])));
    *reinterpret_cast<uint4*>(p.y + (size_t)t * p.C + c) = o;
  } else {
    p.y[(size_t)t * p.C + c] = __float2bfloat16(acc[0] / (1.f + __expf(-acc[0])));
  }
}

// conv_state[slot][c][:] <- the last kw-1 inputs of the sequence (mixing old state and new tokens when the chunk is short).
// Must run after gdn_conv_kernel (it overwrites what that kernel reads). One thread per (request, channel).
__global__ void gdn_conv_state_kernel(const GdnConvParams p) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int r = blockIdx.y;
  if (c >= p.C) return;
  const int t0 = p.query_start_loc[r], t1 = p.query_start_loc[r + 1];
  int n = t1 - t0;
  if (n <= 0) return;
  if (p.n_valid != nullptr) n = min(n, max(p.n_valid[r], 0));  // speculative commit: only the accepted tokens count
  const int slot = p.state_slots[r];
  const bool has_init = p.has_initial_state[r] != 0;
  const int m = p.kw - 1;
  __nv_bfloat16* st = p.conv_state + ((size_t)slot * p.C + c) * m;
  // the state *before* the chunk: the slot itself, or a snapshot when the slot was already advanced by the full chunk
  const __nv_bfloat16* before = p.prev_state != nullptr ? p.prev_state + ((size_t)r * p.C + c) * m : st;
  float vals[8];
  for (int j = 0; j < m; ++j) {
    const int idx = n - m + j;  // position relative to this chunk's first token
    if (idx >= 0) vals[j] = __bfloat162float(p.x[(size_t)(t0 + idx) * p.ldx + c]);
    else vals[j] = (has_init || p.prev_state != nullptr) ? __bfloat162float(before[m + idx]) : 0.f;
  }
  for (int j = 0; j < m; ++j) st[j] = __float2bfloat16(vals[j]);
}

constexpr int GK = 128, GV = 128;

constexpr int CH = 16;      // tokens whose inputs are staged together (their global loads are in flight at the same time)
constexpr int VC = 32;      // state columns per CTA
constexpr int NP = 4;       // lanes per state column
constexpr int GT = NP * VC; // threads per CTA
constexpr int HK = GK / NP; // state rows per thread

// One CTA per (sequence, value head, group of 32 state columns). The K x V fp32 state lives in registers: a warp owns 8 columns and
// a column is split over four of its lanes (lane = column + 8 * part, part p holds rows 32p .. 32p + 31), so a thread keeps 32 state
// values and the 32 key values of the current token, and partial dot products meet through two shuffles. Tokens are strictly
// sequential, so a warp is latency-bound per token (measured: 0.4 instructions per cycle); 16 warps per head put enough warps on
// every scheduler even for a single long sequence. The q/k/v rows of CH tokens are copied asynchronously into shared memory while
// the previous chunk is processed, and the dot products run on four independent accumulators.
__global__ void __launch_bounds__(GT) gdn_recurrent_kernel(const GdnParams p) {
  __shared__ __align__(16) float sq[CH][GK], sk[CH][GK];
  __shared__ float sv[CH][VC];
  __shared__ float sdecay[CH], sbeta[CH];
  __shared__ __align__(16) __nv_bfloat16 raw[CH][2][GK];  // the next chunk's q and k rows as they are in global memory
  __shared__ __align__(16) __nv_bfloat16 rawv[CH][VC];    // and this CTA's slice of the v rows
  const int r = blockIdx.x, hv = blockIdx.y, c0 = blockIdx.z * VC;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int lc = warp * 8 + (lane & 7), col = c0 + lc, half = lane >> 3;  // `half` = which quarter of the rows
  const int t0 = p.query_start_loc[r], t1 = p.query_start_loc[r + 1];
  if (t1 <= t0 || (p.skip_min_len > 0 && t1 - t0 >= p.skip_min_len)) return;
  const int hk = hv / (p.Hv / p.Hk);
  // sequences short enough for the recording buffer are recorded (and committed later by the host); longer ones, e.g. a
  // prefill chunk sharing the step with verification requests, update their slot directly
  const bool rec = p.spec_state != nullptr && (t1 - t0) <= p.spec_q;
  const int slot = p.state_slots[r];
  float* Sg = p.state + ((size_t)slot * p.Hv + hv) * GK * GV + (size_t)half * HK * GV + col;
  float S[HK];
  if (p.has_initial_state[r]) {
#pragma unroll
    for (int k = 0; k < HK; ++k) S[k] = Sg[(size_t)k * GV];
  } else {
#pragma unroll
    for (int k = 0; k < HK; ++k) S[k] = 0.f;
  }
  const float neg_a = -__expf(p.A_log[hv]);
  const float dtb = p.dt_bias[hv];
  const float scale = rsqrtf((float)GK);

  float ra = 0.f, rb = 0.f;
  // asynchronous 16-byte copies of a chunk's rows: warp w copies tokens w, w + 4, ...; per token the 32 lanes copy the 16 + 16
  // segments of the q and k rows (256 bytes each) and lanes 0-3 this CTA's 64-byte slice of the v row
  auto fetch = [&](int tc) {
    const int n = min(CH, t1 - tc);
    for (int i = warp; i < n; i += GT / 32) {
      const size_t row = (size_t)(tc + i) * p.ld_qkv;
      const int which = lane >> 4, seg = lane & 15;
      const __nv_bfloat16* src = (which == 0 ? p.q : p.k) + row + hk * GK + seg * 8;
      uint32_t dst = (uint32_t)__cvta_generic_to_shared(&raw[i][which][seg * 8]);
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
      if (lane < VC / 8) {
        src = p.v + row + hv * GV + c0 + lane * 8;
        dst = (uint32_t)__cvta_generic_to_shared(&rawv[i][lane * 8]);
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    if (tid < n) {
      ra = __bfloat162float(p.a[(size_t)(tc + tid) * p.ld_ba + hv]);
      rb = __bfloat162float(p.b[(size_t)(tc + tid) * p.ld_ba + hv]);
    }
  };
  fetch(t0);
  for (int tc = t0; tc < t1; tc += CH) {
    const int n = min(CH, t1 - tc);
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();  // the chunk has landed, and the previous chunk's recurrence is done with the float arrays
    if (tid < n) {
      const float av = ra + dtb;
      const float sp = av > 20.f ? av : log1pf(__expf(av));
      sdecay[tid] = __expf(neg_a * sp);
      sbeta[tid] = 1.f / (1.f + __expf(-rb));
    }
    // convert and L2-normalise q and k of every token of the chunk (warp w takes tokens w, w + 4, ...), convert the v slice
#pragma unroll 1
    for (int i = warp; i < n; i += GT / 32) {
      float q4[4], k4[4], q2 = 0.f, k2 = 0.f;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        q4[e] = __bfloat162float(raw[i][0][lane + 32 * e]);
        k4[e] = __bfloat162float(raw[i][1][lane + 32 * e]);
        q2 += q4[e] * q4[e];
        k2 += k4[e] * k4[e];
      }
      sv[i][lane] = __bfloat162float(rawv[i][lane]);
      q2 = warp_sum(q2);
      k2 = warp_sum(k2);
      const float qs = rsqrtf(q2 + 1e-6f) * scale, ks = rsqrtf(k2 + 1e-6f);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        sq[i][lane + 32 * e] = q4[e] * qs;
        sk[i][lane + 32 * e] = k4[e] * ks;
      }
    }
    __syncthreads();  // the raw rows have been consumed, the float arrays are complete
    if (tc + CH < t1) fetch(tc + CH);  // in flight while this chunk is processed
#pragma unroll 1
    for (int i = 0; i < n; ++i) {
      const float decay = sdecay[i], beta = sbeta[i], vj = sv[i][lc];
      const float4* k4p = reinterpret_cast<const float4*>(&sk[i][half * HK]);
      const float4* q4p = reinterpret_cast<const float4*>(&sq[i][half * HK]);
      float kr[HK];
      float pj[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int k = 0; k < HK; k += 4) {
        const float4 kk = k4p[k >> 2];
        kr[k] = kk.x; kr[k + 1] = kk.y; kr[k + 2] = kk.z; kr[k + 3] = kk.w;
        S[k] *= decay; S[k + 1] *= decay; S[k + 2] *= decay; S[k + 3] *= decay;
        pj[0] += kk.x * S[k]; pj[1] += kk.y * S[k + 1]; pj[2] += kk.z * S[k + 2]; pj[3] += kk.w * S[k + 3];
      }
      float proj = (pj[0] + pj[1]) + (pj[2] + pj[3]);
      proj += __shfl_xor_sync(0xffffffffu, proj, 8);
      proj += __shfl_xor_sync(0xffffffffu, proj, 16);
      const float d = (vj - proj) * beta;
      float oj[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int k = 0; k < HK; k += 4) {
        const float4 qq = q4p[k >> 2];
        S[k] += kr[k] * d; S[k + 1] += kr[k + 1] * d; S[k + 2] += kr[k + 2] * d; S[k + 3] += kr[k + 3] * d;
        oj[0] += qq.x * S[k]; oj[1] += qq.y * S[k + 1]; oj[2] += qq.z * S[k + 2]; oj[3] += qq.w * S[k + 3];
      }
      float o = (oj[0] + oj[1]) + (oj[2] + oj[3]);
      o += __shfl_xor_sync(0xffffffffu, o, 8);
      o += __shfl_xor_sync(0xffffffffu, o, 16);
      const int t = tc + i;
      if (half == 0) p.out[(size_t)t * p.Hv * GV + hv * GV + col] = __float2bfloat16(o);
      if (rec) {
        float* dst = p.spec_state + (((size_t)r * p.spec_q + (t - t0)) * p.Hv + hv) * GK * GV + (size_t)half * HK * GV + col;
#pragma unroll
        for (int k = 0; k < HK; ++k) dst[(size_t)k * GV] = S[k];
      }
    }
  }
  if (p.write_state || !rec) {
#pragma unroll
    for (int k = 0; k < HK; ++k) Sg[(size_t)k * GV] = S[k];
  }
}

}  // namespace

int gdn_conv_launch(const GdnConvParams& p, cudaStream_t st) {
  if (p.T == 0) return 0;
  if (p.kw < 2 || p.kw > 8) return -1;
  if (p.kw == 4 && p.C % 8 == 0 && p.ldx % 8 == 0 && ((uintptr_t)p.x & 15) == 0 && ((uintptr_t)p.y & 15) == 0 && ((uintptr_t)p.w & 15) == 0) {
    dim3 grid((p.C / 8 + 127) / 128, p.T);
    gdn_conv_kernel<8><<<grid, 128, 0, st>>>(p);
  } else {
    dim3 grid((p.C + 255) / 256, p.T);
    gdn_conv_kernel<1><<<grid, 256, 0, st>>>(p);
  }
  dim3 g2((p.C + 255) / 256, p.R);
  gdn_conv_state_kernel<<<g2, 256, 0, st>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int gdn_conv_commit_launch(const GdnConvParams& p, cudaStream_t st) {
  if (p.R == 0) return 0;
  dim3 g2((p.C + 255) / 256, p.R);
  gdn_conv_state_kernel<<<g2, 256, 0, st>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int gdn_recurrent_launch(const GdnParams& p, cudaStream_t st) {
  if (p.R == 0) return 0;
  if (p.K != GK || p.V != GV || p.Hv % p.Hk) return -1;
  dim3 grid(p.R, p.Hv, GV / VC);
  gdn_recurrent_kernel<<<grid, GT, 0, st>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

unsigned int gdn_read_status(bool clear) { return read_status_tu(clear); }
void gdn_read_status_async(unsigned int* dst, cudaStream_t st) { read_status_tu_async(dst, st); }

}  // namespace oc
