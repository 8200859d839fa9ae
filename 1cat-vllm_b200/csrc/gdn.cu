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
// (or zero without an initial state). One thread per (token, channel).
__global__ void gdn_conv_kernel(const GdnConvParams p) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int t = blockIdx.y;
  if (c >= p.C) return;
  const int r = find_request(p.query_start_loc, p.R, t);
  const int t0 = p.query_start_loc[r];
  const int slot = p.state_slots[r];
  const bool has_init = p.has_initial_state[r] != 0;
  const int kw = p.kw;
  float acc = 0.f;
  for (int j = 0; j < kw; ++j) {
    const int tt = t - (kw - 1) + j;
    float xv;
    if (tt >= t0) xv = __bfloat162float(p.x[(size_t)tt * p.ldx + c]);
    else if (has_init) xv = __bfloat162float(p.conv_state[((size_t)slot * p.C + c) * (kw - 1) + (kw - 1) + (tt - t0)]);
    else xv = 0.f;
    acc += xv * __bfloat162float(p.w[(size_t)c * kw + j]);
  }
  p.y[(size_t)t * p.C + c] = __float2bfloat16(acc / (1.f + __expf(-acc)));
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

__global__ void __launch_bounds__(GV) gdn_recurrent_kernel(const GdnParams p) {
  __shared__ float sq[GK], sk[GK];
  __shared__ float red[2][4];
  const int r = blockIdx.x, hv = blockIdx.y;
  const int j = threadIdx.x;
  const int t0 = p.query_start_loc[r], t1 = p.query_start_loc[r + 1];
  if (t1 <= t0) return;
  const int hk = hv / (p.Hv / p.Hk);
  // sequences short enough for the recording buffer are recorded (and committed later by the host); longer ones, e.g. a
  // prefill chunk sharing the step with verification requests, update their slot directly
  const bool rec = p.spec_state != nullptr && (t1 - t0) <= p.spec_q;
  const int slot = p.state_slots[r];
  float* Sg = p.state + ((size_t)slot * p.Hv + hv) * GK * GV;
  float S[GK];
  if (p.has_initial_state[r]) {
#pragma unroll
    for (int k = 0; k < GK; ++k) S[k] = Sg[(size_t)k * GV + j];
  } else {
#pragma unroll
    for (int k = 0; k < GK; ++k) S[k] = 0.f;
  }
  const float neg_a = -__expf(p.A_log[hv]);
  const float dtb = p.dt_bias[hv];
  const float scale = rsqrtf((float)GK);
  for (int t = t0; t < t1; ++t) {
    // q, k of the key head: L2-normalise (block reduction over K = blockDim)
    const float qv = __bfloat162float(p.q[(size_t)t * p.ld_qkv + hk * GK + j]);
    const float kv = __bfloat162float(p.k[(size_t)t * p.ld_qkv + hk * GK + j]);
    float q2 = warp_sum(qv * qv), k2 = warp_sum(kv * kv);
    __syncthreads();  // previous iteration is done with sq/sk/red
    if ((j & 31) == 0) { red[0][j >> 5] = q2; red[1][j >> 5] = k2; }
    __syncthreads();
    q2 = red[0][0] + red[0][1] + red[0][2] + red[0][3];
    k2 = red[1][0] + red[1][1] + red[1][2] + red[1][3];
    sq[j] = qv * rsqrtf(q2 + 1e-6f) * scale;
    sk[j] = kv * rsqrtf(k2 + 1e-6f);
    __syncthreads();
    const float av = __bfloat162float(p.a[(size_t)t * p.ld_ba + hv]) + dtb;
    const float sp = av > 20.f ? av : log1pf(__expf(av));
    const float decay = __expf(neg_a * sp);
    const float bv = __bfloat162float(p.b[(size_t)t * p.ld_ba + hv]);
    const float beta = 1.f / (1.f + __expf(-bv));
    const float vj = __bfloat162float(p.v[(size_t)t * p.ld_qkv + hv * GV + j]);
    float proj = 0.f;
#pragma unroll
    for (int k = 0; k < GK; ++k) {
      S[k] *= decay;
      proj += sk[k] * S[k];
    }
    const float d = (vj - proj) * beta;
    float o = 0.f;
#pragma unroll
    for (int k = 0; k < GK; ++k) {
      S[k] += sk[k] * d;
      o += sq[k] * S[k];
    }
    p.out[(size_t)t * p.Hv * GV + hv * GV + j] = __float2bfloat16(o);
    if (rec) {
      float* dst = p.spec_state + (((size_t)r * p.spec_q + (t - t0)) * p.Hv + hv) * GK * GV;
#pragma unroll
      for (int k = 0; k < GK; ++k) dst[(size_t)k * GV + j] = S[k];
    }
  }
  if (p.write_state || !rec) {
#pragma unroll
    for (int k = 0; k < GK; ++k) Sg[(size_t)k * GV + j] = S[k];
  }
}

}  // namespace

int gdn_conv_launch(const GdnConvParams& p, cudaStream_t st) {
  if (p.T == 0) return 0;
  if (p.kw < 2 || p.kw > 8) return -1;
  dim3 grid((p.C + 255) / 256, p.T);
  gdn_conv_kernel<<<grid, 256, 0, st>>>(p);
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
  dim3 grid(p.R, p.Hv);
  gdn_recurrent_kernel<<<grid, GV, 0, st>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

unsigned int gdn_read_status(bool clear) { return read_status_tu(clear); }

}  // namespace oc
