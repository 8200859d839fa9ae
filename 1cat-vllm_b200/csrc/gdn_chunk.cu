// Gated-DeltaNet prefill in chunked (WY) form on tensor cores.
//
// The recurrence   S_t = a_t (I - b_t k_t k_t^T) S_{t-1} + b_t k_t v_t^T ,  o_t = S_t^T q_t   (a_t = e^{g_t}, b_t = beta_t)
// is sequential per token; over a chunk of C = 64 tokens it can be restated with a handful of small matrix products. With the
// in-chunk cumulative log-decay G_i = sum_{j<=i} g_j and Gamma_ij = e^{G_i - G_j}:
//   A     = strictly-lower( diag(b) (K K^T) .* Gamma )                T = (I + A)^-1              (unit lower triangular)
//   W     = T diag(b e^G) K        U = T diag(b) V                    P = lower-incl( (Q K^T) .* Gamma )
//   Vnew  = U - W S0               O = (e^G .* Q) S0 + P Vnew         S_end = e^{G_C} S0 + (e^{G_C - G} .* K)^T Vnew
// Everything that does not involve S0 is independent across chunks (kernel A below, one CTA per chunk and value head); what is
// left per chunk on the sequential path is three products against the 128 x 128 state (kernel B, one CTA per sequence, value head
// and 64-column half of the state, which lives in fp32 accumulator registers for the whole sequence).
//
// Why mma.sync and not tcgen05 here: kernel B is a chain of dependent 64 x 64 x 128 products per 64 tokens with a register-resident
// fp32 state; each link would pay a tcgen05.commit / mbarrier / tcgen05.ld round trip, and the products are far too small for the
// tensor pipe to be the limit. Warp-level MMAs keep operands and state in registers and shared memory with four CTA barriers per
// chunk. Kernel A uses the same instruction so that both share fragment helpers.
// (reference: layers/fla/ops/chunk.py:23 chunk_gated_delta_rule; layers/mamba/ops/gdn_chunk_cutedsl/kernel_{kkt_inv_uw,h,o}.py;
//  flash_qla/ops/gated_delta_rule/chunk/sm70/csrc/gdn_forward.cu:243)
#include "common.cuh"
#include "kernels.h"

namespace oc {
namespace {

constexpr int C = 64;        // tokens per chunk
constexpr int D = 128;       // key and value head size
constexpr int P128 = 136;    // shared-memory row pitch (elements) of a [*][128] bf16 tile: 272 bytes, 8 rows hit 8 different bank groups
constexpr int P64 = 72;      // same for a [*][64] tile: 144 bytes

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
// A fragment (16 x 16) of a row-major [m][k] tile: element (m0 + i, k0 + j)
__device__ __forceinline__ uint32_t a_addr(uint32_t base, int pitch, int m0, int k0, int lane) {
  return base + (uint32_t)(((m0 + (lane & 7) + ((lane >> 3) & 1) * 8) * pitch + k0 + (lane >> 4) * 8) * 2);
}
// B fragments of two adjacent n tiles from a tile stored [n][k] (k contiguous): r0, r1 = tile n0; r2, r3 = tile n0 + 8
__device__ __forceinline__ uint32_t bnk_addr(uint32_t base, int pitch, int n0, int k0, int lane) {
  return base + (uint32_t)(((n0 + (lane & 7) + (lane >> 4) * 8) * pitch + k0 + ((lane >> 3) & 1) * 8) * 2);
}
// B fragments of two adjacent n tiles from a tile stored [k][n] (n contiguous), loaded transposed
__device__ __forceinline__ uint32_t bkn_addr(uint32_t base, int pitch, int k0, int n0, int lane) {
  return base + (uint32_t)(((k0 + (lane & 7) + ((lane >> 3) & 1) * 8) * pitch + n0 + (lane >> 4) * 8) * 2);
}
// A fragment of X^T where X is stored [k][m] (m contiguous), loaded transposed: element (m0 + i, k0 + j) = X[k0 + j][m0 + i]
__device__ __forceinline__ uint32_t at_addr(uint32_t base, int pitch, int m0, int k0, int lane) {
  return base + (uint32_t)(((k0 + (lane & 7) + (lane >> 4) * 8) * pitch + m0 + ((lane >> 3) & 1) * 8) * 2);
}

// ---------------------------------------------------------------------------------------------------------------- kernel A
// grid (chunks, Hv), 128 threads. Workspace per (chunk, head): W, U, Qg, Kd as bf16 [64][128], P as bf16 [64][64], e^{G_C} as float.
constexpr size_t kWsTile = (size_t)C * D;                        // elements
constexpr size_t kWsPerHead = 4 * kWsTile + (size_t)C * C + 8;   // + 8 bf16 = 16 bytes for the closing decay (kept 16-byte aligned)

// Storage is reused so that four CTAs fit an SM (the kernel is a chain of short dependent phases; resident warps hide its latencies):
//   q: normalised q rows -> fp32 T of the triangular solve -> beta-scaled v rows;   a: fp32 A -> bf16 T (the A operand of W and U)
struct SmemA {
  __nv_bfloat16 q[C][P128], k[C][P128];
  float a[C][C + 1];
  float m[3][16][17];
  float G[C], beta[C];
};

__global__ void __launch_bounds__(128) gdn_chunk_prepare_kernel(const GdnChunkParams p) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  SmemA& s = *reinterpret_cast<SmemA*>(smem_raw);
  const int ci = blockIdx.x, hv = blockIdx.y;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int r = p.chunk_req[ci];
  const int tc = p.chunk_t0[ci];                 // first token of the chunk
  const int t1 = p.query_start_loc[r + 1];
  const int n = min(C, t1 - tc);
  const int hk = hv / (p.Hv / p.Hk);
  const float neg_a = -__expf(p.A_log[hv]);
  const float dtb = p.dt_bias[hv];
  const float scale = rsqrtf((float)D);
  // gates: log-decay g and beta per token (tokens past the end of the sequence: g = 0, beta = 0, which leaves the state alone)
  if (tid < C) {
    float g = 0.f, be = 0.f;
    if (tid < n) {
      const float av = __bfloat162float(p.a[(size_t)(tc + tid) * p.ld_ba + hv]) + dtb;
      const float sp = av > 20.f ? av : log1pf(__expf(av));
      g = neg_a * sp;
      be = 1.f / (1.f + __expf(-__bfloat162float(p.b[(size_t)(tc + tid) * p.ld_ba + hv])));
    }
    s.G[tid] = g;
    s.beta[tid] = be;
  }
  __syncthreads();
  if (warp == 0) {  // inclusive scan of the 64 log-decays
    float x0 = s.G[lane], x1 = s.G[lane + 32];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float y0 = __shfl_up_sync(0xffffffffu, x0, o), y1 = __shfl_up_sync(0xffffffffu, x1, o);
      if (lane >= o) { x0 += y0; x1 += y1; }
    }
    x1 += __shfl_sync(0xffffffffu, x0, 31);
    s.G[lane] = x0;
    s.G[lane + 32] = x1;
  }
  // rows: L2-normalised q (with the output scale) and k as bf16 (warp w takes tokens w, w + 4, ...)
  for (int i = warp; i < C; i += 4) {
    float q4[4] = {0.f, 0.f, 0.f, 0.f}, k4[4] = {0.f, 0.f, 0.f, 0.f};
    if (i < n) {
      const size_t row = (size_t)(tc + i) * p.ld_qkv;
      const uint2 qr = *reinterpret_cast<const uint2*>(p.q + row + hk * D + lane * 4);
      const uint2 kr = *reinterpret_cast<const uint2*>(p.k + row + hk * D + lane * 4);
      const __nv_bfloat16* qp = reinterpret_cast<const __nv_bfloat16*>(&qr);
      const __nv_bfloat16* kp = reinterpret_cast<const __nv_bfloat16*>(&kr);
#pragma unroll
      for (int e = 0; e < 4; ++e) { q4[e] = __bfloat162float(qp[e]); k4[e] = __bfloat162float(kp[e]); }
    }
    float q2 = q4[0] * q4[0] + q4[1] * q4[1] + q4[2] * q4[2] + q4[3] * q4[3];
    float k2 = k4[0] * k4[0] + k4[1] * k4[1] + k4[2] * k4[2] + k4[3] * k4[3];
    q2 = warp_sum(q2);
    k2 = warp_sum(k2);
    const float qs = rsqrtf(q2 + 1e-6f) * scale, ks = rsqrtf(k2 + 1e-6f);
    *reinterpret_cast<uint2*>(&s.q[i][lane * 4]) = make_uint2(pack2(q4[0] * qs, q4[1] * qs), pack2(q4[2] * qs, q4[3] * qs));
    *reinterpret_cast<uint2*>(&s.k[i][lane * 4]) = make_uint2(pack2(k4[0] * ks, k4[1] * ks), pack2(k4[2] * ks, k4[3] * ks));
  }
  __syncthreads();
  __nv_bfloat16* ws = p.ws + ((size_t)ci * p.Hv + hv) * kWsPerHead;
  __nv_bfloat16* wsW = ws, *wsU = ws + kWsTile, *wsQ = ws + 2 * kWsTile, *wsK = ws + 3 * kWsTile, *wsP = ws + 4 * kWsTile;
  const int g = lane >> 2, t4 = lane & 3;
  const int m0 = warp * 16;
  const uint32_t sq = smem_u32(&s.q[0][0]), sk = smem_u32(&s.k[0][0]), sv = sq, st = smem_u32(&s.a[0][0]);
  {
    // K K^T and Q K^T for this warp's 16 rows (all 64 columns)
    float kk[8][4], qk[8][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) kk[nt][e] = qk[nt][e] = 0.f;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      uint32_t ak[4], aq[4];
      ldsm_x4(ak, a_addr(sk, P128, m0, ks * 16, lane));
      ldsm_x4(aq, a_addr(sq, P128, m0, ks * 16, lane));
#pragma unroll
      for (int np = 0; np < 4; ++np) {
        uint32_t b[4];
        ldsm_x4(b, bnk_addr(sk, P128, np * 16, ks * 16, lane));
        mma16816(kk[2 * np], ak, b[0], b[1]);
        mma16816(kk[2 * np + 1], ak, b[2], b[3]);
        mma16816(qk[2 * np], aq, b[0], b[1]);
        mma16816(qk[2 * np + 1], aq, b[2], b[3]);
      }
    }
    // A (fp32, shared) and P (bf16, workspace)
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int i = m0 + g + 8 * h;
        const float Gi = s.G[i], bi = s.beta[i];
        float pv[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int j = nt * 8 + t4 * 2 + e;
          const float gam = j <= i ? __expf(Gi - s.G[j]) : 0.f;
          s.a[i][j] = j < i ? bi * kk[nt][2 * h + e] * gam : 0.f;
          pv[e] = qk[nt][2 * h + e] * gam;
        }
        *reinterpret_cast<uint32_t*>(wsP + (size_t)i * C + nt * 8 + t4 * 2) = pack2(pv[0], pv[1]);
      }
  }
  __syncthreads();
  // Qg = e^G .* Q and Kd = e^{G_C - G} .* K go out now: the q tile's storage is reused for the triangular solve below
  for (int i = warp; i < C; i += 4) {
    const float eg = __expf(s.G[i]), ek = __expf(s.G[C - 1] - s.G[i]);
    const __nv_bfloat162* qp = reinterpret_cast<const __nv_bfloat162*>(&s.q[i][lane * 4]);
    const __nv_bfloat162* kp = reinterpret_cast<const __nv_bfloat162*>(&s.k[i][lane * 4]);
    const float2 q0 = __bfloat1622float2(qp[0]), q1 = __bfloat1622float2(qp[1]);
    const float2 k0 = __bfloat1622float2(kp[0]), k1 = __bfloat1622float2(kp[1]);
    *reinterpret_cast<uint2*>(wsQ + (size_t)i * D + lane * 4) = make_uint2(pack2(q0.x * eg, q0.y * eg), pack2(q1.x * eg, q1.y * eg));
    *reinterpret_cast<uint2*>(wsK + (size_t)i * D + lane * 4) = make_uint2(pack2(k0.x * ek, k0.y * ek), pack2(k1.x * ek, k1.y * ek));
  }
  __syncthreads();
  {
    // T = (I + A)^-1, blocked 4 x 4 in 16 x 16 blocks: the diagonal blocks by forward substitution (one column per thread, in
    // registers), then the block sub-diagonals d = 1, 2, 3 from  T_ij = -T_ii * sum_{j <= k < i} A_ik T_kj ; all in fp32
    float (*T)[C + 1] = reinterpret_cast<float (*)[C + 1]>(&s.q[0][0]);   // fp32 [64][65] over the q tile (16.6 KB <= 17 KB)
    float (*M)[16][17] = s.m;                                            // up to three 16 x 16 temporaries
    for (int e = tid; e < C * C; e += 128) T[e >> 6][e & 63] = 0.f;
    __syncthreads();
    if (tid < C) {
      const int b0 = (tid >> 4) * 16, c = tid & 15;
      float col[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        float acc = 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j)
          if (j < i) acc += s.a[b0 + i][b0 + j] * col[j];
        col[i] = i < c ? 0.f : (i == c ? 1.f : -acc);
      }
#pragma unroll
      for (int i = 0; i < 16; ++i) T[b0 + i][b0 + c] = col[i];
    }
    __syncthreads();
#pragma unroll 1
    for (int d = 1; d < 4; ++d) {
      const int nblk = 4 - d;
      for (int o = tid; o < nblk * 256; o += 128) {  // M = sum_k A_ik T_kj for block (i, j) = (blk + d, blk)
        const int blk = o >> 8, r = (o >> 4) & 15, c = o & 15;
        const int i0 = (blk + d) * 16, j0 = blk * 16;
        float acc = 0.f;
        for (int k = j0; k < i0; ++k) acc += s.a[i0 + r][k] * T[k][j0 + c];
        M[blk][r][c] = acc;
      }
      __syncthreads();
      for (int o = tid; o < nblk * 256; o += 128) {  // T_ij = -T_ii M
        const int blk = o >> 8, r = (o >> 4) & 15, c = o & 15;
        const int i0 = (blk + d) * 16, j0 = blk * 16;
        float acc = 0.f;
#pragma unroll
        for (int m = 0; m < 16; ++m) acc += T[i0 + r][i0 + m] * M[blk][m][c];
        T[i0 + r][j0 + c] = -acc;
      }
      __syncthreads();
    }
    // bf16 copy of T (the A operand of W and U) over the storage of A, which the solve no longer needs: every thread first reads
    // its share of T, then all of them write
    {
      __nv_bfloat16 (*Tb)[P64] = reinterpret_cast<__nv_bfloat16 (*)[P64]>(&s.a[0][0]);
      float tv[32];
#pragma unroll
      for (int e = 0; e < 32; ++e) {
        const int idx = tid + e * 128;
        tv[e] = T[idx >> 6][idx & 63];
      }
      __syncthreads();
#pragma unroll
      for (int e = 0; e < 32; ++e) {
        const int idx = tid + e * 128;
        Tb[idx >> 6][idx & 63] = __float2bfloat16(tv[e]);
      }
    }
    // B operands: k rows scaled by beta e^G in place; v rows scaled by beta, loaded now into the storage T has left
    for (int i = warp; i < C; i += 4) {
      const float bk = s.beta[i] * __expf(s.G[i]), bv = s.beta[i];
      __nv_bfloat162* kp = reinterpret_cast<__nv_bfloat162*>(&s.k[i][lane * 4]);
      float v4[4] = {0.f, 0.f, 0.f, 0.f};
      if (i < n) {
        const uint2 vr = *reinterpret_cast<const uint2*>(p.v + (size_t)(tc + i) * p.ld_qkv + hv * D + lane * 4);
        const __nv_bfloat16* vp = reinterpret_cast<const __nv_bfloat16*>(&vr);
#pragma unroll
        for (int e = 0; e < 4; ++e) v4[e] = __bfloat162float(vp[e]);
      }
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const float2 kf = __bfloat1622float2(kp[e]);
        kp[e] = __floats2bfloat162_rn(kf.x * bk, kf.y * bk);
      }
      *reinterpret_cast<uint2*>(&s.q[i][lane * 4]) = make_uint2(pack2(v4[0] * bv, v4[1] * bv), pack2(v4[2] * bv, v4[3] * bv));
    }
  }
  __syncthreads();
  // W = T (b e^G K), U = T (b V): this warp's 16 rows, 128 columns in two halves
#pragma unroll 1
  for (int which = 0; which < 2; ++which) {
    const uint32_t sb = which == 0 ? sk : sv;
    __nv_bfloat16* dst = which == 0 ? wsW : wsU;
#pragma unroll 1
    for (int nh = 0; nh < 2; ++nh) {
      float acc[8][4];
#pragma unroll
      for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[nt][e] = 0.f;
#pragma unroll
      for (int ks = 0; ks < C / 16; ++ks) {
        uint32_t a[4];
        ldsm_x4(a, a_addr(st, P64, m0, ks * 16, lane));
#pragma unroll
        for (int np = 0; np < 4; ++np) {
          uint32_t b[4];
          ldsm_x4_t(b, bkn_addr(sb, P128, ks * 16, nh * 64 + np * 16, lane));
          mma16816(acc[2 * np], a, b[0], b[1]);
          mma16816(acc[2 * np + 1], a, b[2], b[3]);
        }
      }
#pragma unroll
      for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int h = 0; h < 2; ++h)
          *reinterpret_cast<uint32_t*>(dst + (size_t)(m0 + g + 8 * h) * D + nh * 64 + nt * 8 + t4 * 2) = pack2(acc[nt][2 * h], acc[nt][2 * h + 1]);
    }
  }
  if (tid == 0) *reinterpret_cast<float*>(ws + 4 * kWsTile + (size_t)C * C) = __expf(s.G[C - 1]);
}

// ---------------------------------------------------------------------------------------------------------------- kernel B
// grid (long sequences, Hv, 2 column halves), 256 threads. The state slice [128][64] is fp32 in MMA accumulator layout: warp w
// owns rows 16w .. 16w + 15.
struct SmemBuf {
  __nv_bfloat16 w[C][P128], q[C][P128], k[C][P128];
  __nv_bfloat16 u[C][P64], p[C][P64];
};
struct SmemB {
  SmemBuf buf[2];
  __nv_bfloat16 s[D][P64];   // bf16 copy of the state slice: B operand [k = key dim][n = column]
  __nv_bfloat16 vn[C][P64];  // Vnew: B operand [k = token][n = column]
  float gc[2];
};

__global__ void __launch_bounds__(256) gdn_chunk_scan_kernel(const GdnChunkParams p) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  SmemB& s = *reinterpret_cast<SmemB*>(smem_raw);
  const int li = blockIdx.x, hv = blockIdx.y, half = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t4 = lane & 3;
  const int r = p.long_req[li];
  const int t0 = p.query_start_loc[r], t1 = p.query_start_loc[r + 1];
  const int nchunks = (t1 - t0 + C - 1) / C;
  const int cbase = p.long_chunk0[li];
  const int slot = p.state_slots[r];
  float* Sg = p.state + ((size_t)slot * p.Hv + hv) * D * D + half * 64;
  // state rows 16 warp + g (+8), columns nt * 8 + 2 t4 (+1)
  float S[8][4];
  if (p.has_initial_state[r]) {
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const float2 x = *reinterpret_cast<const float2*>(Sg + (size_t)(warp * 16 + g + 8 * h) * D + nt * 8 + t4 * 2);
        S[nt][2 * h] = x.x;
        S[nt][2 * h + 1] = x.y;
      }
  } else {
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) S[nt][e] = 0.f;
  }
  auto fetch = [&](int c, int b) {
    const __nv_bfloat16* ws = p.ws + ((size_t)(cbase + c) * p.Hv + hv) * kWsPerHead;
    SmemBuf& d = s.buf[b];
    // three [64][128] tiles: 16 x 16-byte segments per row
    for (int e = tid; e < 3 * C * 16; e += 256) {
      const int which = e / (C * 16), rem = e - which * (C * 16), row = rem >> 4, seg = rem & 15;
      const __nv_bfloat16* src = ws + (which == 0 ? 0 : which == 1 ? 2 * kWsTile : 3 * kWsTile) + (size_t)row * D + seg * 8;
      __nv_bfloat16* dst = which == 0 ? &d.w[row][seg * 8] : which == 1 ? &d.q[row][seg * 8] : &d.k[row][seg * 8];
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
    }
    // this half of U, and P: [64][64] tiles, 8 segments per row
    for (int e = tid; e < 2 * C * 8; e += 256) {
      const int which = e / (C * 8), rem = e - which * (C * 8), row = rem >> 3, seg = rem & 7;
      const __nv_bfloat16* src = which == 0 ? ws + kWsTile + (size_t)row * D + half * 64 + seg * 8 : ws + 4 * kWsTile + (size_t)row * C + seg * 8;
      __nv_bfloat16* dst = which == 0 ? &d.u[row][seg * 8] : &d.p[row][seg * 8];
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
    }
    if (tid == 0) s.gc[b] = *reinterpret_cast<const float*>(ws + 4 * kWsTile + (size_t)C * C);
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  fetch(0, 0);
  const int mt = warp & 3, nh = warp >> 2;  // token tile and column half of this warp in the token-major products
  const uint32_t ss = smem_u32(&s.s[0][0]), svn = smem_u32(&s.vn[0][0]);
  for (int c = 0; c < nchunks; ++c) {
    const int b = c & 1;
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    // publish the state as a bf16 B operand
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int h = 0; h < 2; ++h)
        *reinterpret_cast<uint32_t*>(&s.s[warp * 16 + g + 8 * h][nt * 8 + t4 * 2]) = pack2(S[nt][2 * h], S[nt][2 * h + 1]);
    __syncthreads();  // chunk c has landed for every thread; the state copy is complete; buffer b ^ 1 is free
    if (c + 1 < nchunks) fetch(c + 1, b ^ 1);
    const SmemBuf& d = s.buf[b];
    const uint32_t sw = smem_u32(&d.w[0][0]), sq = smem_u32(&d.q[0][0]), sk = smem_u32(&d.k[0][0]), sp = smem_u32(&d.p[0][0]);
    // ---- Vnew = U - W S0  (tokens 16 mt .., columns 32 nh ..)
    float acc[4][4];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[nt][e] = 0.f;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      uint32_t a[4];
      ldsm_x4(a, a_addr(sw, P128, mt * 16, ks * 16, lane));
#pragma unroll
      for (int np = 0; np < 2; ++np) {
        uint32_t bb[4];
        ldsm_x4_t(bb, bkn_addr(ss, P64, ks * 16, nh * 32 + np * 16, lane));
        mma16816(acc[2 * np], a, bb[0], bb[1]);
        mma16816(acc[2 * np + 1], a, bb[2], bb[3]);
      }
    }
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int i = mt * 16 + g + 8 * h, col = nh * 32 + nt * 8 + t4 * 2;
        const float2 u = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&d.u[i][col]));
        *reinterpret_cast<uint32_t*>(&s.vn[i][col]) = pack2(u.x - acc[nt][2 * h], u.y - acc[nt][2 * h + 1]);
      }
    __syncthreads();  // Vnew is complete
    // ---- O = Qg S0 + P Vnew
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[nt][e] = 0.f;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      uint32_t a[4];
      ldsm_x4(a, a_addr(sq, P128, mt * 16, ks * 16, lane));
#pragma unroll
      for (int np = 0; np < 2; ++np) {
        uint32_t bb[4];
        ldsm_x4_t(bb, bkn_addr(ss, P64, ks * 16, nh * 32 + np * 16, lane));
        mma16816(acc[2 * np], a, bb[0], bb[1]);
        mma16816(acc[2 * np + 1], a, bb[2], bb[3]);
      }
    }
#pragma unroll
    for (int ks = 0; ks < C / 16; ++ks) {
      uint32_t a[4];
      ldsm_x4(a, a_addr(sp, P64, mt * 16, ks * 16, lane));
#pragma unroll
      for (int np = 0; np < 2; ++np) {
        uint32_t bb[4];
        ldsm_x4_t(bb, bkn_addr(svn, P64, ks * 16, nh * 32 + np * 16, lane));
        mma16816(acc[2 * np], a, bb[0], bb[1]);
        mma16816(acc[2 * np + 1], a, bb[2], bb[3]);
      }
    }
    {
      const int tbase = t0 + c * C;
#pragma unroll
      for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int t = tbase + mt * 16 + g + 8 * h;
          if (t < t1)
            *reinterpret_cast<uint32_t*>(p.out + (size_t)t * p.Hv * D + hv * D + half * 64 + nh * 32 + nt * 8 + t4 * 2) =
                pack2(acc[nt][2 * h], acc[nt][2 * h + 1]);
        }
    }
    // ---- S = e^{G_C} S + Kd^T Vnew  (state rows 16 warp .., all 64 columns of the half)
    {
      const float gc = s.gc[b];
#pragma unroll
      for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) S[nt][e] *= gc;
#pragma unroll
      for (int ks = 0; ks < C / 16; ++ks) {
        uint32_t a[4];
        ldsm_x4_t(a, at_addr(sk, P128, warp * 16, ks * 16, lane));
#pragma unroll
        for (int np = 0; np < 4; ++np) {
          uint32_t bb[4];
          ldsm_x4_t(bb, bkn_addr(svn, P64, ks * 16, np * 16, lane));
          mma16816(S[2 * np], a, bb[0], bb[1]);
          mma16816(S[2 * np + 1], a, bb[2], bb[3]);
        }
      }
    }
    __syncthreads();  // every warp is done with the state copy, Vnew and buffer b before the next round rewrites them
  }
  if (p.write_state) {
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int h = 0; h < 2; ++h)
        *reinterpret_cast<float2*>(Sg + (size_t)(warp * 16 + g + 8 * h) * D + nt * 8 + t4 * 2) = make_float2(S[nt][2 * h], S[nt][2 * h + 1]);
  }
}

}  // namespace

size_t gdn_chunk_workspace_elems(int num_chunks, int Hv) { return (size_t)num_chunks * Hv * kWsPerHead; }

int gdn_chunk_launch(const GdnChunkParams& p, cudaStream_t st) {
  if (p.num_chunks == 0 || p.num_long == 0) return 0;
  if (p.K != D || p.V != D || p.Hv % p.Hk || (p.ld_qkv % 4) != 0) return -1;
  static bool configured_dev[kMaxDevices] = {};
  bool& configured = configured_dev[current_device_slot()];
  if (!configured) {
    if (cudaFuncSetAttribute(gdn_chunk_prepare_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(SmemA)) != cudaSuccess) return -4;
    if (cudaFuncSetAttribute(gdn_chunk_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(SmemB)) != cudaSuccess) return -4;
    configured = true;
  }
  gdn_chunk_prepare_kernel<<<dim3(p.num_chunks, p.Hv), 128, sizeof(SmemA), st>>>(p);
  gdn_chunk_scan_kernel<<<dim3(p.num_long, p.Hv, 2), 256, sizeof(SmemB), st>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

}  // namespace oc
