// Multi-head latent attention decode (DeepSeek-V2/V3): multi-query attention over the paged latent cache, with W_UK already
// folded into the query ("absorbed" form) and W_UV applied by the caller to the result.
//   scores = [q_nope_abs | q_rope] . [latent | k_rope]^T   (576 = 512 + 64 wide)       out = softmax(scores) . latent   (512 wide)
// All heads of a token share the same keys, so heads are the rows of the tile: a CTA owns 16 (head, query-token) rows of one request
// and one split of its context. Its four warps each compute the full 16 x 64 score tile (cheap next to the memory traffic) but own
// a different 128-column slice of the 512-wide output, so the accumulator stays in registers. The key tile is loaded once into
// shared memory and serves as K (all 576 columns) and as V (first 512): the latent is read from HBM exactly once per CTA.
// Split-KV partials are merged by mla_combine_kernel. bf16 mma.sync.m16n8k16, fp32 softmax state in the exp2 domain.
// (reference: csrc/attention/mla/sm100_cutlass_mla_kernel.cu; csrc/cpu/mla_decode.cpp; layers/attention/mla_attention.py forward_mqa)
#include "common.cuh"
#include "kernels.h"

namespace oc {
namespace {

constexpr int DK = 576, DV = 512, KEYS = 64, ROWS = 16;
constexpr int CHK = DK / 8;  // 72 16-byte chunks per key row

__device__ __forceinline__ void cp16(void* smem, const void* g) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem)), "l"(g) : "memory");
}
__device__ __forceinline__ void ldsm4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm4t(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pk(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
// rows are 1152 bytes (72 chunks); XOR the low 3 chunk bits with the row to spread ldmatrix over the banks
__device__ __forceinline__ uint32_t koff(int row, int chunk) { return (uint32_t)(row * DK * 2 + (((chunk & ~7) | ((chunk ^ row) & 7)) << 4)); }

__global__ void __launch_bounds__(128) mla_decode_kernel(const MlaParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* sQ = smem;                        // [16][576]
  uint8_t* sK = sQ + ROWS * DK * 2;          // [2][64][576]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g_ = lane >> 2, tg = lane & 3;
  const int r = blockIdx.x, rt = blockIdx.y, split = blockIdx.z;
  const int qs = p.query_start_loc[r], qlen = p.query_start_loc[r + 1] - qs, S = p.seq_lens[r];
  if (qlen <= 0 || S <= 0) return;
  const int total_rows = qlen * p.H;         // row = token * H + head
  const int row0 = rt * ROWS;
  if (row0 >= total_rows) return;
  const int nrows = min(ROWS, total_rows - row0);
  const int ctx0 = S - qlen;
  const int last_tok = (row0 + nrows - 1) / p.H;
  const int kv_end = min(S, ctx0 + last_tok + 1);
  const int ntiles = (kv_end + KEYS - 1) / KEYS;
  int lo = 0, hi = ntiles;
  if (p.splits > 1) {
    const int per = (ntiles + p.splits - 1) / p.splits;
    lo = split * per;
    hi = min(ntiles, lo + per);
  }
  const int* bt = p.block_table + (size_t)r * p.bt_stride;
  // Q rows: [q_abs (512) | q_rope (64)]
  for (int idx = threadIdx.x; idx < ROWS * CHK; idx += 128) {
    const int row = idx / CHK, ch = idx % CHK;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (row < nrows) {
      const int gr = row0 + row, tok = gr / p.H, hd = gr % p.H;
      const __nv_bfloat16* src = ch < 64 ? p.q_abs + ((size_t)(qs + tok) * p.H + hd) * DV + ch * 8
                                         : p.q_rope + ((size_t)(qs + tok) * p.H + hd) * 64 + (ch - 64) * 8;
      v = *reinterpret_cast<const uint4*>(src);
    }
    *reinterpret_cast<uint4*>(sQ + koff(row, ch)) = v;
  }
  auto load_tile = [&](int tile, int buf) {
    uint8_t* dk = sK + (size_t)buf * KEYS * DK * 2;
    for (int idx = threadIdx.x; idx < KEYS * CHK; idx += 128) {
      const int row = idx / CHK, ch = idx % CHK, key = tile * KEYS + row;
      if (key < kv_end) {
        const int blk = bt[key >> p.bs_shift];
        cp16(dk + koff(row, ch), p.cache + ((size_t)blk * p.bs + (key & (p.bs - 1))) * DK + ch * 8);
      } else {
        *reinterpret_cast<uint4*>(dk + koff(row, ch)) = make_uint4(0, 0, 0, 0);
      }
    }
  };
  float o[16][4];  // this warp's 128 output columns: 16 n-blocks of 8
#pragma unroll
  for (int i = 0; i < 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m2[2] = {-INFINITY, -INFINITY}, l2[2] = {0.f, 0.f};
  const float sc = p.scale * 1.4426950408889634f;
  if (lo < hi) load_tile(lo, 0);
  asm volatile("cp.async.commit_group;" ::: "memory");
  for (int tile = lo; tile < hi; ++tile) {
    const int buf = (tile - lo) & 1;
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    if (tile + 1 < hi) load_tile(tile + 1, buf ^ 1);
    asm volatile("cp.async.commit_group;" ::: "memory");
    const uint32_t kb = smem_u32(sK + (size_t)buf * KEYS * DK * 2), qb = smem_u32(sQ);
    float s[8][4];
#pragma unroll
    for (int n = 0; n < 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
    for (int kk = 0; kk < DK / 16; ++kk) {
      uint32_t a[4];
      ldsm4(a, qb + koff(lane & 15, kk * 2 + (lane >> 4)));
#pragma unroll
      for (int n2 = 0; n2 < 4; ++n2) {
        uint32_t b[4];
        ldsm4(b, kb + koff(n2 * 16 + (lane & 7) + ((lane >> 4) << 3), kk * 2 + ((lane >> 3) & 1)));
        mma16816(s[n2 * 2], a, b[0], b[1]);
        mma16816(s[n2 * 2 + 1], a, b[2], b[3]);
      }
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int gr = row0 + g_ + h * 8;
      const int qpos = ctx0 + gr / p.H;
      float mx = -INFINITY;
#pragma unroll
      for (int n = 0; n < 8; ++n)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int key = tile * KEYS + n * 8 + tg * 2 + e;
          float v = s[n][h * 2 + e] * sc;
          v = (key <= qpos && key < kv_end) ? v : -INFINITY;
          s[n][h * 2 + e] = v;
          mx = fmaxf(mx, v);
        }
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float mn = fmaxf(m2[h], mx), mu = (mn == -INFINITY) ? 0.f : mn;
      const float alpha = exp2f(m2[h] - mu);
      float sum = 0.f;
#pragma unroll
      for (int n = 0; n < 8; ++n)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const float pv = exp2f(s[n][h * 2 + e] - mu);
          s[n][h * 2 + e] = pv;
          sum += pv;
        }
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      l2[h] = l2[h] * alpha + sum;
      m2[h] = mn;
#pragma unroll
      for (int i = 0; i < 16; ++i) { o[i][h * 2] *= alpha; o[i][h * 2 + 1] *= alpha; }
    }
    // O[:, warp*128 .. +128) += P . latent[:, that slice]
#pragma unroll
    for (int n2 = 0; n2 < 4; ++n2) {
      uint32_t a[4] = {pk(s[n2 * 2][0], s[n2 * 2][1]), pk(s[n2 * 2][2], s[n2 * 2][3]), pk(s[n2 * 2 + 1][0], s[n2 * 2 + 1][1]), pk(s[n2 * 2 + 1][2], s[n2 * 2 + 1][3])};
#pragma unroll
      for (int d2 = 0; d2 < 8; ++d2) {
        uint32_t b[4];
        ldsm4t(b, kb + koff(n2 * 16 + (lane & 15), warp * 16 + d2 * 2 + (lane >> 4)));
        mma16816(o[d2 * 2], a, b[0], b[1]);
        mma16816(o[d2 * 2 + 1], a, b[2], b[3]);
      }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int row = g_ + h * 8;
    if (row >= nrows) continue;
    const int gr = row0 + row, tok = gr / p.H, hd = gr % p.H;
    const size_t orow = (size_t)(qs + tok) * p.H + hd;
    if (p.splits > 1) {
      float* wo = p.ws_o + ((size_t)split * p.T * p.H + orow) * DV + warp * 128;
#pragma unroll
      for (int i = 0; i < 16; ++i) *reinterpret_cast<float2*>(wo + i * 8 + tg * 2) = make_float2(o[i][h * 2], o[i][h * 2 + 1]);
      if (warp == 0 && tg == 0) {
        float* wm = p.ws_ml + ((size_t)split * p.T * p.H + orow) * 2;
        wm[0] = m2[h];
        wm[1] = l2[h];
      }
    } else {
      const float inv = l2[h] > 0.f ? 1.f / l2[h] : 0.f;
      __nv_bfloat16* dst = p.out + orow * DV + warp * 128;
#pragma unroll
      for (int i = 0; i < 16; ++i) *reinterpret_cast<uint32_t*>(dst + i * 8 + tg * 2) = pk(o[i][h * 2] * inv, o[i][h * 2 + 1] * inv);
    }
  }
}

__global__ void mla_combine_kernel(const MlaParams p) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int rows = p.T * p.H;
  if (warp >= rows) return;
  float M = -INFINITY;
  for (int s = 0; s < p.splits; ++s) M = fmaxf(M, p.ws_ml[((size_t)s * rows + warp) * 2]);
  float L = 0.f, acc[DV / 32];
#pragma unroll
  for (int i = 0; i < DV / 32; ++i) acc[i] = 0.f;
  for (int s = 0; s < p.splits; ++s) {
    const float ms = p.ws_ml[((size_t)s * rows + warp) * 2];
    const float f = (ms == -INFINITY) ? 0.f : exp2f(ms - M);
    L += p.ws_ml[((size_t)s * rows + warp) * 2 + 1] * f;
    const float* src = p.ws_o + ((size_t)s * rows + warp) * DV;
#pragma unroll
    for (int i = 0; i < DV / 32; ++i) acc[i] += src[lane + 32 * i] * f;
  }
  const float inv = L > 0.f ? 1.f / L : 0.f;
#pragma unroll
  for (int i = 0; i < DV / 32; ++i) p.out[(size_t)warp * DV + lane + 32 * i] = __float2bfloat16(acc[i] * inv);
}

}  // namespace

int mla_decode_launch(const MlaParams& p, cudaStream_t st) {
  if (p.R == 0 || p.T == 0) return 0;
  if (p.kv_lora != DV || p.rope != 64 || p.bs < 16 || (p.bs & (p.bs - 1))) return -1;
  const int smem = ROWS * DK * 2 + 2 * KEYS * DK * 2;
  static bool configured_dev[kMaxDevices] = {};
  bool& configured = configured_dev[current_device_slot()];  // the limit is an attribute of (kernel, device)
  if (!configured) {
    if (cudaFuncSetAttribute(mla_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -4;
    configured = true;
  }
  const int row_tiles = (p.max_q_len * p.H + ROWS - 1) / ROWS;
  dim3 grid(p.R, row_tiles, p.splits);
  mla_decode_kernel<<<grid, 128, smem, st>>>(p);
  if (p.splits > 1) mla_combine_kernel<<<(p.T * p.H * 32 + 255) / 256, 256, 0, st>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

unsigned int mla_read_status(bool clear) { return read_status_tu(clear); }
void mla_read_status_async(unsigned int* dst, cudaStream_t st) { read_status_tu_async(dst, st); }

}  // namespace oc
