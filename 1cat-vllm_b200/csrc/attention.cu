// Paged-KV flash attention for head sizes 64, 128 and 256: causal, GQA-packed, variable-length batches where each
// request's queries are the last rows of its context (so decode, multi-token verify and chunked prefill over a cached
// prefix are one kernel family).
//   mode 0 (prefill): a CTA owns a tile of 64 (token, q-head-in-group) rows of one KV head; its 4 warps own 16 rows each
//                     and stream 64-key tiles of K and V through double-buffered shared memory.
//   mode 1 (decode / verify): rows fit in 16 or 32; the 4 warps split each 64-key tile by keys, grid.z splits the context
//                     (split-KV), partial (max, sum, O) are merged across warps in shared memory and across splits by a
//                     second small kernel.
// K/V pages are [block][2][Hkv][block_size][D] so one (page, head) is contiguous. Tensor-core math is bf16
// mma.sync.m16n8k16 with fp32 accumulation (softmax in the exp2 domain).
// Options for the Gemma / GPT-OSS / Mistral families: a sliding window (a query at position i sees keys i-window+1 .. i; key tiles
// wholly before the window are skipped), tanh soft-capping of the scaled scores, and per-head attention sinks (a learned logit that
// joins the softmax denominator only).
// FP8 KV cache (KV8): pages hold e4m3 bytes in the same layout; tiles stream through a byte-wide cp.async ring and are widened to
// bf16 into one working tile per operand before the MMAs; the per-tensor scales fold into the softmax scale (K) and the output (V).
// (reference: flash-attention-v100/kernel/fused_mha_forward_paged.cu:364, flash_decode_paged.cu:667,831,1301;
//  v1/attention/backends/flash_attn_v100.py:2216 for the math)
#include <cuda_fp8.h>
#include <stdlib.h>

#include "common.cuh"
#include "kernels.h"

namespace oc {
namespace {

constexpr int kKeysPerTile = 64;

__device__ __forceinline__ void cp_async16(void* smem, const void* g) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem)), "l"(g) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
// byte offset of the 16-byte chunk `chunk` of row `row` in a [rows][D] bf16 tile with XOR swizzle
template <int D>
__device__ __forceinline__ uint32_t sw_off(int row, int chunk) {
  return (uint32_t)(row * D * 2 + ((chunk ^ (row & 7)) << 4));
}

// 16 e4m3 bytes -> 16 bf16, exactly (every e4m3 value is a bf16 value). A byte's sign goes to bit 15 and its exponent and mantissa
// four places below the top of the bf16 exponent field, which reads as value * 2^-120 (e4m3 subnormals become bf16 subnormals);
// one bf16x2 multiply by 2^120 restores the value.
__device__ __forceinline__ uint32_t widen_fp8_pair(uint32_t w, uint32_t sel) {
  uint32_t t;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(t) : "r"(w), "r"(0u), "r"(sel));
  uint32_t v = (t & 0x80008000u) | ((t >> 4) & 0x07f007f0u);
  const uint32_t two120 = 0x7b807b80u;
  __nv_bfloat162 r = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&v), *reinterpret_cast<const __nv_bfloat162*>(&two120));
  return *reinterpret_cast<uint32_t*>(&r);
}
__device__ __forceinline__ void widen_fp8x16(const uint4& in, uint4& lo, uint4& hi) {
  lo = make_uint4(widen_fp8_pair(in.x, 0x1404u), widen_fp8_pair(in.x, 0x3424u), widen_fp8_pair(in.y, 0x1404u), widen_fp8_pair(in.y, 0x3424u));
  hi = make_uint4(widen_fp8_pair(in.z, 0x1404u), widen_fp8_pair(in.z, 0x3424u), widen_fp8_pair(in.w, 0x1404u), widen_fp8_pair(in.w, 0x3424u));
}

template <int D, int MODE, int MB, bool KV8, int ST = 3>
__global__ void __launch_bounds__(128) attn_kernel(const AttnParams p) {
  pdl_trigger();
  pdl_wait();
  constexpr int STAGES = ST;                    // K/V tiles in the cp.async ring (a fourth stage of byte tiles measured no faster)
  constexpr int MBW = (MODE == 0) ? 1 : MB;     // 16-row blocks per warp
  constexpr int NB2 = (MODE == 0) ? 4 : 1;      // 16-key groups per warp per tile
  constexpr int ROWS = (MODE == 0) ? 64 : 16 * MB;
  constexpr int CH = D / 8;                     // 16-byte chunks per row
  extern __shared__ __align__(128) uint8_t smem[];
  // bf16 cache: sK / sV are the cp.async rings of bf16 tiles. fp8 cache: they are rings of byte tiles, followed by one bf16
  // working tile per operand (sKb / sVb)
  constexpr int ESZ = KV8 ? 1 : 2;
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + ROWS * D * 2;
  uint8_t* sV = sK + STAGES * kKeysPerTile * D * ESZ;
  uint8_t* sKb = sV + STAGES * kKeysPerTile * D * ESZ;
  uint8_t* sVb = sKb + kKeysPerTile * D * 2;
  __shared__ int s_req, s_tile0;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = p.Hq / p.Hkv;
  const int hkv = blockIdx.y;
  int r, tq0, tq1;
  if (MODE == 0) {
    const int TQ = 64 / G;
    if (threadIdx.x == 0) {
      int b = blockIdx.x, found = -1, t0 = 0;
      for (int i = 0; i < p.R; ++i) {
        int ql = p.query_start_loc[i + 1] - p.query_start_loc[i];
        int nt = (ql > p.short_q_len) ? (ql + TQ - 1) / TQ : 0;  // short queries belong to the decode kernel
        if (b < nt) { found = i; t0 = b * TQ; break; }
        b -= nt;
      }
      s_req = found;
      s_tile0 = t0;
    }
    __syncthreads();
    r = s_req;
    if (r < 0) return;
    tq0 = s_tile0;
    int ql = p.query_start_loc[r + 1] - p.query_start_loc[r];
    tq1 = min(tq0 + TQ, ql);
  } else {
    r = blockIdx.x;
    tq0 = 0;
    tq1 = p.query_start_loc[r + 1] - p.query_start_loc[r];
    if (tq1 > p.short_q_len) return;  // long queries belong to the prefill kernel (uniform exit: before any barrier)
  }
  const int qs = p.query_start_loc[r];
  const int qlen = p.query_start_loc[r + 1] - qs;
  const int S = p.seq_lens[r];
  if (qlen <= 0 || S <= 0) return;
  const int ctx0 = S - qlen;
  const int nrows = (tq1 - tq0) * G;
  const int kv_end = min(S, ctx0 + tq1);
  const int ntiles = (kv_end + kKeysPerTile - 1) / kKeysPerTile;
  // sliding window: the first row of the tile sees the earliest key, ctx0 + tq0 - window + 1
  const int wlo = p.window > 0 ? p.window : 0x3fffffff;
  const int tile_first = p.window > 0 ? max(0, ctx0 + tq0 - p.window + 1) / kKeysPerTile : 0;
  int tile_lo = tile_first, tile_hi = ntiles;
  if (MODE == 1 && p.splits > 1) {
    int per = (ntiles - tile_first + p.splits - 1) / p.splits;
    tile_lo = tile_first + blockIdx.z * per;
    tile_hi = min(ntiles, tile_lo + per);
  }
  const int* bt = p.block_table + (size_t)r * p.bt_stride;
  const size_t page_elems = (size_t)p.bs * D;

  // each thread always copies the same 16-byte column chunk of rows (tid / CH) + i * (128 / CH); pages are a power of
  // two tokens long, so the block-table lookup is a shift and a mask
  constexpr int LCH = KV8 ? D / 16 : CH;        // 16-byte chunks per cache row
  const int ld_ch = threadIdx.x % LCH, ld_row0 = threadIdx.x / LCH;
  constexpr int kRowStep = 128 / LCH;
  const int bs_shift = p.bs_shift, bs_mask = p.bs - 1;
  // byte addressing covers both element sizes
  const uint8_t* kv_head = reinterpret_cast<const uint8_t*>(p.kv_cache) + ((size_t)hkv * page_elems) * ESZ + ld_ch * 16;
  const size_t blk_stride = (size_t)2 * p.Hkv * page_elems * ESZ, v_off = (size_t)p.Hkv * page_elems * ESZ;
  // One block-table lookup per 16-key chunk of the tile: pages are at least 16 keys long and tiles start at multiples of 64, so
  // the 16 / kRowStep rows that a thread copies inside a chunk share a page.
  auto load_tile = [&](int tile, int buf) {
    const int k0 = tile * kKeysPerTile;
    uint8_t* dk = sK + (size_t)buf * kKeysPerTile * D * ESZ;
    uint8_t* dv = sV + (size_t)buf * kKeysPerTile * D * ESZ;
    if constexpr (kRowStep <= 16) {
      constexpr int RPC = 16 / kRowStep;
#pragma unroll
      for (int c = 0; c < kKeysPerTile / 16; ++c) {
        const int key_c = k0 + c * 16;
        const uint8_t* src = kv_head;
        if (key_c < kv_end) src += (size_t)bt[key_c >> bs_shift] * blk_stride + (size_t)((key_c & bs_mask) + ld_row0) * (D * ESZ);
#pragma unroll
        for (int j = 0; j < RPC; ++j) {
          const int row = c * 16 + ld_row0 + j * kRowStep;
          const uint32_t off = KV8 ? (uint32_t)(row * D + ld_ch * 16) : sw_off<D>(row, ld_ch);
          if (k0 + row < kv_end) {
            cp_async16(dk + off, src + (size_t)j * (kRowStep * D * ESZ));
            cp_async16(dv + off, src + (size_t)j * (kRowStep * D * ESZ) + v_off);
          } else {
            *reinterpret_cast<uint4*>(dk + off) = make_uint4(0, 0, 0, 0);
            *reinterpret_cast<uint4*>(dv + off) = make_uint4(0, 0, 0, 0);
          }
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < kKeysPerTile / kRowStep; ++i) {
        const int row = ld_row0 + i * kRowStep;
        const int key = k0 + row;
        const uint32_t off = KV8 ? (uint32_t)(row * D + ld_ch * 16) : sw_off<D>(row, ld_ch);
        if (key < kv_end) {
          const int blk = bt[key >> bs_shift];
          const uint8_t* src = kv_head + (size_t)blk * blk_stride + (size_t)(key & bs_mask) * D * ESZ;
          cp_async16(dk + off, src);
          cp_async16(dv + off, src + v_off);
        } else {
          *reinterpret_cast<uint4*>(dk + off) = make_uint4(0, 0, 0, 0);
          *reinterpret_cast<uint4*>(dv + off) = make_uint4(0, 0, 0, 0);
        }
      }
    }
  };

  // Decode: the four warps see disjoint keys, so each warp streams its own 16 keys of every tile through its own cp.async groups
  // (and widens its own e4m3 bytes) and the main loop needs no CTA-wide barrier: the warps drift apart and hide one another's
  // latencies (measured in lock step, a CTA took 1.9 us per tile, a dependent chain of copy wait, barrier, QK, softmax, PV).
  constexpr bool WARP_PIPE = (MODE == 1);
  constexpr int WCH = KV8 ? D / 16 : CH;        // 16-byte chunks per cache row
  const uint8_t* kv_warp = reinterpret_cast<const uint8_t*>(p.kv_cache) + ((size_t)hkv * page_elems) * ESZ;
  auto load_tile_w = [&](int tile, int buf) {
    const int key0 = tile * kKeysPerTile + warp * 16;
    uint8_t* dk = sK + (size_t)buf * kKeysPerTile * D * ESZ;
    uint8_t* dv = sV + (size_t)buf * kKeysPerTile * D * ESZ;
    const uint8_t* src = kv_warp;
    if (key0 < kv_end) src += (size_t)bt[key0 >> bs_shift] * blk_stride + (size_t)(key0 & bs_mask) * (D * ESZ);
#pragma unroll
    for (int i = 0; i < 16 * WCH / 32; ++i) {
      const int idx = lane + 32 * i, rl = idx / WCH, ch = idx % WCH;
      const uint32_t off = KV8 ? (uint32_t)((warp * 16 + rl) * D + ch * 16) : sw_off<D>(warp * 16 + rl, ch);
      if (key0 + rl < kv_end) {
        cp_async16(dk + off, src + (size_t)rl * (D * ESZ) + ch * 16);
        cp_async16(dv + off, src + (size_t)rl * (D * ESZ) + ch * 16 + v_off);
      } else {
        *reinterpret_cast<uint4*>(dk + off) = make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4*>(dv + off) = make_uint4(0, 0, 0, 0);
      }
    }
  };

  float o[MBW][D / 8][4];
  float mrow[MBW][2], lrow[MBW][2];
#pragma unroll
  for (int b = 0; b < MBW; ++b) {
    mrow[b][0] = mrow[b][1] = -INFINITY;
    lrow[b][0] = lrow[b][1] = 0.f;
#pragma unroll
    for (int i = 0; i < D / 8; ++i) o[b][i][0] = o[b][i][1] = o[b][i][2] = o[b][i][3] = 0.f;
  }
  // plain: s * scale * log2(e); soft-capped: cap * tanh(s * scale / cap) * log2(e)
  const bool capped = p.softcap > 0.f;
  const float qk_scale = KV8 ? p.scale * p.k_scale : p.scale;   // K was stored as k / k_scale
  const float sc = capped ? qk_scale / p.softcap : qk_scale * 1.4426950408889634f;
  const float sc_post = p.softcap * 1.4426950408889634f;
  const int row_base = (MODE == 0) ? warp * 16 : 0;
  const int key_base = (MODE == 0) ? 0 : warp * 16;
  const int g_ = lane >> 2, tg = lane & 3;

#pragma unroll
  for (int i = 0; i < STAGES - 1; ++i) {
    if (tile_lo + i < tile_hi) {
      if constexpr (WARP_PIPE) load_tile_w(tile_lo + i, i);
      else load_tile(tile_lo + i, i);
    }
    cp_async_commit();
  }
  // ---- Q tile -> shared memory (zero rows past the end), behind the first K/V copies so that its latency overlaps theirs; the
  // first barrier of the loop publishes it
  for (int idx = threadIdx.x; idx < ROWS * CH; idx += 128) {
    int row = idx / CH, ch = idx % CH;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (row < nrows) {
      int tok = tq0 + row / G, gh = row % G;
      v = *reinterpret_cast<const uint4*>(p.q + (size_t)(qs + tok) * p.q_st + (size_t)(hkv * G + gh) * p.q_sh + ch * 8);
    }
    *reinterpret_cast<uint4*>(sQ + sw_off<D>(row, ch)) = v;
  }
  if constexpr (WARP_PIPE) __syncthreads();  // publishes the Q tile; the loop below has no CTA-wide barrier

  for (int tile = tile_lo; tile < tile_hi; ++tile) {
    const int buf = (tile - tile_lo) % STAGES;
    cp_async_wait<STAGES - 2>();  // the group of this tile has landed (one group is committed per iteration)
    if constexpr (WARP_PIPE) {
      __syncwarp();                // ...for every lane of this warp, whose ldmatrix reads of the buffer refilled below are done
      if (tile + STAGES - 1 < tile_hi) load_tile_w(tile + STAGES - 1, (tile - tile_lo + STAGES - 1) % STAGES);
    } else {
      __syncthreads();             // ...for every thread, and everybody has finished the buffer refilled below
      if (tile + STAGES - 1 < tile_hi) load_tile(tile + STAGES - 1, (tile - tile_lo + STAGES - 1) % STAGES);
    }
    cp_async_commit();
    if (KV8) {
      const uint8_t* k8 = sK + (size_t)buf * kKeysPerTile * D;
      const uint8_t* v8 = sV + (size_t)buf * kKeysPerTile * D;
      if constexpr (WARP_PIPE) {
        // this warp's 16 keys -> its rows of the bf16 working tiles (its own MMAs of the previous tile are done: program order)
#pragma unroll
        for (int i = 0; i < 16 * WCH / 32; ++i) {
          const int idx = lane + 32 * i, row = warp * 16 + idx / WCH, ch = idx % WCH;
          uint4 lo, hi;
          widen_fp8x16(*reinterpret_cast<const uint4*>(k8 + row * D + ch * 16), lo, hi);
          *reinterpret_cast<uint4*>(sKb + sw_off<D>(row, ch * 2)) = lo;
          *reinterpret_cast<uint4*>(sKb + sw_off<D>(row, ch * 2 + 1)) = hi;
          widen_fp8x16(*reinterpret_cast<const uint4*>(v8 + row * D + ch * 16), lo, hi);
          *reinterpret_cast<uint4*>(sVb + sw_off<D>(row, ch * 2)) = lo;
          *reinterpret_cast<uint4*>(sVb + sw_off<D>(row, ch * 2 + 1)) = hi;
        }
        __syncwarp();
      } else {
        // widen this tile's bytes into the bf16 working tiles (everyone is past the previous tile's MMAs: barrier above)
#pragma unroll
        for (int i = 0; i < kKeysPerTile / kRowStep; ++i) {
          const int row = ld_row0 + i * kRowStep;
          uint4 lo, hi;
          widen_fp8x16(*reinterpret_cast<const uint4*>(k8 + row * D + ld_ch * 16), lo, hi);
          *reinterpret_cast<uint4*>(sKb + sw_off<D>(row, ld_ch * 2)) = lo;
          *reinterpret_cast<uint4*>(sKb + sw_off<D>(row, ld_ch * 2 + 1)) = hi;
          widen_fp8x16(*reinterpret_cast<const uint4*>(v8 + row * D + ld_ch * 16), lo, hi);
          *reinterpret_cast<uint4*>(sVb + sw_off<D>(row, ld_ch * 2)) = lo;
          *reinterpret_cast<uint4*>(sVb + sw_off<D>(row, ld_ch * 2 + 1)) = hi;
        }
        __syncthreads();
      }
    }
    const uint32_t kb = smem_u32(KV8 ? sKb : sK + (size_t)buf * kKeysPerTile * D * 2);
    const uint32_t vb = smem_u32(KV8 ? sVb : sV + (size_t)buf * kKeysPerTile * D * 2);
    const uint32_t qb = smem_u32(sQ);
    const int k0 = tile * kKeysPerTile + key_base;

    // ---- S = Q K^T
    float s[MBW][NB2 * 2][4];
#pragma unroll
    for (int b = 0; b < MBW; ++b)
#pragma unroll
      for (int n = 0; n < NB2 * 2; ++n) s[b][n][0] = s[b][n][1] = s[b][n][2] = s[b][n][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      uint32_t a[MBW][4];
#pragma unroll
      for (int b = 0; b < MBW; ++b) {
        int row = row_base + b * 16 + (lane & 15);
        ldsm_x4(a[b], qb + sw_off<D>(row, kk * 2 + (lane >> 4)));
      }
#pragma unroll
      for (int n2 = 0; n2 < NB2; ++n2) {
        uint32_t bfr[4];
        int krow = key_base + n2 * 16 + (lane & 7) + ((lane >> 4) << 3);
        ldsm_x4(bfr, kb + sw_off<D>(krow, kk * 2 + ((lane >> 3) & 1)));
#pragma unroll
        for (int b = 0; b < MBW; ++b) {
          mma_bf16(s[b][n2 * 2], a[b], bfr[0], bfr[1]);
          mma_bf16(s[b][n2 * 2 + 1], a[b], bfr[2], bfr[3]);
        }
      }
    }
    // ---- mask, online softmax
    float alpha_r[MBW][2];
#pragma unroll
    for (int b = 0; b < MBW; ++b) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int row = row_base + b * 16 + g_ + h * 8;
        const int qpos = ctx0 + tq0 + row / G;  // rows past nrows are never stored
        float mx = -INFINITY;
#pragma unroll
        for (int n = 0; n < NB2 * 2; ++n) {
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            int key = k0 + n * 8 + tg * 2 + e;
            float v = s[b][n][h * 2 + e] * sc;
            if (capped) v = tanhf(v) * sc_post;
            v = (key <= qpos && key < kv_end && key + wlo > qpos) ? v : -INFINITY;
            s[b][n][h * 2 + e] = v;
            mx = fmaxf(mx, v);
          }
        }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(mrow[b][h], mx);
        const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
        const float alpha = exp2f(mrow[b][h] - m_use);
        float sum = 0.f;
#pragma unroll
        for (int n = 0; n < NB2 * 2; ++n) {
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            float pv = exp2f(s[b][n][h * 2 + e] - m_use);
            s[b][n][h * 2 + e] = pv;
            sum += pv;
          }
        }
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        lrow[b][h] = lrow[b][h] * alpha + sum;
        mrow[b][h] = m_new;
        alpha_r[b][h] = alpha;
      }
    }
    // the running maxima settle after a few tiles: rescale the accumulator only when some row of the warp moved
#pragma unroll
    for (int b = 0; b < MBW; ++b) {
      if (__any_sync(0xffffffffu, alpha_r[b][0] != 1.f || alpha_r[b][1] != 1.f)) {
#pragma unroll
        for (int i = 0; i < D / 8; ++i) {
          o[b][i][0] *= alpha_r[b][0];
          o[b][i][1] *= alpha_r[b][0];
          o[b][i][2] *= alpha_r[b][1];
          o[b][i][3] *= alpha_r[b][1];
        }
      }
    }
    // ---- O += P V
#pragma unroll
    for (int n2 = 0; n2 < NB2; ++n2) {
      uint32_t a[MBW][4];
#pragma unroll
      for (int b = 0; b < MBW; ++b) {
        a[b][0] = pack_bf16(s[b][n2 * 2][0], s[b][n2 * 2][1]);
        a[b][1] = pack_bf16(s[b][n2 * 2][2], s[b][n2 * 2][3]);
        a[b][2] = pack_bf16(s[b][n2 * 2 + 1][0], s[b][n2 * 2 + 1][1]);
        a[b][3] = pack_bf16(s[b][n2 * 2 + 1][2], s[b][n2 * 2 + 1][3]);
      }
#pragma unroll
      for (int d2 = 0; d2 < D / 16; ++d2) {
        uint32_t bfr[4];
        int krow = key_base + n2 * 16 + (lane & 15);
        ldsm_x4_t(bfr, vb + sw_off<D>(krow, d2 * 2 + (lane >> 4)));
#pragma unroll
        for (int b = 0; b < MBW; ++b) {
          mma_bf16(o[b][d2 * 2], a[b], bfr[0], bfr[1]);
          mma_bf16(o[b][d2 * 2 + 1], a[b], bfr[2], bfr[3]);
        }
      }
    }
  }
  cp_async_wait<0>();

  if (MODE == 0) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int row = row_base + g_ + h * 8;
      if (row >= nrows) continue;
      const int tok = tq0 + row / G, gh = row % G;
      const float den = lrow[0][h] + (p.sinks != nullptr ? exp2f(p.sinks[hkv * G + gh] * 1.4426950408889634f - mrow[0][h]) : 0.f);
      const float inv = den > 0.f ? (KV8 ? p.v_scale : 1.f) / den : 0.f;
      __nv_bfloat16* dst = p.out + ((size_t)(qs + tok) * p.Hq + hkv * G + gh) * D;
#pragma unroll
      for (int i = 0; i < D / 8; ++i)
        *reinterpret_cast<uint32_t*>(dst + i * 8 + tg * 2) = pack_bf16(o[0][i][h * 2] * inv, o[0][i][h * 2 + 1] * inv);
      if (p.lse != nullptr && tg == 0)
        p.lse[(size_t)(qs + tok) * p.Hq + hkv * G + gh] = (mrow[0][h] + log2f(lrow[0][h])) * 0.6931471805599453f;
    }
    return;
  }

  // ---- mode 1: merge the four warps' partial results (they saw disjoint keys), then store or hand to the split combine
  __syncthreads();  // everyone is done reading K/V tiles; reuse that memory
  float* mo = reinterpret_cast<float*>(sK);             // [4][ROWS][D]
  float* mm = reinterpret_cast<float*>(sQ);             // [4][ROWS][2] (the Q tile is no longer needed)
#pragma unroll
  for (int b = 0; b < MBW; ++b)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int row = b * 16 + g_ + h * 8;
      float* dst = mo + ((size_t)warp * ROWS + row) * D;
#pragma unroll
      for (int i = 0; i < D / 8; ++i) {
        dst[i * 8 + tg * 2] = o[b][i][h * 2];
        dst[i * 8 + tg * 2 + 1] = o[b][i][h * 2 + 1];
      }
      if (tg == 0) {
        mm[((size_t)warp * ROWS + row) * 2] = mrow[b][h];
        mm[((size_t)warp * ROWS + row) * 2 + 1] = lrow[b][h];
      }
    }
  __syncthreads();
  for (int idx = threadIdx.x; idx < nrows * (D / 4); idx += 128) {
    const int row = idx / (D / 4), c4 = (idx % (D / 4)) * 4;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) M = fmaxf(M, mm[((size_t)w * ROWS + row) * 2]);
    float L = 0.f, acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      float mw = mm[((size_t)w * ROWS + row) * 2];
      float f = (mw == -INFINITY) ? 0.f : exp2f(mw - M);
      L += mm[((size_t)w * ROWS + row) * 2 + 1] * f;
      const float4 v = *reinterpret_cast<const float4*>(mo + ((size_t)w * ROWS + row) * D + c4);
      acc[0] += v.x * f; acc[1] += v.y * f; acc[2] += v.z * f; acc[3] += v.w * f;
    }
    const int tok = row / G, gh = row % G;
    const size_t orow = (size_t)(qs + tok) * p.Hq + hkv * G + gh;
    if (p.splits > 1) {
      float* wo = p.ws_o + ((size_t)blockIdx.z * p.T * p.Hq + orow) * D + c4;
      *reinterpret_cast<float4*>(wo) = make_float4(acc[0], acc[1], acc[2], acc[3]);
      if (c4 == 0) {
        float* wm = p.ws_ml + ((size_t)blockIdx.z * p.T * p.Hq + orow) * 2;
        wm[0] = M;
        wm[1] = L;
      }
    } else {
      const float den = L + (p.sinks != nullptr ? exp2f(p.sinks[hkv * G + gh] * 1.4426950408889634f - M) : 0.f);
      const float inv = den > 0.f ? (KV8 ? p.v_scale : 1.f) / den : 0.f;
      __nv_bfloat16* dst = p.out + orow * D + c4;
      *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf16(acc[0] * inv, acc[1] * inv), pack_bf16(acc[2] * inv, acc[3] * inv));
      if (p.lse != nullptr && c4 == 0) p.lse[orow] = (M + log2f(L)) * 0.6931471805599453f;
    }
  }
}

// merges split-KV partials: one warp per (token, head)
template <int D>
__global__ void attn_combine_kernel(const AttnParams p) {
  pdl_trigger();
  pdl_wait();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int rows = p.T * p.Hq;
  if (warp >= rows) return;
  float M = -INFINITY;
  for (int s = 0; s < p.splits; ++s) M = fmaxf(M, p.ws_ml[((size_t)s * rows + warp) * 2]);
  float L = 0.f;
  float acc[D / 32];
#pragma unroll
  for (int i = 0; i < D / 32; ++i) acc[i] = 0.f;
  for (int s = 0; s < p.splits; ++s) {
    const float ms = p.ws_ml[((size_t)s * rows + warp) * 2];
    const float f = (ms == -INFINITY) ? 0.f : exp2f(ms - M);
    L += p.ws_ml[((size_t)s * rows + warp) * 2 + 1] * f;
    const float* src = p.ws_o + ((size_t)s * rows + warp) * D;
#pragma unroll
    for (int i = 0; i < D / 32; ++i) acc[i] += src[lane + 32 * i] * f;
  }
  const float den = L + (p.sinks != nullptr ? exp2f(p.sinks[warp % p.Hq] * 1.4426950408889634f - M) : 0.f);
  const float inv = den > 0.f ? (p.kv_fp8 ? p.v_scale : 1.f) / den : 0.f;
#pragma unroll
  for (int i = 0; i < D / 32; ++i) p.out[(size_t)warp * D + lane + 32 * i] = __float2bfloat16(acc[i] * inv);
  if (p.lse != nullptr && lane == 0) p.lse[warp] = (M + log2f(L)) * 0.6931471805599453f;
}

template <int D, int MODE, int MB, bool KV8, int ST = 3>
int launch_one(const AttnParams& p, cudaStream_t st) {
  constexpr int ROWS = (MODE == 0) ? 64 : 16 * MB;
  const int smem = ROWS * D * 2 + (KV8 ? 2 * ST * kKeysPerTile * D + 2 * kKeysPerTile * D * 2 : 2 * ST * kKeysPerTile * D * 2);
  static int configured_dev[kMaxDevices] = {};
  int& configured = configured_dev[current_device_slot()];  // the limit is an attribute of (kernel, device)
  if (!configured) {
    if (cudaFuncSetAttribute(attn_kernel<D, MODE, MB, KV8, ST>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -4;
    configured = 1;
  }
  dim3 grid(MODE == 0 ? p.num_q_tiles : p.R, p.Hkv, MODE == 0 ? 1 : p.splits);
  if (grid.x == 0) return 0;
  launch_k(attn_kernel<D, MODE, MB, KV8, ST>, grid, dim3(128), (size_t)smem, st, true, p);
  if (MODE == 1 && p.splits > 1) {
    int rows = p.T * p.Hq;
    launch_k(attn_combine_kernel<D>, dim3((rows * 32 + 255) / 256), dim3(256), 0, st, true, p);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

}  // namespace

int attention_launch(const AttnParams& p, int mode, cudaStream_t st) {
  if (p.Hq % p.Hkv || p.bs < 16 || (p.bs & (p.bs - 1)) || (p.D != 64 && p.D != 128 && p.D != 256)) return -1;
  const int G = p.Hq / p.Hkv;
  if (G > 64) return -1;
  const bool f8 = p.kv_fp8 != 0;
  if (mode == 1) {
    const int rows = p.short_q_len * G;
    if (p.D == 64) {
      if (rows <= 16) return f8 ? launch_one<64, 1, 1, true>(p, st) : launch_one<64, 1, 1, false>(p, st);
      if (rows <= 32) return f8 ? launch_one<64, 1, 2, true>(p, st) : launch_one<64, 1, 2, false>(p, st);
    } else if (p.D == 128) {
      if (rows <= 16) {
        if (f8) return launch_one<128, 1, 1, true>(p, st);
        // two ring stages leave room for a third CTA per SM (experiment switch; three stages and two CTAs are the default)
        static const int two_stage = getenv("ONECAT_ATTN_STAGES") && atoi(getenv("ONECAT_ATTN_STAGES")) == 2;
        return two_stage ? launch_one<128, 1, 1, false, 2>(p, st) : launch_one<128, 1, 1, false>(p, st);
      }
      if (rows <= 32) return f8 ? launch_one<128, 1, 2, true>(p, st) : launch_one<128, 1, 2, false>(p, st);
    } else {
      if (rows <= 16) return f8 ? launch_one<256, 1, 1, true>(p, st) : launch_one<256, 1, 1, false>(p, st);
    }
    return -6;  // caller must use mode 0 for longer queries
  }
  if (p.D == 64) return f8 ? launch_one<64, 0, 1, true>(p, st) : launch_one<64, 0, 1, false>(p, st);
  if (p.D == 128) return f8 ? launch_one<128, 0, 1, true>(p, st) : launch_one<128, 0, 1, false>(p, st);
  return f8 ? launch_one<256, 0, 1, true>(p, st) : launch_one<256, 0, 1, false>(p, st);
}

unsigned int attention_read_status(bool clear) { return read_status_tu(clear); }
void attention_read_status_async(unsigned int* dst, cudaStream_t st) { read_status_tu_async(dst, st); }

}  // namespace oc
