// Paged flash-attention prefill on tcgen05 tensor cores (head size 128, causal with prefix, GQA).
//
// One CTA owns 128 consecutive query tokens of one request for one query head and walks the keys in tiles of 128:
//   S = Q K^T      tcgen05.mma, both operands in shared memory (TMA, 128-byte swizzle), S in TMEM (fp32, double-buffered)
//   P = softmax    eight warps, two threads per query row (64 keys each; the row maximum is exchanged through shared memory):
//                  tcgen05.ld S, running max / sum in registers, P written back to TMEM as bf16 (tcgen05.st)
//   O_tile = P V   tcgen05.mma with operand A (P) read from TMEM and V as an MN-major shared-memory operand straight from the
//                  paged cache layout [key][d]; the softmax threads add O_tile into their fp32 output row in registers, rescaled
//                  by exp2(old max - new max), so no accumulator in TMEM ever needs a correction pass
// Roles: warp 0 = TMA producer (the 16 page loads of a K or V tile are issued by 16 lanes at once), warp 1 = MMA issue
// (one thread), warps 2-9 = softmax + epilogue (two warps per scheduler, so one warp's latencies hide behind the other's work; each
// thread accumulates half of its row's output columns). The MMA thread issues Q K^T of tile j+1 before P V of tile j, so the tensor
// pipe works on the next scores while the softmax warps are busy.
// Every wait is bounded; on expiry the CTA raises the status word and tears down (see common.cuh).
//
// Role in the reference's terms: the paged prefill of Flash-V100 / FA2 (reference: flash-attention-v100/kernel/
// fused_mha_forward_paged.cu:364,3297; vllm/v1/attention/backends/flash_attn.py) for D = 128; D = 256 stays on the mma.sync kernel.
#include "common.cuh"
#include "kernels.h"

namespace oc {

namespace {

constexpr int TQ = 128;   // query rows per CTA = UMMA M
constexpr int TK = 128;   // keys per tile = UMMA N of S and the k extent of P V
constexpr int HD = 128;   // head size
constexpr int kHalf = TK * 128;          // bytes of one 64-column half of a 128-row operand tile (rows of 128 bytes)
constexpr int kTile = 2 * kHalf;         // 32 KB: Q, or one K tile, or one V tile
constexpr int kStages = 2;
constexpr int kSmem = kTile + kStages * 2 * kTile + 1024 + 2 * 2 * TQ * 4;  // Q + K/V ring + barriers + row-maximum exchange
constexpr int kThreads = 320;
// TMEM columns: S0 | S1 | O_tile | P0 | P1
constexpr uint32_t kColS = 0, kColO = 256, kColP = 384;

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// V tile as UMMA operand B, MN-major (d contiguous): 64 d-values x 8 keys form a 1024-byte swizzle atom; the next 8 keys are
// 1024 bytes on (stride byte offset), the next 64 d-values are in the other half of the tile (leading byte offset).
__device__ __forceinline__ uint64_t umma_desc_sw128_mn(uint32_t smem_addr, uint32_t lbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

__global__ void __launch_bounds__(kThreads, 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmKV, const AttnParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sKV = smem + kTile;  // stage s: K at s * 2 * kTile, V right after it
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kTile + kStages * 2 * kTile);
  uint64_t* q_full = bars;            // [1]
  uint64_t* k_full = bars + 1;        // [kStages]
  uint64_t* v_full = k_full + kStages;
  uint64_t* k_empty = v_full + kStages;
  uint64_t* v_empty = k_empty + kStages;
  uint64_t* s_full = v_empty + kStages;   // [2] scores of a tile are complete
  uint64_t* p_ready = s_full + 2;         // [2] probabilities written (and the scores consumed)
  uint64_t* o_full = p_ready + 2;         // [1] P V of a tile is complete
  uint64_t* o_free = o_full + 1;          // [1] the softmax warps have read O_tile
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_free + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* s_req = const_cast<int*>(reinterpret_cast<volatile int*>(tmem_slot + 2));
  float* s_xch = reinterpret_cast<float*>(smem + kTile + kStages * 2 * kTile + 1024);  // [2 tile parities][2 halves][TQ]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y;
  const int G = p.Hq / p.Hkv;
  const int hkv = h / G;

  if (threadIdx.x == 0) {
    // which request and which of its 128-token tiles this CTA owns (short queries belong to the decode kernel)
    int b = blockIdx.x, found = -1, t0 = 0;
    for (int i = 0; i < p.R; ++i) {
      const int ql = p.query_start_loc[i + 1] - p.query_start_loc[i];
      const int nt = (ql > p.short_q_len) ? (ql + TQ - 1) / TQ : 0;
      if (b < nt) { found = i; t0 = b * TQ; break; }
      b -= nt;
    }
    s_req[0] = found;
    s_req[1] = t0;
    mbar_init(q_full, 1);
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&p_ready[i], 8);
    }
    mbar_init(o_full, 1);
    mbar_init(o_free, 8);
    *abort_flag = 0;
    mbar_fence_init();
    prefetch_tmap(&tmQ);
    prefetch_tmap(&tmKV);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int r = s_req[0], tq0 = s_req[1];

  int ntiles = 0, qs = 0, qlen = 0, S = 0, ctx0 = 0;
  if (r >= 0) {
    qs = p.query_start_loc[r];
    qlen = p.query_start_loc[r + 1] - qs;
    S = p.seq_lens[r];
    ctx0 = S - qlen;
    const int kv_end = min(S, ctx0 + min(tq0 + TQ, qlen));  // keys the last row of this tile may see
    ntiles = (kv_end + TK - 1) / TK;
  }

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (ntiles > 0) {
      if (lane == 0) {
        mbar_expect_tx(q_full, kTile);
        // rows past the end of the tensor are zero-filled; rows of the next request are loaded and never stored
        tma_load_2d(sQ, &tmQ, h * HD, qs + tq0, q_full);
        tma_load_2d(sQ + kHalf, &tmQ, h * HD + 64, qs + tq0, q_full);
      }
      const int* bt = p.block_table + (size_t)r * p.bt_stride;
      // lane -> (K or V, column half, 16-key chunk)
      const int is_v = lane >> 4, half = (lane >> 3) & 1, chunk = lane & 7;
      Ring st;
      bool ok = true;
      for (int j = 0; j < ntiles && ok; ++j) {
        const int key0 = j * TK + chunk * 16;
        int page = 0, off = 0;  // keys past the sequence read the null block
        if (key0 < S) {
          page = bt[key0 >> p.bs_shift];
          off = key0 & (p.bs - 1);
        }
        const int row = ((page * 2 + is_v) * p.Hkv + hkv) * p.bs + off;
        if (lane == 0) {
          ok = mbar_wait(&k_empty[st.idx], st.phase ^ 1, abort_flag);
          if (ok) ok = mbar_wait(&v_empty[st.idx], st.phase ^ 1, abort_flag);
          if (ok) {
            mbar_expect_tx(&k_full[st.idx], kTile);
            mbar_expect_tx(&v_full[st.idx], kTile);
          }
        }
        ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
        if (!ok) break;
        uint8_t* dst = sKV + (st.idx * 2 + is_v) * kTile + half * kHalf + chunk * 2048;
        tma_load_2d(dst, &tmKV, half * 64, row, is_v ? &v_full[st.idx] : &k_full[st.idx]);
        st.advance(kStages);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issue
    if (lane == 0 && ntiles > 0) {
      const uint32_t idesc_qk = umma_idesc_bf16(TQ, TK);
      const uint32_t idesc_pv = umma_idesc_bf16(TQ, HD) | (1u << 16);  // operand B (V) is MN-major
      const uint32_t q_addr = smem_u32(sQ), kv_addr = smem_u32(sKV);
      bool ok = mbar_wait(q_full, 0, abort_flag);
      auto issue_qk = [&](int j) {
        const int s = j % kStages;
        ok = mbar_wait(&k_full[s], (j / kStages) & 1, abort_flag);
        if (!ok) return;
        tc_fence_after();
        const uint32_t d_addr = tmem_base + kColS + (j & 1) * TK;
        const uint32_t k_base = kv_addr + (s * 2) * kTile;
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          const uint64_t da = umma_desc_sw128(q_addr + hf * kHalf), db = umma_desc_sw128(k_base + hf * kHalf);
#pragma unroll
          for (int jj = 0; jj < 4; ++jj)
            umma_bf16(d_addr, da + (uint64_t)(jj * 2), db + (uint64_t)(jj * 2), idesc_qk, (hf | jj) ? 1u : 0u);
        }
        umma_commit(&s_full[j & 1]);
        umma_commit(&k_empty[s]);
      };
      if (ok) issue_qk(0);
      for (int j = 0; j < ntiles && ok; ++j) {
        if (j + 1 < ntiles) issue_qk(j + 1);
        if (!ok) break;
        const int s = j % kStages;
        ok = mbar_wait(&p_ready[j & 1], (j >> 1) & 1, abort_flag);
        if (ok) ok = mbar_wait(&v_full[s], (j / kStages) & 1, abort_flag);
        if (ok && j > 0) ok = mbar_wait(o_free, (j - 1) & 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
        const uint32_t v_base = kv_addr + (s * 2 + 1) * kTile;
        const uint32_t pa = tmem_base + kColP + (j & 1) * (TK / 2);
#pragma unroll
        for (int jj = 0; jj < TK / 16; ++jj) {
          // 16 keys per MMA: 8 TMEM columns of P, two 8-key groups (2048 bytes) of V
          const uint64_t db = umma_desc_sw128_mn(v_base + jj * 2048, kHalf);
          umma_bf16_ts(tmem_base + kColO, pa + jj * 8, db, idesc_pv, jj ? 1u : 0u);
        }
        umma_commit(o_full);
        umma_commit(&v_empty[s]);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax + epilogue: two threads per query row
    const int q4 = warp & 3;                 // TMEM lane quarter this warp may touch
    const int half = (warp - 2) >> 2;        // which 64 keys of a tile / which 64 output columns this thread owns
    const int row = q4 * 32 + lane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(q4 * 32) << 16);
    const float sl2 = p.scale * 1.4426950408889634f;
    const int tq = tq0 + row;                       // query token inside the request
    const int limit = min(S, ctx0 + tq + 1);        // keys [0, limit) are visible to this row
    constexpr int HC = HD / 2, KC = TK / 2;
    float o[HC];
#pragma unroll
    for (int i = 0; i < HC; ++i) o[i] = 0.f;
    float m = -INFINITY, l = 0.f;
    float alpha[2] = {1.f, 1.f};
    bool ok = ntiles > 0;
    // the two warps that share a lane quarter meet on a named barrier of 64 threads
    auto pair_sync = [&]() { asm volatile("bar.sync %0, 64;" ::"r"(1 + q4) : "memory"); };

    // Both warps of a pair call pair_sync exactly ntiles + 1 times whatever happens (a named barrier has no time-out): a warp whose
    // bounded wait failed keeps walking the tiles without touching TMEM, and its partner learns of it through the abort flag.
    auto softmax_tile = [&](int j) {
      if (ok) ok = mbar_wait(&s_full[j & 1], (j >> 1) & 1, abort_flag);
      tc_fence_after();
      const uint32_t s_addr = lane_addr + kColS + (j & 1) * TK + half * KC;
      const int k0 = j * TK + half * KC;
      const bool masked = k0 + KC > limit;
      // pass 1: maximum of this thread's 64 scores, then of the row
      float raw = -INFINITY;
      if (ok) {
#pragma unroll
        for (int c = 0; c < KC; c += 32) {
          uint32_t v[32];
          tmem_ld_32x32(s_addr + c, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            float x = __uint_as_float(v[i]);
            if (masked && k0 + c + i >= limit) x = -INFINITY;
            raw = fmaxf(raw, x);
          }
        }
      }
      float* xch = s_xch + (j & 1) * 2 * TQ;
      xch[half * TQ + row] = raw;
      pair_sync();
      if (!ok || *abort_flag) { ok = false; return; }
      const float mx = fmaxf(m, fmaxf(raw, xch[(half ^ 1) * TQ + row]) * sl2);
      const float m_use = (mx == -INFINITY) ? 0.f : mx;  // a row that sees no key yet keeps zeros
      alpha[j & 1] = (m == -INFINITY) ? 0.f : ex2(m - m_use);
      m = mx;
      // pass 2: probabilities -> bf16 pairs in TMEM, partial row sum
      float sum = 0.f;
      uint32_t pk[32];
#pragma unroll
      for (int c = 0; c < KC; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32(s_addr + c, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float x0 = __uint_as_float(v[i]) * sl2 - m_use, x1 = __uint_as_float(v[i + 1]) * sl2 - m_use;
          if (masked && k0 + c + i >= limit) x0 = -INFINITY;
          if (masked && k0 + c + i + 1 >= limit) x1 = -INFINITY;
          __nv_bfloat162 b = __floats2bfloat162_rn(ex2(x0), ex2(x1));
          sum += __low2float(b) + __high2float(b);   // the sum of what the tensor core will actually multiply
          pk[(c + i) >> 1] = *reinterpret_cast<uint32_t*>(&b);
        }
      }
      tmem_st_32x32(lane_addr + kColP + (j & 1) * (TK / 2) + half * (KC / 2), pk);
      l = l * alpha[j & 1] + sum;
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_ready[j & 1]);
    };

    if (ntiles > 0) softmax_tile(0);
    for (int j = 0; j < ntiles; ++j) {
      if (j + 1 < ntiles) softmax_tile(j + 1);
      if (ok) ok = mbar_wait(o_full, j & 1, abort_flag);
      if (!ok) continue;
      tc_fence_after();
      const float a = alpha[j & 1];
#pragma unroll
      for (int c = 0; c < HC; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32(lane_addr + kColO + half * HC + c, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) o[c + i] = o[c + i] * a + __uint_as_float(v[i]);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(o_free);
    }
    // the row sum is the sum of the two halves' partial sums (both were scaled by the same alphas)
    float* xch = s_xch + (ntiles & 1) * 2 * TQ;
    if (ntiles > 0) {
      xch[half * TQ + row] = l;
      pair_sync();
      l += xch[(half ^ 1) * TQ + row];
    }
    if (ok && !*abort_flag && tq < qlen) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      const size_t orow = (size_t)(qs + tq) * p.Hq + h;
      uint4* dst = reinterpret_cast<uint4*>(p.out + orow * HD + half * HC);
#pragma unroll
      for (int i = 0; i < HC; i += 8) {
        __nv_bfloat162 b0 = __floats2bfloat162_rn(o[i] * inv, o[i + 1] * inv), b1 = __floats2bfloat162_rn(o[i + 2] * inv, o[i + 3] * inv);
        __nv_bfloat162 b2 = __floats2bfloat162_rn(o[i + 4] * inv, o[i + 5] * inv), b3 = __floats2bfloat162_rn(o[i + 6] * inv, o[i + 7] * inv);
        dst[i >> 3] = make_uint4(*reinterpret_cast<uint32_t*>(&b0), *reinterpret_cast<uint32_t*>(&b1), *reinterpret_cast<uint32_t*>(&b2),
                                 *reinterpret_cast<uint32_t*>(&b3));
      }
      if (p.lse != nullptr && half == 0) p.lse[orow] = (m + log2f(l)) * 0.6931471805599453f;
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_flag && threadIdx.x == 0) {
    // give copies that are still in flight a bounded chance to land before the CTA's shared memory is released
    uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) {}
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres);
    fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// bf16 [rows][cols] with a row pitch in bytes -> boxes of {64 columns, box_rows rows}, 128-byte swizzle, zero fill
int make_tmap(CUtensorMap* tm, const void* base, uint64_t rows, uint64_t cols, uint64_t pitch_bytes, uint32_t box_rows) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return -1;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {pitch_bytes};
  cuuint32_t box[2] = {64, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

}  // namespace

// Prefill attention of every request with more than `short_q_len` query tokens. `num_q_tiles` = sum over those requests of
// ceil(q_len / 128); `num_blocks` = pages in the cache. Needs D == 128, the heads of a token contiguous in q (q_sh == D),
// 16-byte aligned bases and pitches.
int attention_prefill_tc_launch(const AttnParams& p, long long num_blocks, cudaStream_t st) {
  if (p.D != HD || p.q_sh != HD || p.Hq % p.Hkv || p.bs < 16 || (p.bs & (p.bs - 1))) return -1;
  if (((uintptr_t)p.q & 15) || ((uintptr_t)p.kv_cache & 15) || ((uintptr_t)p.out & 15) || (p.q_st * 2) % 16) return -1;
  if (p.num_q_tiles <= 0) return 0;
  CUtensorMap tmQ, tmKV;
  if (make_tmap(&tmQ, p.q, (uint64_t)p.T, (uint64_t)p.Hq * HD, (uint64_t)p.q_st * 2, TQ)) return -2;
  if (make_tmap(&tmKV, p.kv_cache, (uint64_t)num_blocks * 2 * p.Hkv * p.bs, HD, HD * 2, 16)) return -3;
  static bool configured_dev[kMaxDevices] = {};
  bool& configured = configured_dev[current_device_slot()];  // the limit is an attribute of (kernel, device)
  if (!configured) {
    if (cudaFuncSetAttribute(attn_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem + 1024) != cudaSuccess) return -4;
    configured = true;
  }
  dim3 grid(p.num_q_tiles, p.Hq);
  attn_prefill_tc_kernel<<<grid, kThreads, kSmem + 1024, st>>>(tmQ, tmKV, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

unsigned int attention_tc_read_status(bool clear) { return read_status_tu(clear); }
void attention_tc_read_status_async(unsigned int* dst, cudaStream_t st) { read_status_tu_async(dst, st); }

}  // namespace oc
