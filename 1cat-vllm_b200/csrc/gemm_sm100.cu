// out[t, n] = sum_k X[t, k] * W[n, k]  on tcgen05 tensor cores with TMEM accumulators.
//
// One persistent, warp-specialised kernel serves dense bf16 weights and weight-only quantised layers whose weights are
// dequantised to bf16 on their way into the tensor core: 4-bit integer with group scales and zero points (AWQ/GPTQ, WKIND 1),
// FP8 e4m3 with block scales (WKIND 2), FP4 e2m1 with power-of-two scales per 32 k (MXFP4, WKIND 3) and FP4 e2m1 with e4m3 scales per
// 16 k times a global scale (NVFP4, WKIND 4):
//   * The weight tile (128 output features x 64 k) is UMMA operand A, so the 128 TMEM lanes are output features and
//     the accumulator columns are tokens. The token tile TN (32..256) is UMMA N: decode batches and 8192-token
//     prefill chunks run the same code, and a 4-bit weight tile is dequantised once per 128 x TN x 64 MMA block.
//   * warp 0: producer (TMA tensor copies of X and of bf16 W)
//     warp 1: TMEM allocation + single-thread tcgen05.mma issue
//     warps 2-9 (4-bit only): 4-bit -> bf16 dequantisation straight into TMEM (tcgen05.st); the MMA reads operand A from there
//     next four warps: epilogue (tcgen05.ld -> bf16 store | SiLU*mul | fp32 split-K partial + last-arriver reduction)
//     last warp (4-bit only): bulk copies of packed 4-bit tiles, running up to `pstages` tiles ahead of the operand stages
//   * one ring of stages carries both operands of a k tile, with one full and one empty barrier per stage: measured on
//     B200 the MMA-issuing thread is the critical path (a ready mbarrier wait, four tcgen05.mma and a tcgen05.commit cost it
//     about 450 cycles per k tile), so it does exactly one wait and one commit per k tile.
//   * two accumulators of TN columns each: the epilogue of tile i overlaps the main loop of tile i+1.
// Every wait is bounded; on expiry the CTA raises the status word and tears down (see common.cuh).
//
// Role of this file in the reference's terms: replaces the TurboMind s884 GEMM family and its dispatch
// (reference: csrc/sm70_turbomind/ops/awq_sm70_gemm.cu:3161,3278; gemm_universal.h:238) and cuBLAS for dense layers.
#include <stdlib.h>

#include <map>
#include <mutex>

#include "common.cuh"
#include "gemm_sm100.h"

namespace oc {

namespace {

#ifdef ONECAT_GEMM_TRACE
#define TRACE(slot) do { if (p.trace) p.trace[blockIdx.x * 16 + (slot)] = globaltimer_ns(); } while (0)
#define TDECL(...) long long __VA_ARGS__
#define TSTART() long long _t0 = clock64()
#define TLAP(acc) do { long long _t1 = clock64(); (acc) += _t1 - _t0; _t0 = _t1; } while (0)
#define TPUT(slot, v) do { if (p.trace) p.trace[blockIdx.x * 16 + (slot)] = (unsigned long long)(v); } while (0)
#else
#define TRACE(slot) do { } while (0)
#define TDECL(...) do { } while (0)
#define TSTART() do { } while (0)
#define TLAP(acc) do { } while (0)
#define TPUT(slot, v) do { } while (0)
#endif

// warp roles: 0 X producer, 1 MMA, then the dequantisation warps (4-bit weights: two groups of four that take alternate k tiles,
// so one group's shared-memory and TMEM latencies hide behind the other's arithmetic), four epilogue warps, and for 4-bit
// weights one more warp that streams packed tiles.
//
// SMALL (packed weights, token tile <= 64): a lighter CTA of which two share an SM. Measured on B200, the thread that issues
// tcgen05.mma spends ~80 cycles per instruction whatever the token tile, so a 128 x 64 x 64 block of four MMAs costs it more than
// the tensor pipe (4 x 32 cycles) or the memory system needs; a second resident CTA brings a second issuing thread and a second
// barrier chain. Such a CTA has one group of four dequantisation warps, one accumulator and half of the SM's TMEM columns.
template <int WKIND, int SMALL> struct Roles {
  // SMALL: one dequantisation group. Measured on B200 with two groups per light CTA (the first one also draining the accumulator
  // in place of the epilogue warps) the packed bf16 arithmetic of the SM was already saturated by four such warps per scheduler and
  // every warp simply ran half as fast: 78 against 56 microseconds on the gate|up decode shape.
  static constexpr int kDqGroups = SMALL ? 1 : 2;
  static constexpr bool kDqDrains = false;            // true: no epilogue warps, the first dequantisation group drains the accumulator
  static constexpr int kDqWarps = WKIND >= 1 ? 4 * kDqGroups : 0;
  static constexpr int kEpiWarps = kDqDrains ? 0 : 4;
  static constexpr int kEpi0 = 2 + kDqWarps;          // first epilogue warp (2, 6 or 10: all are 2 mod 4, the quarters line up)
  static constexpr int kPacked = kEpi0 + kEpiWarps;   // packed-tile producer (4-bit only)
  static constexpr int kThreads = (kPacked + (WKIND >= 1 ? 1 : 0)) * 32;
  static constexpr int kEpiThread0 = kDqDrains ? 64 : kEpi0 * 32;  // first of the 128 threads that run the epilogue
  static constexpr int kCtasPerSm = SMALL ? 2 : 1;
  static constexpr int kTmemCols = SMALL ? 256 : 512;
};
constexpr int BM = 128;  // weight rows (output features) per tile = UMMA M
constexpr int BK = 64;   // k per stage: one 128-byte swizzle atom of bf16
constexpr int kWStageBytes = BM * BK * 2;   // 16 KB
// packed 128 x 64 weight tile: 4 KB of nibbles (int4, fp4) or 8 KB of fp8 bytes, followed in its ring slot by one 32-bit
// word per weight row: int4 -> bf16 scale | bf16 (128 + zero) << 16; fp8 -> bf16 (scale * 2^120); fp4 -> the bf16 scales
// (* 2^126) of the tile's two 32-k groups
__host__ __device__ constexpr int packed_bytes(int wkind) { return wkind == 2 ? BM * BK : BM * BK / 2; }
// nvfp4 has four 16-k groups per k tile: two words per row (four bf16 scales, already multiplied by the global scale and 2^126)
__host__ __device__ constexpr int sz_words(int wkind) { return wkind == 4 ? 2 : 1; }
__host__ __device__ constexpr int sz_bytes(int wkind) { return BM * 4 * sz_words(wkind); }
__host__ __device__ constexpr int packed_slot(int wkind) { return packed_bytes(wkind) + sz_bytes(wkind); }
// 4-bit weights: the dequantised weight tiles form a ring in TMEM (32 columns per 128 x 64 tile) at the top of the 512 columns,
// `stages` deep and in lock step with the X ring in shared memory: 8 tiles when the two accumulators fit 256 columns (token tile
// <= 128), else 4 (token tile 192).

constexpr uint32_t kStagePitch = 320;                   // epilogue staging: 128 bf16 per token row + 64 bytes (rows land in different banks)
constexpr uint32_t kStageBytes = 2 * 32 * kStagePitch;  // two buffers of 32 token rows
struct SmemLayout {
  uint32_t x_off, w_off, p_off, stage_off, bar_off, total;
};
__host__ __device__ inline SmemLayout make_layout(int tn, int nt_sub, int xstages, int stages, int pstages, int wkind, int kps) {
  SmemLayout L;
  uint32_t o = 0;
  L.x_off = o;
  o += (uint32_t)xstages * kps * nt_sub * tn * 128;
  L.w_off = o;
  o += (pstages > 0 ? 0u : (uint32_t)stages * kWStageBytes);  // 4-bit weights are dequantised into TMEM, not shared memory
  L.p_off = o;
  o += (uint32_t)pstages * packed_slot(wkind);
  o = (o + 15u) & ~15u;
  L.stage_off = o;
  o += kStageBytes;
  L.bar_off = o;
  o += 1024;
  L.total = o;
  return L;
}

__device__ __forceinline__ uint32_t dq_pair(uint32_t w, uint32_t zb2, uint32_t s2) {
  // two nibbles (bits 0-3 and 16-19 of w) -> bf16x2 ((q - z) * s); 0x4300 is bf16 128.0 whose ulp is 1
  uint32_t v = (w & 0x000f000fu) | 0x43004300u;
  __nv_bfloat162 r = __hmul2(__hsub2(*reinterpret_cast<__nv_bfloat162*>(&v), *reinterpret_cast<__nv_bfloat162*>(&zb2)),
                             *reinterpret_cast<__nv_bfloat162*>(&s2));
  return *reinterpret_cast<uint32_t*>(&r);
}

// Two fp8 e4m3 bytes of `w` (picked by the prmt selector into bits 8-15 and 24-31) -> bf16x2 * s2. The seven exponent and mantissa
// bits land in the bf16 exponent/mantissa fields four places down, which reads as value * 2^-120 (also for e4m3 subnormals, which
// become bf16 subnormals); the scale word carries the 2^120 back.
__device__ __forceinline__ uint32_t dq_fp8_pair(uint32_t w, uint32_t sel, uint32_t s2) {
  uint32_t t;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(t) : "r"(w), "r"(0u), "r"(sel));
  uint32_t v = (t & 0x80008000u) | ((t >> 4) & 0x07f007f0u);
  __nv_bfloat162 r = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&v), *reinterpret_cast<__nv_bfloat162*>(&s2));
  return *reinterpret_cast<uint32_t*>(&r);
}

// Two fp4 e2m1 nibbles (bits 0-3 and 16-19 of w) -> bf16x2 * s2: sign to bit 15, the two exponent bits and the mantissa bit to
// bits 8..6, which reads as value * 2^-126; the scale word carries the 2^126 back.
__device__ __forceinline__ uint32_t dq_fp4_pair(uint32_t w, uint32_t s2) {
  uint32_t v = ((w & 0x00080008u) << 12) | ((w & 0x00070007u) << 6);
  __nv_bfloat162 r = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&v), *reinterpret_cast<__nv_bfloat162*>(&s2));
  return *reinterpret_cast<uint32_t*>(&r);
}

template <int WKIND, int SMALL>
__global__ void __launch_bounds__((Roles<WKIND, SMALL>::kThreads), (Roles<WKIND, SMALL>::kCtasPerSm))
gemm_wx_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW, const GemmParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // dynamic shared memory is only guaranteed 16-byte aligned: round up to the 1024 bytes the swizzle needs
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int kPackedBytes = packed_bytes(WKIND), kPackedSlot = packed_slot(WKIND);
  // NT token sub-tiles per work item (1 or 2): with two, a dequantised weight tile feeds two accumulators (2 x tn tokens), which
  // halves the dequantisation and MMA-issue work per token; both accumulators then belong to one work item.
  using R = Roles<WKIND, SMALL>;
  constexpr int kTmemCols = R::kTmemCols;
  const int NT = SMALL ? 1 : p.nt_sub, NB = SMALL ? 1 : 2 / NT;
  // k tiles per stage: a stage of the X / dequantised-W ring carries KPS k tiles behind one full and one empty barrier
  const int KPS = p.kps;
  const SmemLayout L = make_layout(p.tn, NT, p.xstages, p.stages, p.pstages, WKIND, KPS);
  uint8_t* sx = smem + L.x_off;
  uint8_t* sw = smem + L.w_off;
  uint8_t* sp = smem + L.p_off;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L.bar_off);
  // One ring of S stages carries both operands of a k tile: X in shared memory and W in shared memory (bf16, by TMA) or in TMEM
  // (4-bit, written by the dequantisation warps). Each stage has ONE full barrier (the TMA transaction bytes plus, for 4-bit
  // weights, one arrival per dequantisation warp) and ONE empty barrier (a single tcgen05.commit): the MMA thread's cost per k
  // tile is one wait, four MMAs and one commit, and that thread is the kernel's critical path.
  const int S = p.stages, PS = p.pstages;
  uint64_t* full = bars;                        // [S] operands of the stage are in place
  uint64_t* empty = full + S;                   // [S] MMA finished reading the stage
  uint64_t* pfull = empty + S;                  // [PS] packed tile landed
  uint64_t* pempty = pfull + PS;                // [PS] packed tile consumed
  uint64_t* tfull = pempty + PS;                // [2] accumulator complete
  uint64_t* tempty = tfull + 2;                 // [2] accumulator drained
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* red_flag = const_cast<int*>(reinterpret_cast<volatile int*>(tmem_slot + 2));
  uint64_t* red_bar = bars + 120;               // cluster split-K: one arrival per CTA of the cluster once its partial is in shared memory

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tn = p.tn;

  if (threadIdx.x == 0) {
    TRACE(0);
    for (int i = 0; i < S; ++i) {
      mbar_init(&full[i], WKIND >= 1 ? 5 : 1);  // the producer's expect_tx arrival (+ one per dequantisation warp of the group)
      mbar_init(&empty[i], 1);
    }
    for (int i = 0; i < PS; ++i) {
      mbar_init(&pfull[i], 1);
      mbar_init(&pempty[i], 4);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tfull[i], 1);
      mbar_init(&tempty[i], 4);     // one arrival per epilogue warp
    }
    if (p.cluster > 1) mbar_init(red_bar, (uint32_t)p.splits);
    *abort_flag = 0;
    mbar_fence_init();
    prefetch_tmap(&tmX);
    if (WKIND == 0) prefetch_tmap(&tmW);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (p.cluster > 1) cluster_sync_all();   // no CTA may signal a peer's barrier before that peer has initialised it
  const uint32_t tmem_base = *tmem_slot;
  if (threadIdx.x == 0) TRACE(1);

  // Work items. Dense: (n tile, token tile, k split) enumerated arithmetically. Grouped (mixture-of-experts): a device-built list of
  // {weight row tile in the stacked expert matrix, first token row, number of valid rows, output column base}; its length is
  // read from device memory, so the launch needs no host knowledge of how tokens were routed.
  // Programmatic dependent launch: everything above overlaps the previous kernel's tail. With packed weights and arithmetic work
  // items the weight producer, the dequantisation warps and the MMA warp touch no memory that another kernel writes (weights,
  // shared memory, TMEM), so they run ahead and fill the rings; only the activation producer and the epilogue warps wait.
  // A device-built work list, or bf16 weights loaded by the same thread as the activations, makes every thread wait here.
  pdl_trigger();
  const bool pdl_roles = WKIND >= 1 && p.work == nullptr;
  if (!pdl_roles) pdl_wait();
  const int total_work = p.work != nullptr ? *p.work_count : p.num_n_tiles * p.num_t_tiles * p.splits;
  const int ktiles = p.K / BK;
  auto decode = [&](int w, int& nt, int& tt, int& sp_, int& k0, int& k1) {
    if (p.work != nullptr) {
      const int4 it = p.work[w];
      nt = it.x;          // row tile of the stacked weights
      tt = it.y;          // first token row (not a tile index in this mode)
      sp_ = 0;
      k0 = 0;
      k1 = ktiles;
      return;
    }
    sp_ = w % p.splits;
    int tile = w / p.splits;
    tt = tile % p.num_t_tiles;
    nt = tile / p.num_t_tiles;
    k0 = sp_ * p.ktiles_per_split;
    k1 = min(k0 + p.ktiles_per_split, ktiles);
  };
  const bool grouped = p.work != nullptr;


  // ------------------------------------------------------------------ epilogue (run by the epilogue warps, or by the first
  // dequantisation group of a SMALL CTA)
  // The accumulator is [feature (TMEM lane)][token (column)] and the output is [token][feature], so up to 32 tokens at a time are
  // transposed through a shared-memory staging buffer and leave as 16-byte row segments: two lanes exchange one value per token
  // pair and store packed bf16x2 words, then the 128 epilogue threads copy the chunk out with full-sector vector stores (to the
  // local output, or to the peers' slabs of a tensor-parallel push). Two buffers alternate, so one named barrier per chunk
  // orders both the hand-over and the reuse.
  const int q = warp & 3;              // TMEM lane quarter this warp may read
  const int row = q * 32 + lane;       // weight row inside the tile
  const int et = threadIdx.x - R::kEpiThread0;    // 0..127 in the warps that run the epilogue
  uint32_t chunk_i = 0;
  const bool silu = p.epi == EPI_SILU_MUL;
  const uint32_t stg_u32 = smem_u32(smem + L.stage_off);
  // which of the rotating arrival buffers a tensor-parallel push goes to: a device word that the previous reduction kernel advances,
  // so it is read only after this thread has passed pdl_wait()
  size_t sel_off = 0;
  auto load_sel = [&]() {
    if (p.n_push > 0 && p.push_sel != nullptr) sel_off = (size_t)(*reinterpret_cast<const volatile int*>(p.push_sel)) * (size_t)p.push_sel_stride;
  };
  if (!pdl_roles) load_sel();
  auto strip = [](uint32_t w) -> uint32_t {  // bf16 -0.0 marks an empty slot of an arrival buffer: send +0.0 instead
    if ((w & 0xffffu) == 0x8000u) w &= 0xffff0000u;
    if ((w >> 16) == 0x8000u) w &= 0x0000ffffu;
    return w;
  };
  // emits `rows` staged token rows; staged row r is token t0 + tok0 + (r / 4) * tok_gstride + (r % 4) (a plain chunk has
  // tok_gstride 4); a[] are this thread's feature row, one value per staged token
  auto emit = [&](float (&a)[32], int rows, int tok0, int tok_gstride, int n_base, int t0, int t_end, float bias_v) {
    const uint32_t buf = stg_u32 + (chunk_i & 1u) * (32 * kStagePitch);
    if (silu) {
#pragma unroll
      for (int j = 0; j < 32; ++j) {  // lanes 0-15 hold gate rows, lanes 16-31 the matching up rows
        const float other = __shfl_xor_sync(0xffffffffu, a[j], 16);
        a[j] = a[j] / (1.f + __expf(-a[j])) * other;
      }
    } else if (bias_v != 0.f) {
#pragma unroll
      for (int j = 0; j < 32; ++j) a[j] += bias_v;
    }
    // feature pair (f, f + 1) of staged token j goes to the even lane, of token j + 1 to the odd lane
    const uint32_t col_b = silu ? (uint32_t)(q * 16 + (lane & 14)) * 2u : (uint32_t)(q * 32 + (lane & 30)) * 2u;
#pragma unroll
    for (int j = 0; j < 32; j += 2) {
      const float send = (lane & 1) ? a[j] : a[j + 1];
      const float recv = __shfl_xor_sync(0xffffffffu, send, 1);
      const float lo = (lane & 1) ? recv : a[j], hi = (lane & 1) ? a[j + 1] : recv;
      __nv_bfloat162 pk = __floats2bfloat162_rn(lo, hi);
      if (!silu || lane < 16)
        asm volatile("st.shared.b32 [%0], %1;" ::"r"(buf + (uint32_t)(j + (lane & 1)) * kStagePitch + col_b), "r"(*reinterpret_cast<uint32_t*>(&pk)) : "memory");
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    const int vpr = silu ? 8 : 16;                       // 16-byte vectors per staged token row
    const int nb = silu ? n_base / 2 : n_base, nlim = silu ? p.n_out : p.N;
    for (int v = et; v < rows * vpr; v += 128) {
      const int r = v / vpr, cv = v - r * vpr;
      const int t = t0 + tok0 + (r >> 2) * tok_gstride + (r & 3), n0 = nb + cv * 8;
      if (t >= t_end || n0 >= nlim) continue;
      uint4 val = lds128(buf + (uint32_t)r * kStagePitch + (uint32_t)cv * 16u);
      if (p.n_push > 0 && p.push_sel != nullptr) { val.x = strip(val.x); val.y = strip(val.y); val.z = strip(val.z); val.w = strip(val.w); }
      const size_t off = (size_t)t * p.ldo + n0 + sel_off;
      const int nd = p.n_push == 0 ? 1 : (p.push_rows > 0 ? 1 : p.n_push);
      for (int d = 0; d < nd; ++d) {
        __nv_bfloat16* dst = (p.n_push == 0 ? p.out : (p.push_rows > 0 ? p.push_dst[t / p.push_rows] : p.push_dst[d])) + off;
        if (p.vec_ok && n0 + 8 <= nlim) {
          *reinterpret_cast<uint4*>(dst) = val;
        } else {
          const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&val);
          for (int i = 0; i < 8 && n0 + i < nlim; ++i) dst[i] = e[i];
        }
      }
    }
    ++chunk_i;
  };
  // drains the accumulator of work item w (the tile_i-th item of this CTA); false when a wait gave up
  auto epilogue_item = [&](int w, uint32_t tile_i) -> bool {
    int nt, tt, sp_, k0, k1;
    decode(w, nt, tt, sp_, k0, k1);
    const int acc = tile_i % NB;
    if (!mbar_wait(&tfull[acc], (tile_i / NB) & 1, abort_flag)) return false;
    tc_fence_after();
    if (et == 0) TRACE(4);
    const uint32_t taddr0 = tmem_base + acc * NT * p.acc_stride + ((uint32_t)(q * 32) << 16);
    const int tn_eff = tn * NT;  // tokens per work item
    // TMEM address of the 32-column chunk that starts at token column c of the work item (sub-tile c / tn)
    auto taddr_of = [&](int c) -> uint32_t { return NT == 1 ? taddr0 + c : taddr0 + (c / tn) * p.acc_stride + (c % tn); };
    int n_base = nt * BM, t0 = tt * tn_eff, t_end = p.T;
    if (grouped) {
      const int4 it = p.work[w];
      t0 = it.y;
      t_end = it.y + it.z;
      n_base = it.w;
    }
    const int n = n_base + row;
    const float bias_v = (!silu && p.bias != nullptr && n < p.N) ? __bfloat162float(p.bias[n]) : 0.f;
    if (p.splits > 1 && p.cluster > 1) {
      // Split-K inside a thread-block cluster: the CTAs that share a tile are the cluster (rank = split index, one work item per
      // CTA). Each leaves its fp32 partial in its own shared memory ([token / 4][row][4], over the operand ring, which is idle once
      // the last MMA has committed), tells every CTA of the cluster, and then reduces the token quads q with q % splits == rank
      // by reading all partials through distributed shared memory in split order (bit-stable). The reduction runs on all CTAs of
      // the cluster at once and never touches global memory; the cluster barrier at the end of the kernel keeps every CTA's
      // shared memory alive until its peers have read it.
      const uint32_t red_u32 = smem_u32(smem + L.x_off);
      for (int c = 0; c < tn_eff; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32(taddr_of(c), v);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          sts128(red_u32 + (uint32_t)(((c + j) >> 2) * (BM * 16) + row * 16), make_uint4(v[j], v[j + 1], v[j + 2], v[j + 3]));
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
      asm volatile("bar.sync 2, 128;" ::: "memory");
      if (et < p.splits) mbar_arrive_cluster(mapa_shared(smem_u32(red_bar), (uint32_t)et));
      if (!mbar_wait_cluster(red_bar, 0, abort_flag)) return false;
      const int rank = (int)cluster_ctarank();
      const int quads = tn_eff >> 2;
      // rounds of up to eight quads per CTA (32 staged token rows, one emit): quad base + rank + i * splits
      for (int qb = 0; qb < quads; qb += 8 * p.splits) {
        float a[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) a[j] = 0.f;
        int nq = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int qd = qb + rank + i * p.splits;
          if (qd < quads) {
            const uint32_t local = red_u32 + (uint32_t)(qd * (BM * 16) + row * 16);
            // four splits' pieces of the quad in flight at a time (a cluster has at most 8 CTAs); summed in split order
#pragma unroll
            for (int h = 0; h < 8; h += 4) {
              if (h < p.splits) {
                float4 f[4];
#pragma unroll
                for (int s2 = 0; s2 < 4; ++s2)
                  f[s2] = h + s2 < p.splits ? ld_dsmem_f4(mapa_shared(local, (uint32_t)(h + s2))) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int s2 = 0; s2 < 4; ++s2) {
                  a[4 * i] += f[s2].x; a[4 * i + 1] += f[s2].y; a[4 * i + 2] += f[s2].z; a[4 * i + 3] += f[s2].w;
                }
              }
            }
            nq = i + 1;
          }
        }
        if (nq > 0) emit(a, 4 * nq, 4 * (qb + rank), 4 * p.splits, n_base, t0, t_end, bias_v);   // nq is uniform over the CTA
      }
      if (p.n_push > 0) __threadfence_system();
      return true;
    }
    if (p.splits > 1) {
      // Split-K: every CTA of the tile writes its fp32 partial ([token / 4][row][4], so a warp's 16-byte accesses are contiguous) and
      // bumps the tile's counter; the CTA that arrives last sums the partials in split order (bit-stable) and runs the real epilogue.
      // Nobody waits for anybody, so the scheme needs no guarantee about which CTAs are resident together.
      const int tile_id = nt * p.num_t_tiles + tt;
      float* wsp = p.ws + ((size_t)tile_id * p.splits + sp_) * BM * tn_eff + row * 4;
      for (int c = 0; c < tn_eff; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32(taddr_of(c), v);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          __stcg(reinterpret_cast<uint4*>(wsp + (size_t)((c + j) >> 2) * (BM * 4)), make_uint4(v[j], v[j + 1], v[j + 2], v[j + 3]));
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
      __threadfence();
      asm volatile("bar.sync 2, 128;" ::: "memory");
      if (et == 0) {
        const int old = atomicAdd(&p.counters[tile_id], 1);
        const int last = (old == p.splits - 1);
        if (last) p.counters[tile_id] = 0;  // ready for the next launch
        *red_flag = last;
      }
      asm volatile("bar.sync 2, 128;" ::: "memory");
      if (!*red_flag) return true;
      __threadfence();
      const float* base = p.ws + (size_t)tile_id * p.splits * BM * tn_eff + row * 4;
      const size_t sstride = (size_t)BM * tn_eff;
      for (int c = 0; c < tn_eff; c += 32) {
        float a[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) a[j] = 0.f;
        // one round per split with the chunk's eight loads in flight (the order of the sums stays split 0, 1, 2, ...)
        for (int s2 = 0; s2 < p.splits; ++s2) {
          const float* src = base + (size_t)s2 * sstride + (size_t)(c >> 2) * (BM * 4);
          float4 f[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) f[i] = __ldcg(reinterpret_cast<const float4*>(src + (size_t)i * (BM * 4)));
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            a[4 * i] += f[i].x; a[4 * i + 1] += f[i].y; a[4 * i + 2] += f[i].z; a[4 * i + 3] += f[i].w;
          }
        }
        emit(a, 32, c, 4, n_base, t0, t_end, bias_v);
      }
      if (p.n_push > 0) __threadfence_system();
      return true;
    }
    // ---- single-pass epilogue
    for (int c = 0; c < tn_eff; c += 32) {
      uint32_t v[32];
      tmem_ld_32x32(taddr_of(c), v);
      tmem_ld_wait();
      float a[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) a[j] = __uint_as_float(v[j]);
      if (c + 32 >= tn_eff) {  // the accumulator is in registers: the MMA warp may start the next tile on it
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty[acc]);
      }
      emit(a, 32, c, 4, n_base, t0, t_end, bias_v);
    }
    if (p.n_push > 0) __threadfence_system();  // peers will read these rows after this rank's next kernel raises its flag
    return true;
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      if (pdl_roles) pdl_wait();
      Ring st;
      bool ok = true;
      const uint32_t xs = (uint32_t)tn * 128;  // one token sub-tile
      const uint32_t bytes = NT * xs + (WKIND == 0 ? kWStageBytes : 0);
      for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
        int nt, tt, sp_, k0, k1;
        decode(w, nt, tt, sp_, k0, k1);
        for (int kt = k0; kt < k1; kt += KPS) {
          const int kc = min(KPS, k1 - kt);
          ok = mbar_wait(&empty[st.idx], st.phase ^ 1, abort_flag);
          if (!ok) break;
          mbar_expect_tx(&full[st.idx], bytes * kc);
          for (int j = 0; j < kc; ++j) {
            for (int i = 0; i < NT; ++i)  // rows past T are zero-filled by the copy
              tma_load_2d(sx + ((st.idx * KPS + j) * NT + i) * xs, &tmX, (kt + j) * BK, grouped ? tt : (tt * NT + i) * tn, &full[st.idx]);
            if (WKIND == 0) tma_load_2d(sw + (st.idx * KPS + j) * kWStageBytes, &tmW, (kt + j) * BK, nt * BM, &full[st.idx]);
          }
          st.advance(S);
        }
      }
    }
  } else if (warp == R::kPacked) {
    // ------------------------------------------------------------------ packed-weight producer (runs PS tiles ahead)
    if (WKIND >= 1 && lane == 0) {
      Ring pr;
      bool ok = true;
      const int gk = p.group_ktiles;
      for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
        int nt, tt, sp_, k0, k1;
        decode(w, nt, tt, sp_, k0, k1);
        const uint8_t* wsrc = p.w4 + ((size_t)nt * ktiles + k0) * kPackedBytes;
        const uint32_t* zsrc = p.w4_sz + (size_t)nt * BM * sz_words(WKIND);
        int g = k0 / gk, gi = k0 - g * gk;  // quantisation group of the k tile and position inside it
        for (int kt = k0; kt < k1; ++kt) {
          ok = mbar_wait(&pempty[pr.idx], pr.phase ^ 1, abort_flag);
          if (!ok) break;
          uint8_t* dst = sp + pr.idx * kPackedSlot;
          mbar_expect_tx(&pfull[pr.idx], kPackedSlot);
          bulk_load(dst, wsrc, kPackedBytes, &pfull[pr.idx]);
          // the group's scales/zeros ride along, so the dequantisation warps never touch global memory
          bulk_load(dst + kPackedBytes, zsrc + (size_t)g * p.n_pad * sz_words(WKIND), sz_bytes(WKIND), &pfull[pr.idx]);
          wsrc += kPackedBytes;
          if (++gi == gk) { gi = 0; ++g; }
          pr.advance(PS);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issue
    // The whole warp walks the loop in uniform control flow and one elected lane issues: descriptors and TMEM addresses then live in
    // uniform registers, where a loop run by a single lane would move every operand of every tcgen05.mma across from the vector
    // registers (measured: about 70 cycles per instruction on that path).
    {
      const uint32_t idesc = umma_idesc_bf16(BM, tn);
      uint32_t tile_i = 0;
      Ring st;
      bool ok = true;
      const uint32_t xs = (uint32_t)tn * 128;
      const uint32_t a_base = smem_u32(sw), b_base = smem_u32(sx);
      const uint32_t ta_base = tmem_base + (kTmemCols - S * KPS * 32);
      TDECL(c_wfull = 0, c_issue = 0, c_wtempty = 0);
      TSTART();
      for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x, ++tile_i) {
        int nt, tt, sp_, k0, k1;
        decode(w, nt, tt, sp_, k0, k1);
        const int acc = tile_i % NB;
        ok = mbar_wait(&tempty[acc], ((tile_i / NB) & 1) ^ 1, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        TLAP(c_wtempty);
        const uint32_t d_addr = tmem_base + acc * NT * p.acc_stride;
        uint32_t accum = 0;
        for (int kt = k0; kt < k1; kt += KPS) {
          const int kc = min(KPS, k1 - kt);
          const int s = st.idx;
          ok = mbar_wait(&full[s], st.phase, abort_flag);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after();
          TLAP(c_wfull);
          if (tile_i == 0 && kt == k0 && lane == 0) TRACE(2);
          for (int jj = 0; jj < kc; ++jj) {
            const int sk = s * KPS + jj;  // k tile slot of the ring
            const uint64_t db = umma_desc_sw128(b_base + sk * NT * xs);
            if (WKIND >= 1) {
              const uint32_t ta = ta_base + sk * 32;  // 64 k of bf16 = 32 columns per k tile
              if (NT == 1) {
                if (elect_one()) {
#pragma unroll
                  for (int j = 0; j < BK / 16; ++j) umma_bf16_ts(d_addr, ta + j * 8, db + (uint64_t)(j * 2), idesc, (accum | j) ? 1u : 0u);
                }
              } else {
                for (int i = 0; i < NT; ++i) {
                  const uint64_t dbi = umma_desc_sw128(b_base + (sk * NT + i) * xs);
                  if (elect_one()) {
#pragma unroll
                    for (int j = 0; j < BK / 16; ++j)
                      umma_bf16_ts(d_addr + i * p.acc_stride, ta + j * 8, dbi + (uint64_t)(j * 2), idesc, (accum | j) ? 1u : 0u);
                  }
                }
              }
            } else {
              const uint64_t da = umma_desc_sw128(a_base + sk * kWStageBytes);
              if (elect_one()) {
#pragma unroll
                for (int j = 0; j < BK / 16; ++j)  // +2 in the 16-byte-unit start address = 32 bytes = 16 bf16 along k inside the swizzle atom
                  umma_bf16(d_addr, da + (uint64_t)(j * 2), db + (uint64_t)(j * 2), idesc, (accum | j) ? 1u : 0u);
              }
            }
            accum = 1;
          }
          if (elect_one()) umma_commit(&empty[s]);  // frees the stage (both operands) once these MMAs have read it
          __syncwarp();
          st.advance(S);
          TLAP(c_issue);
        }
        if (ok && elect_one()) umma_commit(&tfull[acc]);
        __syncwarp();
        if (lane == 0) TRACE(3);
      }
      if (lane == 0) { TPUT(8, c_wfull); TPUT(9, c_issue); TPUT(10, c_wtempty); }
    }
  } else if (warp < R::kEpi0) {
    // ------------------------------------------------------------------ 4-bit -> bf16 dequantisation
    if (WKIND >= 1) {
      if (R::kDqDrains && pdl_roles) {  // a group that also drains accumulators writes global memory
        pdl_wait();
        load_sel();
      }
      const int r = (warp & 3) * 32 + lane;  // weight row = TMEM lane this warp may write
      const int grp = (warp - 2) >> 2;       // 0: even stages of the CTA's sequence, 1: odd ones (one group when SMALL)
      uint32_t seq = 0;
      Ring st, pr;
      bool ok = true;
      const uint32_t sp_u32 = smem_u32(sp);
      const uint32_t ta_row = tmem_base + (kTmemCols - S * KPS * 32) + ((uint32_t)((warp & 3) * 32) << 16);
      TDECL(c_wempty = 0, c_wpfull = 0, c_math = 0, c_st = 0);
      uint32_t dq_tile_i = 0;
      TSTART();
      for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
        int nt, tt, sp_, k0, k1;
        decode(w, nt, tt, sp_, k0, k1);
        for (int kt = k0; kt < k1 && ok; kt += KPS) {
          const int kc = min(KPS, k1 - kt);
          if (R::kDqGroups > 1 && (int)(seq++ & 1u) != grp) {  // the other group's stage: just keep the ring cursors in step
            st.advance(S);
            for (int j = 0; j < kc; ++j) pr.advance(PS);
            continue;
          }
          TLAP(c_st);
          ok = mbar_wait(&empty[st.idx], st.phase ^ 1, abort_flag);
          if (!ok) break;
          tc_fence_after();
          TLAP(c_wempty);
         for (int jj = 0; jj < kc; ++jj) {
          ok = mbar_wait(&pfull[pr.idx], pr.phase, abort_flag);
          if (!ok) break;
          TLAP(c_wpfull);
          const uint32_t slot = sp_u32 + pr.idx * kPackedSlot;
          const uint32_t szv = WKIND == 4 ? 0u : lds32(slot + kPackedBytes + r * 4);
          const uint32_t s2 = (szv & 0xffffu) | (szv << 16);          // low half replicated
          const uint32_t zb2 = (szv >> 16) | (szv & 0xffff0000u);    // high half replicated
          uint32_t o[32];  // 64 bf16 of this row: column c holds k = 2c (low half) and 2c+1 (high half)
          if (WKIND == 2) {
            // fp8 tile: four chunks of [128 rows][16 bytes]; byte i of a row's chunk c is k = 16c + i
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              const uint4 h = lds128(slot + c * 2048 + r * 16);
              const uint32_t w4[4] = {h.x, h.y, h.z, h.w};
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                o[8 * c + 2 * i] = dq_fp8_pair(w4[i], 0x1404u, s2);
                o[8 * c + 2 * i + 1] = dq_fp8_pair(w4[i], 0x3424u, s2);
              }
            }
          } else {
            const uint4 h0 = lds128(slot + r * 16), h1 = lds128(slot + 2048 + r * 16);
            const uint32_t words[8] = {h0.x, h0.y, h0.z, h0.w, h1.x, h1.y, h1.z, h1.w};
#pragma unroll
            for (int c = 0; c < 8; ++c) {
              const uint32_t q = words[c];
              if (WKIND == 1) {
                o[4 * c] = dq_pair(q, zb2, s2);
                o[4 * c + 1] = dq_pair(q >> 4, zb2, s2);
                o[4 * c + 2] = dq_pair(q >> 8, zb2, s2);
                o[4 * c + 3] = dq_pair(q >> 12, zb2, s2);
              } else if (WKIND == 4) {  // words 2g, 2g + 1 are the 16 k of group g
                const uint32_t szw = lds32(slot + kPackedBytes + r * 8 + (c >> 2) * 4);
                const uint32_t sc = (c & 2) ? ((szw >> 16) | (szw & 0xffff0000u)) : ((szw & 0xffffu) | (szw << 16));
                o[4 * c] = dq_fp4_pair(q, sc);
                o[4 * c + 1] = dq_fp4_pair(q >> 4, sc);
                o[4 * c + 2] = dq_fp4_pair(q >> 8, sc);
                o[4 * c + 3] = dq_fp4_pair(q >> 12, sc);
              } else {  // words 0-3 are k 0..31 (first scale), words 4-7 are k 32..63 (second scale)
                const uint32_t sc = c < 4 ? s2 : zb2;
                o[4 * c] = dq_fp4_pair(q, sc);
                o[4 * c + 1] = dq_fp4_pair(q >> 4, sc);
                o[4 * c + 2] = dq_fp4_pair(q >> 8, sc);
                o[4 * c + 3] = dq_fp4_pair(q >> 12, sc);
              }
            }
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(&pempty[pr.idx]);  // the packed words are in registers (one arrival per warp, not per thread)
          tmem_st_32x32(ta_row + (st.idx * KPS + jj) * 32, o);
          pr.advance(PS);
          TLAP(c_math);
         }
          if (!ok) break;
          tmem_st_wait();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&full[st.idx]);
          st.advance(S);
        }
        if (R::kDqDrains && grp == 0 && ok) ok = epilogue_item(w, dq_tile_i);
        ++dq_tile_i;
      }
      if (warp == 2 && lane == 0) { TPUT(11, c_wempty); TPUT(12, c_wpfull); TPUT(13, c_math); TPUT(14, c_st); }
    }
  } else if (!R::kDqDrains) {
    // ------------------------------------------------------------------ epilogue warps
    if (pdl_roles) {   // outputs, split-K partials and counters may still be in use by the previous kernel
      pdl_wait();
      load_sel();
    }
    uint32_t tile_i = 0;
    bool ok = true;
    for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x, ++tile_i) ok = epilogue_item(w, tile_i);
  }

  // ------------------------------------------------------------------ teardown
  if (threadIdx.x == R::kEpiThread0) TRACE(5);
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0) TRACE(6);
  if (*abort_flag && threadIdx.x == 0) {
    // give copies that are still in flight a bounded chance to land before the CTA's shared memory is released
    uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) {}
  }
  __syncthreads();
  if (p.cluster > 1) cluster_sync_all();   // peers may still be reading this CTA's partial
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
    if (lane == 0) TRACE(7);
  }
}

// ---- host side ------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres);
    fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// bf16 [rows, cols] row-major (row stride ld elements) -> box of {64 cols, box_rows rows}, 128-byte swizzle
int make_tmap_bf16(CUtensorMap* tm, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return -1;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {64, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

}  // namespace

int gemm_smem_bytes(const GemmParams& p) {
  return (int)make_layout(p.tn, (p.nt_sub < 1 || p.small) ? 1 : p.nt_sub, p.xstages, p.stages, p.pstages, p.wkind, p.kps < 1 ? 1 : p.kps).total + 1024;
}

namespace {
// Experiment switches (read once): ONECAT_W4_SMALL=0 keeps decode-sized packed GEMMs on the one-CTA-per-SM variant,
// ONECAT_W4_KPS=n sets the k tiles per stage of the light variant.
int env_int(const char* name, int dflt) {
  const char* v = getenv(name);
  return (v && *v) ? atoi(v) : dflt;
}
}  // namespace

// Picks the token tile, split-K factor and pipeline depths. Split-K spreads few-tile problems (decode) over all SMs.
void gemm_plan(GemmParams& p, int num_sms, bool w4) {
  const int use_small = env_int("ONECAT_W4_SMALL", 1);
  int T = p.T;
  int tn = T <= 32 ? 32 : T <= 64 ? 64 : T <= 128 ? 128 : (w4 ? 192 : 256);  // 4-bit: TMEM also holds the weight ring
  if (T > 256 && !w4) {
    // avoid a nearly empty last token tile when 128 divides the token count better
    int waste256 = ((T + 255) / 256) * 256 - T, waste128 = ((T + 127) / 128) * 128 - T;
    if (waste128 + 64 < waste256 && T < 1024) tn = 128;
  }
  if (w4 && T > 128) {
    const int forced = env_int("ONECAT_W4_PREFILL_TN", 0);   // experiment switch: 128 or 192 tokens per tile for prefill-sized batches
    if (forced == 128 || forced == 192) tn = forced;
  }
  p.tn = tn;
  // decode-sized dense problems with packed weights run the light CTA variant, two per SM (grouped work lists keep the full one:
  // their items are token slices of many experts and the list is sized for one CTA per SM)
  p.small = (w4 && use_small && tn <= 64 && p.work == nullptr) ? 1 : 0;
  const int slots = p.small ? 2 * num_sms : num_sms;
  // packed weights and many token tiles: pair the token tiles so that every dequantised weight tile feeds two accumulators. With one
  // token tile per weight tile the dequantisation warps (bound by the SM's packed-bf16 arithmetic, ~200-250 cycles per 128 x 64 tile)
  // barely keep up with the four MMAs of a 192-token tile (384 cycles); paired, they have twice the time. Both accumulators then
  // belong to one work item, so its epilogue no longer overlaps the next main loop. Measured on B200 (8192 / 1088 tokens):
  // K = 5120: 943 -> 988 and 933 -> 1027 TFLOP/s; K = 17408: 1129 -> 1170 TFLOP/s.
  const int nt_min_ktiles = env_int("ONECAT_W4_NTSUB_KTILES", 64);
  p.nt_sub = (w4 && p.work == nullptr && T > 2 * tn && p.K / BK >= nt_min_ktiles) ? 2 : 1;
  if (p.nt_sub == 2) {
    // Pairing halves the item count, which can cost a whole extra wave when there are few items: compare waves x cycles per k tile
    // (measured at 192-token tiles: 1524 cycles for a paired item, 839 for a single one). Example, 1088 tokens x 7168 rows: 168 paired
    // items = 2 waves (135 us measured) against 336 single items = 3 waves (121 us).
    const long n_tiles = (p.n_rows + BM - 1) / BM;
    const long items2 = n_tiles * ((T + 2 * tn - 1) / (2 * tn)), items1 = n_tiles * ((T + tn - 1) / tn);
    const long waves2 = (items2 + slots - 1) / slots, waves1 = (items1 + slots - 1) / slots;
    if (waves1 * 839 < waves2 * 1524) p.nt_sub = 1;
  }
  p.num_t_tiles = (T + tn * p.nt_sub - 1) / (tn * p.nt_sub);
  p.num_n_tiles = (p.n_rows + BM - 1) / BM;
  int ktiles = p.K / BK;
  int tiles = p.num_t_tiles * p.num_n_tiles;
  int best = 1;
  double best_cost = 1e30;
  // fixed cost of an item in k-tile times (pipeline fill, epilogue); the light variant overlaps it with the other resident CTA
  const double fixed = p.small ? 3.0 : 6.0;
  if (tiles < slots && p.ws != nullptr) {
    // Workspace split-K: fp32 partials through global memory, summed by the CTA that arrives last. Its 128 threads cannot keep more
    // than 16 KB of loads in flight, so the sum costs about 0.7 us per split and 32-token chunk whatever the split count's other
    // merits: measured tails of 8 to 12 us at 64 tokens, i.e. about five k-tile times per split and chunk.
    const int min_per = p.small ? 2 : 4;
    const double per_split = 2.5 * ((tn + 31) / 32);
    for (int s = 1; s <= 32; ++s) {
      int per = (ktiles + s - 1) / s;
      if (per < min_per || (s - 1) * per >= ktiles) continue;  // every split needs work
      if ((size_t)tiles * s * BM * tn * p.nt_sub * 4 > p.ws_bytes || tiles > p.max_counters) break;
      int items = tiles * s;
      int waves = (items + slots - 1) / slots;
      double cost = waves * (per + fixed) + (s > 1 ? 6.0 + per_split * s : 0.0);
      if (cost < best_cost * 0.98) { best_cost = cost; best = s; }
    }
  } else {
    best_cost = ktiles + fixed;
  }
  // Split-K inside a thread-block cluster: the splits of a tile are one cluster (at most 8 CTAs), partials stay in shared memory and
  // every CTA of the cluster reduces a share of the tile through distributed shared memory: no workspace traffic and no serial
  // tail. Every cluster should be resident at once, and clusters are placed inside one GPC, so only part of the CTA slots count.
  p.cluster = 0;
  if (env_int("ONECAT_GEMM_CLUSTER", 1) != 0 && p.work == nullptr && p.nt_sub == 1) {
    int s = (slots * env_int("ONECAT_GEMM_CLUSTER_FILL", 85) / 100) / tiles;
    if (s > 8) s = 8;
    while (s > 1 && ((ktiles + s - 1) / s < 2 || (s - 1) * ((ktiles + s - 1) / s) >= ktiles)) --s;
    if (s > 1) {
      const double cost = (ktiles + s - 1) / s + fixed + 3.0;
      if (cost <= best_cost) {
        best = s;
        p.cluster = s;
      }
    }
  }
  p.splits = best;
  p.ktiles_per_split = (ktiles + best - 1) / best;
  gemm_plan_stages(p, w4);
  if (p.cluster && (p.xstages * p.kps < 4 || p.nt_sub != 1)) {   // the fp32 partial (tn x 512 bytes) lies over the X ring
    p.cluster = 0;
    if (p.ws == nullptr || (size_t)tiles * best * BM * tn * 4 > p.ws_bytes || tiles > p.max_counters) {
      p.splits = 1;
      p.ktiles_per_split = ktiles;
    }
  }
}

// Pipeline depths from the shared-memory budget (227 KB per CTA, half of it for the light variant) for the chosen token tile.
void gemm_plan_stages(GemmParams& p, bool w4) {
  const int env_kps = env_int("ONECAT_W4_KPS", 0);
  const int tn = p.tn;
  if (p.nt_sub < 1) p.nt_sub = 1;
  p.kps = 1;
  if (!w4) {
    const int budget = 222 * 1024;
    p.nt_sub = 1;
    p.pstages = 0;
    p.small = 0;
    int s = (budget - 2048 - (int)kStageBytes) / (tn * 128 + kWStageBytes);
    p.stages = p.xstages = s > 8 ? 8 : (s < 2 ? 2 : s);
    p.acc_stride = 256;
    return;
  }
  const int slot = packed_slot(p.wkind > 0 ? p.wkind : 1);
  if (p.small && tn <= 64) {
    // 256 TMEM columns: one accumulator (64) + six dequantised k tiles (32 each) as 3 stages of 2 or 6 stages of 1
    p.nt_sub = 1;
    p.kps = env_kps > 0 ? env_kps : 2;
    if (p.kps > 3) p.kps = 3;
    p.stages = p.xstages = 6 / p.kps;
    p.acc_stride = 64;
    const int budget = 110 * 1024;
    int left = budget - 2048 - (int)kStageBytes - p.stages * p.kps * tn * 128;
    p.pstages = left / slot;
    if (p.pstages > 16) p.pstages = 16;
    return;
  }
  p.small = 0;
  const int budget = 222 * 1024;
  p.stages = p.xstages = tn <= 128 ? 8 : 4;  // limited by TMEM: 2 accumulators + 32 columns per stage
  p.pstages = tn <= 64 ? 12 : (tn == 128 ? 8 : 6);
  p.acc_stride = tn <= 128 ? 128 : 192;
  // shared memory: X ring (nt_sub sub-tiles per stage) + packed ring + barriers
  int left = budget - 2048 - (int)kStageBytes - p.stages * p.nt_sub * tn * 128;
  while (left < 2 * slot && p.stages > 2) {
    --p.stages;
    p.xstages = p.stages;
    left = budget - 2048 - (int)kStageBytes - p.stages * p.nt_sub * tn * 128;
  }
  if (p.pstages * slot > left) p.pstages = left / slot;
}

int gemm_launch(const GemmParams& p_in, const void* x, int ldx, const void* w_bf16, int ldw, int num_sms, cudaStream_t stream) {
  GemmParams p = p_in;
  const bool w4 = p.w4 != nullptr;
  if (p.nt_sub < 1) p.nt_sub = 1;
  if (p.kps < 1) p.kps = 1;
  CUtensorMap tmX, tmW;
  if (make_tmap_bf16(&tmX, x, (uint64_t)p.T, (uint64_t)p.K, (uint64_t)ldx, (uint32_t)p.tn)) return -2;
  if (!w4) {
    if (make_tmap_bf16(&tmW, w_bf16, (uint64_t)p.n_rows, (uint64_t)p.K, (uint64_t)ldw, BM)) return -3;
  } else {
    tmW = tmX;
  }
  p.vec_ok = (p.ldo % 8 == 0) && (((uintptr_t)p.out & 15) == 0 || p.n_push > 0);
  for (int d = 0; d < p.n_push; ++d) p.vec_ok = p.vec_ok && (((uintptr_t)p.push_dst[d] & 15) == 0);
  if (w4 && p.wkind == 0) p.wkind = 1;  // packed weights without a stated kind are 4-bit integer
  if (!w4) { p.wkind = 0; p.small = 0; }
  if (p.wkind < 0 || p.wkind > 4) return -6;
  if (p.small && (p.tn > 64 || p.work != nullptr)) return -7;
  int total = p.work != nullptr ? p.work_capacity : p.num_n_tiles * p.num_t_tiles * p.splits;
  const int slots = p.small ? 2 * num_sms : num_sms;
  int grid = total < slots ? total : slots;
  if (p.cluster > 1) {
    // one work item per CTA, the splits of a tile adjacent in the grid (cluster rank = split index)
    if (p.cluster != p.splits || p.cluster > 8 || p.work != nullptr || p.nt_sub > 1 || total > slots) return -11;
    grid = total;
  } else if (p.splits > 1 && (p.ws == nullptr || p.counters == nullptr || p.num_n_tiles * p.num_t_tiles > p.max_counters)) {
    return -9;
  }
  int smem = gemm_smem_bytes(p);
  // the opt-in shared-memory limit is a per-device attribute of each kernel: remember it per (device, kernel)
  constexpr int kMaxDev = 64;
  static bool configured[kMaxDev][5][2] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) return -8;
  const int sm = p.small ? 1 : 0;
  static std::mutex cfg_mutex;
  auto launch = [&](auto kernel, int threads) -> int {
    {
      std::lock_guard<std::mutex> lock(cfg_mutex);
      if (!configured[dev][p.wkind][sm]) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, sm ? 113 * 1024 : 227 * 1024) != cudaSuccess) return -4;
        // two light CTAs only fit an SM when the whole unified cache is carved out as shared memory
        cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared);
        configured[dev][p.wkind][sm] = true;
      }
    }
    if (p.cluster > 1) {
      cudaLaunchConfig_t cfg = {};
      cfg.blockDim = dim3(threads);
      cfg.dynamicSmemBytes = (size_t)smem;
      cfg.stream = stream;
      cudaLaunchAttribute at[2];
      at[0].id = cudaLaunchAttributeClusterDimension;
      at[0].val.clusterDim.y = 1;
      at[0].val.clusterDim.z = 1;
      at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      at[1].val.programmaticStreamSerializationAllowed = 1;
      cfg.attrs = at;
      const int tiles = p.num_n_tiles * p.num_t_tiles;
      const int sps = p.cluster;
      p.cluster = sps;
      cfg.gridDim = dim3((unsigned)(tiles * sps));
      at[0].val.clusterDim.x = (unsigned)sps;
      cfg.numAttrs = pdl_enabled() ? 2 : 1;
      return cudaLaunchKernelEx(&cfg, kernel, tmX, tmW, p) == cudaSuccess ? 0 : -12;
    }
    return launch_k(kernel, dim3(grid), dim3(threads), (size_t)smem, stream, true, tmX, tmW, p) == cudaSuccess ? 0 : -10;
  };
  int rc = 0;
  switch (p.wkind * 2 + sm) {
    case 0: rc = launch(gemm_wx_kernel<0, 0>, Roles<0, 0>::kThreads); break;
    case 2: rc = launch(gemm_wx_kernel<1, 0>, Roles<1, 0>::kThreads); break;
    case 3: rc = launch(gemm_wx_kernel<1, 1>, Roles<1, 1>::kThreads); break;
    case 4: rc = launch(gemm_wx_kernel<2, 0>, Roles<2, 0>::kThreads); break;
    case 5: rc = launch(gemm_wx_kernel<2, 1>, Roles<2, 1>::kThreads); break;
    case 6: rc = launch(gemm_wx_kernel<3, 0>, Roles<3, 0>::kThreads); break;
    case 7: rc = launch(gemm_wx_kernel<3, 1>, Roles<3, 1>::kThreads); break;
    case 8: rc = launch(gemm_wx_kernel<4, 0>, Roles<4, 0>::kThreads); break;
    case 9: rc = launch(gemm_wx_kernel<4, 1>, Roles<4, 1>::kThreads); break;
    default: return -6;
  }
  if (rc != 0) return rc;
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

unsigned int gemm_read_status(bool clear) { return read_status_tu(clear); }
void gemm_read_status_async(unsigned int* dst, cudaStream_t st) { read_status_tu_async(dst, st); }

// Diagnostics: what the runtime says about one kernel variant (registers, static shared and local memory per thread, and how many
// CTAs with `smem` bytes of dynamic shared memory it would keep resident per SM).
int gemm_kernel_info(int wkind, int small, int smem, int out[6]) {
  auto fill = [&](auto kernel, int threads) -> int {
    cudaFuncAttributes a;
    if (cudaFuncGetAttributes(&a, kernel) != cudaSuccess) return -1;
    cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, small ? 113 * 1024 : 227 * 1024);
    cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared);
    int occ = -1;
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kernel, threads, smem);
    out[0] = a.numRegs; out[1] = (int)a.sharedSizeBytes; out[2] = (int)a.localSizeBytes; out[3] = threads; out[4] = occ; out[5] = a.maxThreadsPerBlock;
    return 0;
  };
  switch (wkind * 2 + (small ? 1 : 0)) {
    case 0: return fill(gemm_wx_kernel<0, 0>, Roles<0, 0>::kThreads);
    case 2: return fill(gemm_wx_kernel<1, 0>, Roles<1, 0>::kThreads);
    case 3: return fill(gemm_wx_kernel<1, 1>, Roles<1, 1>::kThreads);
    case 4: return fill(gemm_wx_kernel<2, 0>, Roles<2, 0>::kThreads);
    case 5: return fill(gemm_wx_kernel<2, 1>, Roles<2, 1>::kThreads);
    default: return -2;
  }
}

}  // namespace oc

// ---- allocation-free entry point (see gemm_noalloc.h) -----------------------------------------------------------------
#include "gemm_noalloc.h"

namespace {
// Split-K scratch living in the library image: 16 MiB of fp32 partial tiles followed by 2048 tile counters (the first 1024 are used).
// In host code this name is only a handle for the symbol; the device address comes from cudaGetSymbolAddress.
static __device__ __align__(256) unsigned char g_noalloc_scratch[ONECAT_NOALLOC_SCRATCH_BYTES];
constexpr size_t kNoallocPartialBytes = 16u << 20;
constexpr int kNoallocMaxTiles = 1024;
constexpr int kNoallocMaxDevices = 64;
void* g_noalloc_ptr[kNoallocMaxDevices] = {nullptr};
std::mutex g_noalloc_mutex;
}  // namespace

extern "C" int onecat_gemm_bf16_splitk_noalloc(const void* x, const void* w, void* out, int T, int N, int K, int ldx, int ldw, int ldo,
                                               int splits, cudaStream_t stream) {
  using namespace oc;
  if (x == nullptr || w == nullptr || out == nullptr || T <= 0 || N <= 0 || K <= 0 || K % 64 != 0 || splits < 1) return ONECAT_NOALLOC_BAD_ARGUMENT;
  if (((uintptr_t)x & 15) || ((uintptr_t)w & 15) || ((uintptr_t)out & 15) || (ldx % 8) || (ldw % 8) || ldx < K || ldw < K || ldo < N)
    return ONECAT_NOALLOC_BAD_ARGUMENT;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kNoallocMaxDevices) return ONECAT_NOALLOC_SETUP_FAILED;
  int sms = 0;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return ONECAT_NOALLOC_SETUP_FAILED;
  {
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    if (g_noalloc_ptr[dev] == nullptr) {  // first call on this device (it is the current one): resolve the array's device address
      void* ptr = nullptr;
      if (cudaGetSymbolAddress(&ptr, g_noalloc_scratch) != cudaSuccess || ptr == nullptr) return ONECAT_NOALLOC_SETUP_FAILED;
      g_noalloc_ptr[dev] = ptr;
    }
  }
  unsigned char* base = static_cast<unsigned char*>(g_noalloc_ptr[dev]);
  GemmParams p{};
  p.T = T; p.N = N; p.K = K; p.n_rows = N; p.n_out = N; p.n_pad = 0; p.epi = EPI_STORE; p.group_ktiles = 1;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.ldo = ldo;
  p.bias = nullptr;
  p.ws = reinterpret_cast<float*>(base);
  p.ws_bytes = kNoallocPartialBytes;
  p.counters = reinterpret_cast<int*>(base + kNoallocPartialBytes);
  p.max_counters = kNoallocMaxTiles;
  p.w4 = nullptr; p.w4_sz = nullptr;
  gemm_plan(p, sms, false);
  p.cluster = 0;  // this entry point keeps its partials in the static scratch, with the caller's split count
  const int ktiles = K / 64;
  p.splits = splits;
  p.ktiles_per_split = (ktiles + splits - 1) / splits;
  if ((splits - 1) * p.ktiles_per_split >= ktiles) return ONECAT_NOALLOC_BAD_ARGUMENT;  // an empty split
  const size_t tiles = (size_t)p.num_t_tiles * p.num_n_tiles;
  if (tiles > (size_t)kNoallocMaxTiles || tiles * splits * 128 * p.tn * 4 > kNoallocPartialBytes) return ONECAT_NOALLOC_TOO_LARGE;
  if (splits > 1 && cudaMemsetAsync(p.counters, 0, tiles * sizeof(int), stream) != cudaSuccess) return ONECAT_NOALLOC_LAUNCH_FAILED;
  const int rc = gemm_launch(p, x, ldx, w, ldw, sms, stream);
  return rc == 0 ? 0 : ONECAT_NOALLOC_LAUNCH_FAILED;
}
