// Host interface of the tcgen05 GEMM (see gemm_sm100.cu).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace oc {

enum { EPI_STORE = 0, EPI_SILU_MUL = 1 };

struct GemmParams {
  int T, N, K;        // tokens, logical output features, reduction length (multiple of 64)
  int n_rows;         // weight rows the kernel walks (N, or 2*n_out for the interleaved gate|up layout)
  int n_out;          // output columns for EPI_SILU_MUL
  int n_pad;          // padded weight rows (stride of the scale/zero table)
  int tn, num_t_tiles, num_n_tiles, splits, ktiles_per_split;
  int acc_stride;               // TMEM columns between the two accumulators
  int nt_sub;                   // token sub-tiles (of tn tokens) per work item: 2 = one dequantised weight tile feeds both accumulators
  int xstages, stages, pstages;  // ring depths: X tiles, W tiles (bf16 weights: same ring as X), packed 4-bit tiles
  int kps;                      // 64-wide k tiles per ring stage (one full / empty barrier pair per stage); 0 reads as 1
  int small;                    // packed weights, token tile <= 64: the light CTA variant, two resident per SM
  int cluster;                  // > 1: the splits of a tile form a thread-block cluster of this size and reduce through distributed
                                // shared memory (splits == cluster <= 8, one work item per CTA); 0: partials through the workspace
  int epi;
  int group_ktiles;   // 64-wide k tiles per quantisation group (group 128 -> 2)
  __nv_bfloat16* out;
  int ldo;
  const __nv_bfloat16* bias;
  // Tensor-parallel push (row-parallel layers): when n_push > 0 the epilogue stores each output row into peer GPUs' slabs instead
  // of `out`: push_rows == 0 -> every row goes to all n_push destinations (one-shot reduction follows); push_rows > 0 -> row t goes
  // only to destination t / push_rows (its owner in the reduce-scatter). Destinations are [T][ldo] bf16 like `out`.
  __nv_bfloat16* push_dst[8];
  int n_push, push_rows;
  // Flag-free reduction that follows (see comm.cu, COMM_LAMPORT): the destinations are rotating arrival buffers; `push_sel` points at
  // the device word holding the buffer in use, `push_sel_stride` is the distance between buffers in elements, and values equal to the
  // "not here yet" marker (bf16 -0.0) are sent as +0.0
  const int* push_sel;
  long long push_sel_stride;
  int vec_ok;         // set by gemm_launch: every destination row segment is 16-byte aligned (vector stores)
  float* ws;          // split-K workspace
  size_t ws_bytes;
  int* counters;      // one per output tile, zero between launches
  int max_counters;
  const int4* work;         // grouped mode: device-built work items (see gemm_sm100.cu); null for a dense GEMM
  const int* work_count;    // grouped mode: number of items, in device memory
  int work_capacity;        // grouped mode: upper bound of the item count (sizes the grid)
  const uint8_t* w4;        // packed weight tiles [n tile][k tile][4096 B (int4, fp4) or 8192 B (fp8)]; null for bf16 weights
  const uint32_t* w4_sz;    // [group][n_pad] words: int4 bf16 scale | bf16 (128 + zero) << 16; fp8 bf16 (scale * 2^120);
                            // fp4 bf16 scales (* 2^126) of the k tile's two 32-k groups
  unsigned long long* trace;  // debugging aid (builds with ONECAT_GEMM_TRACE only): 8 globaltimer stamps per CTA, else null
  int wkind;                // 0 bf16 weights, 1 int4 with zero points (AWQ/GPTQ), 2 fp8 e4m3 block-scaled, 3 fp4 e2m1 (MXFP4),
                            // 4 fp4 e2m1 with four scales per k tile (NVFP4; two words per row in w4_sz)
};

void gemm_plan(GemmParams& p, int num_sms, bool w4);
void gemm_plan_stages(GemmParams& p, bool w4);
int gemm_smem_bytes(const GemmParams& p);
int gemm_launch(const GemmParams& p, const void* x, int ldx, const void* w_bf16, int ldw, int num_sms, cudaStream_t stream);
unsigned int gemm_read_status(bool clear);
void gemm_read_status_async(unsigned int* dst, cudaStream_t st);
int gemm_kernel_info(int wkind, int small, int smem, int out[6]);

}  // namespace oc
