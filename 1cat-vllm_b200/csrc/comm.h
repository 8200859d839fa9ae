// Peer-memory tensor-parallel reductions (see comm.cu).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

namespace oc {

constexpr int kMaxRanks = 8;
constexpr int kMaxCommBlocks = 1024;
enum { COMM_ONE_SHOT = 0, COMM_TWO_SHOT = 1, COMM_LAMPORT = 2, COMM_NVLS = 3 };
constexpr int kLamportBuffers = 3;

struct CommParams {
  const __nv_bfloat16* part[kMaxRanks];  // every rank's partial sums [T, H] (peer mappings; own entry is local)
  int* flags[kMaxRanks];                 // every rank's flag area: [2 phases][2 stages][tp][kMaxCommBlocks]
  int* seq_local;                        // [kMaxCommBlocks] per-CTA sequence numbers of this rank
  __nv_bfloat16* x_out[kMaxRanks];       // one-shot: only [rank] used (local output); two-shot: every rank's gather buffer
  const __nv_bfloat16* residual_in;      // [T, H] or null
  __nv_bfloat16* residual_out;           // [T, H] or null (two-shot: only owned rows are written)
  const __nv_bfloat16* w;                // RMSNorm weight or null (plain reduction)
  int T, H, tp, rank, mode, gemma, phase;
  float eps;
  unsigned long long wait_ns;
  // COMM_LAMPORT (decode-sized T): every rank's arrival area [3 buffers][tp sources][lam_rows][H] bf16, pre-filled with the
  // "not here yet" value (bf16 -0.0). A source stores its partial rows straight into slot [buffer][its rank] of every rank's
  // area (from the GEMM epilogue, or at the start of this kernel when lam_pushed == 0); the reader polls the data itself.
  __nv_bfloat16* lam[kMaxRanks];
  long long lam_buf_stride, lam_src_stride;  // elements between buffers / between sources
  int* lam_ctr;                              // this rank's device words: [0] buffer in use (0..2), [1] CTAs finished
  int lam_pushed;
};

// Expert-parallel token exchange (see ep_a2a.cu). The slab of every rank has the same layout (byte offsets below).
struct EpParams {
  char* slab[kMaxRanks];
  size_t off_counts;     // int32 [ranks][E]      pairs routed by each source rank to each expert
  size_t off_flags;      // int32 [4 stages][kMaxRanks]
  size_t off_recv_x;     // bf16  [cap][H]        rows dispatched to this rank, expert-major
  size_t off_recv_meta;  // int32 [cap]           (source rank << 24) | pair index at the source
  size_t off_ret;        // bf16  [ret_rows][H]   expert outputs returned to this rank, by pair
  size_t off_gather;     // bf16  [T_total][H]    combined rows of every rank (when gather != 0)
  const int* ids;        // [T][k] global expert ids of this rank's tokens
  const __nv_bfloat16* x;
  long long ldx;
  int* seq;              // [1] sequence number of the exchange in flight (device memory, advanced by the first kernel)
  int* done;             // [3] CTA completion counters
  int* send_base;        // [E]
  int* cursor;           // [E]
  int* counts_local;     // [E_local] rows received per local expert (input of the GEMM work-list builder)
  const int* total_slots;  // [1] rows received in total (written by the work-list builder)
  int n, me, E, E_local, k, H, T, n_pairs, cap, ret_rows, gather, t_off;
  unsigned long long wait_ns;
};
int ep_count_exchange_launch(const EpParams& p, cudaStream_t st);
int ep_dispatch_launch(const EpParams& p, int sms, cudaStream_t st);
int ep_return_launch(const EpParams& p, const void* a2, int sms, cudaStream_t st);
int ep_combine_launch(const EpParams& p, const float* w, void* y, int sms, cudaStream_t st);
unsigned int ep_read_status(bool clear);
void ep_read_status_async(unsigned int* dst, cudaStream_t st);

int tp_reduce_norm_launch(const CommParams& p, int grid, cudaStream_t st);
int comm_alloc(size_t bytes, void** ptr);
int comm_free(void* ptr);
int comm_export(void* ptr, void* handle_out64);
int comm_import(const void* handle64, void** ptr);
int comm_unimport(void* ptr);
unsigned int comm_read_status(bool clear);
void comm_read_status_async(unsigned int* dst, cudaStream_t st);

}  // namespace oc
