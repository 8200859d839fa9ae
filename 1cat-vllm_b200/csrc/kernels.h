// Host launchers of the non-GEMM kernels. All take raw device pointers and a stream; return 0 on success.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace oc {

struct RopeCacheParams {
  __nv_bfloat16 *q, *k, *v;
  long long q_st, q_sh, k_st, v_st;  // element strides: token / head (k and v heads are D apart)
  const int* positions;
  const float* cos_sin;  // [max_pos][rot]: cos | sin
  __nv_bfloat16* kv_cache;  // [blocks][2][Hkv][bs][D] or null
  const int* slot_mapping;
  const __nv_bfloat16 *q_norm, *k_norm;  // per-head RMSNorm weights or null
  int T, Hq, Hkv, D, rot, bs, gemma;
  float eps;
  int kv_fp8;                    // kv_cache holds e4m3 bytes: k / k_scale and v / v_scale, saturated
  float k_scale_inv, v_scale_inv;
  // rotary sections (0 = off): frequencies below mrope_s0 rotate by positions[t], below mrope_s1 by positions[pos_stride + t], the
  // rest by positions[2 * pos_stride + t]
  int mrope_s0, mrope_s1;
  long long pos_stride;
};

int rms_norm_launch(const void* x, const void* res_in, const void* w, void* y, void* res_out, int T, int H, int ldx, float eps,
                    int gemma, cudaStream_t st);
int rms_norm_gated_launch(const void* x, const void* z, const void* w, void* y, int rows, int D, int ldx, int ldz, int heads,
                          float eps, cudaStream_t st);
int silu_and_mul_launch(const void* x, void* y, int T, int I, cudaStream_t st);
int rope_cache_launch(const RopeCacheParams& p, cudaStream_t st);
int argmax_launch(const void* x, int is_fp32, long long* out, unsigned long long* packed, int B, int V, long long ld, cudaStream_t st);
int merge_attn_states_launch(const void* o1, const float* lse1, const void* o2, const float* lse2, void* out, float* lse_out, int rows, int D,
                             cudaStream_t st);
unsigned int elementwise_read_status(bool clear);
void elementwise_read_status_async(unsigned int* dst, cudaStream_t st);

struct AttnParams {
  const __nv_bfloat16* q;     // [T][Hq][D] with strides
  long long q_st, q_sh;
  const __nv_bfloat16* kv_cache;  // [blocks][2][Hkv][bs][D]
  __nv_bfloat16* out;         // [T][Hq][D] contiguous
  float* lse;                 // [T][Hq] or null
  const int* query_start_loc; // [R+1]
  const int* seq_lens;        // [R]
  const int* block_table;     // [R][bt_stride]
  int bt_stride;
  int R, T, Hq, Hkv, D, bs, bs_shift;  // bs: tokens per page (power of two, >= 16)
  float scale;
  int num_q_tiles;            // grid.x for prefill mode (host: sum over requests of ceil(q_len / tokens per tile))
  int splits;                 // decode mode: KV splits per (request, kv head)
  float* ws_o;                // [splits][T][Hq][D] fp32 partial outputs
  float* ws_ml;               // [splits][T][Hq][2]  running max (log2 domain) and sum
  int max_q_len;
  int short_q_len;            // requests with at most this many query tokens run in mode 1, the others in mode 0
  int window;                 // sliding window in tokens (0 = full causal attention); mma.sync kernels only
  float softcap;              // tanh soft-capping of the scaled scores (0 = off); mma.sync kernels only
  const float* sinks;         // [Hq] attention-sink logits or null; mma.sync kernels only
  int kv_fp8;                 // the cache holds e4m3 bytes (value / scale) instead of bf16; mma.sync kernels only
  float k_scale, v_scale;     // per-tensor scales of an fp8 cache
};
// mode 0: rows of a query tile are spread over warps (prefill / long queries); mode 1: keys are spread over warps
// (decode and short verify queries, with split-KV + combine).
int attention_launch(const AttnParams& p, int mode, cudaStream_t st);
unsigned int attention_read_status(bool clear);
void attention_read_status_async(unsigned int* dst, cudaStream_t st);
// tcgen05 prefill (attention_tc.cu): D == 128, 128-token query tiles; num_q_tiles counts those tiles.
int attention_prefill_tc_launch(const AttnParams& p, long long num_blocks, cudaStream_t st);
unsigned int attention_tc_read_status(bool clear);
void attention_tc_read_status_async(unsigned int* dst, cudaStream_t st);


struct RowStats {
  float p_draft;  // target probability of the draft token at the row's temperature
  int arg_all;    // arg-max of the row
  int arg_ex;     // recovered token: arg-max over v != draft of logit/T (+ Gumbel noise for random rows)
};
int rejection_launch(const void* logits, int is_fp32, const long long* draft_ids, const long long* num_draft, const long long* bonus,
                     const double* uniforms, const float* temperature, const float* synth_rates, RowStats* stats, long long* out, int B, int k, int V,
                     long long ld_b, long long ld_pos, unsigned long long seed, int use_noise, cudaStream_t st);

struct SampleParams {
  const void* logits;        // [B][ld] fp32 or bf16
  int is_fp32;
  long long ld;
  int B, V;
  const float* temperature;  // [B]; below 1e-5 the row takes its arg-max
  const int* top_k;          // [B] or null; <= 0 or >= V: off
  const float* top_p;        // [B] or null; >= 1: off
  const float* min_p;        // [B] or null; <= 0: off
  const unsigned long long* seeds;  // [B] one random 64-bit word per row and step
  long long* out;            // [B] sampled token ids
  unsigned char* kept;       // [B][V] or null: 1 where the token survived the filters
};
int sample_launch(const SampleParams& p, cudaStream_t st);

struct RouteParams {
  const __nv_bfloat16* logits;  // [T][ld]
  long long ld;
  const float* bias;            // e_score_correction_bias [E] or null
  float* topk_w;                // [T][k]
  int* topk_ids;                // [T][k]
  int T, E, k, n_group, topk_group, sigmoid, renormalize;
  float scaling;
};
int route_launch(const RouteParams& p, cudaStream_t st);
unsigned int sampling_read_status(bool clear);
void sampling_read_status_async(unsigned int* dst, cudaStream_t st);

struct MoePlanParams {
  int* counts;        // [E] scratch
  int* offsets;       // [E+1] first slot of each local expert
  int* cursor;        // [E] scratch
  int* total_slots;   // [1]
  int* work_count;    // [2] number of work items of the two grouped GEMMs
  int4* work1;        // GEMM 1 items {row tile in stacked w13, first slot, valid rows, output column base}
  int4* work2;        // GEMM 2 items (stacked w2)
  int E, tn, n1, n2;  // local experts, token tile, 128-row tiles per expert in w13 / w2
};
int moe_prepare_launch(const MoePlanParams& p, const int* ids, int n_pairs, int k, int e_off, int* slot_of, const void* x, long long ldx,
                       void* xs, int H, cudaStream_t st);
int moe_plan_launch(const MoePlanParams& p, cudaStream_t st);
int moe_combine_launch(const void* a2, const int* slot_of, const float* w, void* y, int T, int k, int H, cudaStream_t st);
unsigned int moe_read_status(bool clear);
void moe_read_status_async(unsigned int* dst, cudaStream_t st);

struct MlaParams {
  const __nv_bfloat16* q_abs;   // [T][H][512] query with W_UK absorbed
  const __nv_bfloat16* q_rope;  // [T][H][64]
  const __nv_bfloat16* cache;   // [blocks][bs][576] latent | rope key
  __nv_bfloat16* out;           // [T][H][512]
  const int* query_start_loc;
  const int* seq_lens;
  const int* block_table;
  int bt_stride, R, T, H, kv_lora, rope, bs, bs_shift, max_q_len, splits;
  float scale;
  float* ws_o;                  // [splits][T][H][512]
  float* ws_ml;                 // [splits][T][H][2]
};
int mla_decode_launch(const MlaParams& p, cudaStream_t st);
unsigned int mla_read_status(bool clear);
void mla_read_status_async(unsigned int* dst, cudaStream_t st);

struct GdnConvParams {
  const __nv_bfloat16* x;   // [T][ldx] pre-conv mixed q|k|v (column slice allowed)
  long long ldx;
  const __nv_bfloat16* w;   // [C][kw]
  __nv_bfloat16* y;         // [T][C] contiguous
  __nv_bfloat16* conv_state;  // [slots][C][kw-1], updated in place
  const int* query_start_loc;
  const int* state_slots;
  const int* has_initial_state;
  int T, R, C, kw;
  const int* n_valid;              // optional [R]: count only this many tokens of each chunk (speculative commit)
  const __nv_bfloat16* prev_state; // optional [R][C][kw-1]: snapshot of the state before the chunk (speculative commit)
};

struct GdnParams {
  const __nv_bfloat16 *q, *k, *v;  // post-conv tensors: q,k [T][Hk*K], v [T][Hv*V] with a common row pitch ld_qkv
  long long ld_qkv;
  const __nv_bfloat16 *a, *b;      // [T][Hv] gate inputs with row pitch ld_ba
  long long ld_ba;
  const float *A_log, *dt_bias;    // [Hv]
  float* state;                    // [slots][Hv][K][V] fp32
  __nv_bfloat16* out;              // [T][Hv*V]
  const int* query_start_loc;
  const int* state_slots;
  const int* has_initial_state;
  int R, Hk, Hv, K, V;
  int write_state;                 // 0: leave the slot untouched (speculative verification commits later)
  float* spec_state;               // optional [R][spec_q][Hv][K][V]: state after each token
  int spec_q;
  int skip_min_len;                // > 0: sequences with at least this many tokens are left to the chunked kernels
};

// Chunked prefill (gdn_chunk.cu): sequences of at least `GdnParams::skip_min_len` tokens are split into 64-token chunks listed by
// the host; the recurrent kernel skips them.
struct GdnChunkParams {
  const __nv_bfloat16 *q, *k, *v;
  long long ld_qkv;
  const __nv_bfloat16 *a, *b;
  long long ld_ba;
  const float *A_log, *dt_bias;
  float* state;
  __nv_bfloat16* out;
  const int* query_start_loc;
  const int* state_slots;
  const int* has_initial_state;
  int Hk, Hv, K, V, write_state;
  __nv_bfloat16* ws;          // gdn_chunk_workspace_elems(num_chunks, Hv) elements
  const int* chunk_req;       // [num_chunks] request of each chunk
  const int* chunk_t0;        // [num_chunks] first token of each chunk
  int num_chunks;
  const int* long_req;        // [num_long] requests on the chunked path
  const int* long_chunk0;     // [num_long] index of the request's first chunk
  int num_long;
};
size_t gdn_chunk_workspace_elems(int num_chunks, int Hv);
int gdn_chunk_launch(const GdnChunkParams& p, cudaStream_t st);

int gdn_conv_launch(const GdnConvParams& p, cudaStream_t st);
int gdn_conv_commit_launch(const GdnConvParams& p, cudaStream_t st);
int gdn_recurrent_launch(const GdnParams& p, cudaStream_t st);
unsigned int gdn_read_status(bool clear);
void gdn_read_status_async(unsigned int* dst, cudaStream_t st);

}  // namespace oc
