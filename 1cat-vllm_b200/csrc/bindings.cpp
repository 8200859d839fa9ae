// Python bindings of the sm_100a kernels (module onecat_vllm.ops._C). Tensors are validated here so that the kernels
// can assume alignment and layout; every function launches on the current CUDA stream of the tensor's device.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "comm.h"
#include "gemm_sm100.h"
#include "kernels.h"

namespace {

cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

int sm_count() {
  static int n = 0;
  if (!n) n = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  return n;
}

void check_bf16(const torch::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.scalar_type() == torch::kBFloat16, name, " must be bf16");
}

// out[T, n_out or N] = epilogue(X[T,K] @ W^T). Exactly one of `w` (bf16 [n_rows, K]) and `w4` (packed tiles) is given.
void gemm(torch::Tensor x, c10::optional<torch::Tensor> w, c10::optional<torch::Tensor> w4, c10::optional<torch::Tensor> w4_sz,
          torch::Tensor out, c10::optional<torch::Tensor> bias, torch::Tensor ws, torch::Tensor counters, int64_t N, int64_t n_rows,
          int64_t n_out, int64_t n_pad, int64_t epi, int64_t group_ktiles, int64_t force_splits, int64_t force_tn,
          std::vector<int64_t> push_dst, int64_t push_rows, int64_t wkind, int64_t trace_ptr, int64_t push_sel, int64_t push_sel_stride) {
  check_bf16(x, "x");
  check_bf16(out, "out");
  TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1 && out.dim() == 2 && out.stride(1) == 1, "x/out must be row-major 2-D");
  const c10::cuda::CUDAGuard guard(x.device());
  oc::GemmParams p{};
  p.T = (int)x.size(0);
  p.K = (int)x.size(1);
  if (p.T == 0) return;
  TORCH_CHECK(p.K % 64 == 0, "K must be a multiple of 64, got ", p.K);
  TORCH_CHECK(((uintptr_t)x.data_ptr() & 15) == 0 && (x.stride(0) * 2) % 16 == 0, "x must be 16-byte aligned with 16-byte row pitch");
  p.N = (int)N;
  p.n_rows = (int)n_rows;
  p.n_out = (int)n_out;
  p.n_pad = (int)n_pad;
  p.epi = (int)epi;
  p.group_ktiles = (int)group_ktiles;
  p.out = (__nv_bfloat16*)out.data_ptr();
  p.ldo = (int)out.stride(0);
  TORCH_CHECK(out.size(0) >= p.T && out.size(1) >= (epi == oc::EPI_SILU_MUL ? n_out : N), "out is too small");
  p.bias = bias.has_value() ? (const __nv_bfloat16*)bias->data_ptr() : nullptr;
  p.ws = (float*)ws.data_ptr();
  p.ws_bytes = (size_t)ws.numel() * ws.element_size();
  p.counters = (int*)counters.data_ptr();
  p.max_counters = (int)counters.numel();
  const void* wptr = nullptr;
  int ldw = 0;
  if (w4.has_value()) {
    TORCH_CHECK(w4_sz.has_value(), "w4 needs its scale/zero table");
    p.w4 = (const uint8_t*)w4->data_ptr();
    p.w4_sz = (const uint32_t*)w4_sz->data_ptr();
    TORCH_CHECK(((uintptr_t)p.w4 & 15) == 0, "packed weights must be 16-byte aligned");
    TORCH_CHECK(wkind >= 1 && wkind <= 4, "packed weights need wkind 1 (int4), 2 (fp8), 3 (mxfp4) or 4 (nvfp4)");
    p.wkind = (int)wkind;
    TORCH_CHECK(((uintptr_t)p.w4_sz & 15) == 0 && n_pad % 4 == 0, "scale table must be 16-byte aligned");
    TORCH_CHECK((size_t)w4->numel() * w4->element_size() >= (size_t)((n_rows + 127) / 128) * (p.K / 64) * (wkind == 2 ? 8192 : 4096),
                "packed weights are too small");
    TORCH_CHECK((size_t)w4_sz->numel() >= (size_t)((p.K / 64 + group_ktiles - 1) / group_ktiles) * n_pad * (wkind == 4 ? 2 : 1), "scale table is too small");
  } else {
    TORCH_CHECK(w.has_value(), "a weight is required");
    check_bf16(*w, "w");
    TORCH_CHECK(w->dim() == 2 && w->stride(1) == 1 && w->size(1) == p.K && w->size(0) >= n_rows, "w must be [n_rows, K] row-major");
    TORCH_CHECK(((uintptr_t)w->data_ptr() & 15) == 0 && (w->stride(0) * 2) % 16 == 0, "w must be 16-byte aligned");
    wptr = w->data_ptr();
    ldw = (int)w->stride(0);
  }
  TORCH_CHECK(push_dst.size() <= 8 && (push_dst.empty() || epi == oc::EPI_STORE), "push needs the plain store epilogue and at most 8 destinations");
  p.n_push = (int)push_dst.size();
  p.push_rows = (int)push_rows;
  for (size_t i = 0; i < push_dst.size(); ++i) p.push_dst[i] = (__nv_bfloat16*)(uintptr_t)push_dst[i];
  p.trace = (unsigned long long*)(uintptr_t)trace_ptr;
  p.push_sel = (const int*)(uintptr_t)push_sel;
  p.push_sel_stride = (long long)push_sel_stride;
  oc::gemm_plan(p, sm_count(), w4.has_value());
  if (force_tn > 0) {
    TORCH_CHECK(!w4.has_value() || force_tn <= 192, "4-bit weights support token tiles up to 192");
    p.tn = (int)force_tn;
    p.nt_sub = 1;
    p.num_t_tiles = (p.T + p.tn - 1) / p.tn;
    oc::gemm_plan_stages(p, w4.has_value());
  }
  if (force_splits > 0) {
    int ktiles = p.K / 64;
    p.splits = (int)force_splits;
    p.cluster = 0;  // a forced split count takes the workspace path
    p.ktiles_per_split = (ktiles + p.splits - 1) / p.splits;
    TORCH_CHECK((p.splits - 1) * p.ktiles_per_split < ktiles, "too many splits for K");
    TORCH_CHECK((size_t)p.num_t_tiles * p.num_n_tiles * p.splits * 128 * p.tn * (p.nt_sub < 1 ? 1 : p.nt_sub) * 4 <= p.ws_bytes, "split-K workspace too small");
    TORCH_CHECK(p.num_t_tiles * p.num_n_tiles <= p.max_counters, "not enough split-K counters");
    oc::gemm_plan_stages(p, w4.has_value());  // the stage shape depends on whether the k range is split
  }
  int rc = oc::gemm_launch(p, x.data_ptr(), (int)x.stride(0), wptr, ldw, sm_count(), cur_stream());
  TORCH_CHECK(rc == 0, "gemm launch failed with code ", rc);
}

std::tuple<torch::Tensor, c10::optional<torch::Tensor>> rms_norm(torch::Tensor x, torch::Tensor w, double eps,
                                                                c10::optional<torch::Tensor> residual, bool gemma) {
  check_bf16(x, "x");
  check_bf16(w, "w");
  TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1, "x must be [T, H] with unit inner stride");
  const c10::cuda::CUDAGuard guard(x.device());
  const int T = (int)x.size(0), H = (int)x.size(1);
  auto y = torch::empty({T, H}, x.options());
  c10::optional<torch::Tensor> res_out;
  const void* rin = nullptr;
  void* rout = nullptr;
  if (residual.has_value()) {
    check_bf16(*residual, "residual");
    TORCH_CHECK(residual->is_contiguous() && residual->size(0) == T && residual->size(1) == H, "residual must be contiguous [T, H]");
    res_out = torch::empty({T, H}, x.options());
    rin = residual->data_ptr();
    rout = res_out->data_ptr();
  }
  int rc = oc::rms_norm_launch(x.data_ptr(), rin, w.data_ptr(), y.data_ptr(), rout, T, H, (int)x.stride(0), (float)eps, gemma ? 1 : 0, cur_stream());
  TORCH_CHECK(rc == 0, "rms_norm failed: ", rc, " (H must be a multiple of 8 and <= 8192)");
  return {y, res_out};
}

torch::Tensor rms_norm_gated(torch::Tensor x, torch::Tensor z, torch::Tensor w, double eps, int64_t heads) {
  // x, z: [T, heads*D] (possibly column slices); returns contiguous [T*heads, D]
  check_bf16(x, "x");
  check_bf16(z, "z");
  const c10::cuda::CUDAGuard guard(x.device());
  const int T = (int)x.size(0), D = (int)(x.size(1) / heads);
  auto y = torch::empty({T * heads, D}, x.options());
  int rc = oc::rms_norm_gated_launch(x.data_ptr(), z.data_ptr(), w.data_ptr(), y.data_ptr(), (int)(T * heads), D, (int)x.stride(0),
                                     (int)z.stride(0), (int)heads, (float)eps, cur_stream());
  TORCH_CHECK(rc == 0, "rms_norm_gated failed: ", rc);
  return y;
}

torch::Tensor silu_and_mul(torch::Tensor x) {
  check_bf16(x, "x");
  TORCH_CHECK(x.is_contiguous() && x.dim() == 2, "x must be contiguous [T, 2I]");
  const c10::cuda::CUDAGuard guard(x.device());
  const int T = (int)x.size(0), I = (int)(x.size(1) / 2);
  auto y = torch::empty({T, I}, x.options());
  TORCH_CHECK(oc::silu_and_mul_launch(x.data_ptr(), y.data_ptr(), T, I, cur_stream()) == 0, "silu_and_mul failed");
  return y;
}

void rope_and_cache(torch::Tensor q, torch::Tensor k, torch::Tensor v, torch::Tensor positions, torch::Tensor cos_sin,
                    c10::optional<torch::Tensor> kv_cache, torch::Tensor slot_mapping, int64_t rot, c10::optional<torch::Tensor> qn,
                    c10::optional<torch::Tensor> kn, double eps, bool gemma, double k_scale, double v_scale, int64_t mrope_s0, int64_t mrope_s1) {
  check_bf16(q, "q");
  check_bf16(k, "k");
  check_bf16(v, "v");
  TORCH_CHECK(q.dim() == 3 && k.dim() == 3 && v.dim() == 3 && q.stride(2) == 1 && k.stride(2) == 1 && v.stride(2) == 1, "q/k/v must be [T,H,D]");
  TORCH_CHECK(k.stride(1) == k.size(2) && v.stride(1) == v.size(2), "k/v heads must be D apart");
  TORCH_CHECK(positions.scalar_type() == torch::kInt32 && slot_mapping.scalar_type() == torch::kInt32, "positions/slot_mapping must be int32");
  TORCH_CHECK(cos_sin.scalar_type() == torch::kFloat32 && cos_sin.size(1) == rot, "cos_sin must be fp32 [max_pos, rot]");
  const c10::cuda::CUDAGuard guard(q.device());
  oc::RopeCacheParams p{};
  p.q = (__nv_bfloat16*)q.data_ptr();
  p.k = (__nv_bfloat16*)k.data_ptr();
  p.v = (__nv_bfloat16*)v.data_ptr();
  p.q_st = q.stride(0);
  p.q_sh = q.stride(1);
  p.k_st = k.stride(0);
  p.v_st = v.stride(0);
  p.positions = positions.data_ptr<int>();
  if (mrope_s0 > 0) {
    TORCH_CHECK(positions.dim() == 2 && positions.size(0) == 3 && positions.size(1) == q.size(0) && positions.stride(1) == 1,
                "rotary sections need positions [3, T]");
    TORCH_CHECK(mrope_s1 >= mrope_s0 && mrope_s1 <= rot / 2, "rotary sections exceed the rotary width");
    p.mrope_s0 = (int)mrope_s0;
    p.mrope_s1 = (int)mrope_s1;
    p.pos_stride = positions.stride(0);
  } else {
    TORCH_CHECK(positions.dim() == 1, "positions must be [T]");
  }
  p.cos_sin = cos_sin.data_ptr<float>();
  p.slot_mapping = slot_mapping.data_ptr<int>();
  p.T = (int)q.size(0);
  p.Hq = (int)q.size(1);
  p.Hkv = (int)k.size(1);
  p.D = (int)q.size(2);
  p.rot = (int)rot;
  p.gemma = gemma ? 1 : 0;
  p.eps = (float)eps;
  p.bs = 16;
  if (kv_cache.has_value()) {
    TORCH_CHECK(kv_cache->is_cuda() && (kv_cache->scalar_type() == torch::kBFloat16 || kv_cache->scalar_type() == torch::kFloat8_e4m3fn),
                "kv_cache must be a bf16 or float8_e4m3fn CUDA tensor");
    p.kv_fp8 = kv_cache->scalar_type() == torch::kFloat8_e4m3fn;
    p.k_scale_inv = (float)(1.0 / k_scale);
    p.v_scale_inv = (float)(1.0 / v_scale);
    TORCH_CHECK(kv_cache->is_contiguous() && kv_cache->dim() == 5 && kv_cache->size(1) == 2 && kv_cache->size(2) == p.Hkv && kv_cache->size(4) == p.D,
                "kv_cache must be contiguous [blocks, 2, Hkv, block_size, D]");
    p.kv_cache = (__nv_bfloat16*)kv_cache->data_ptr();
    p.bs = (int)kv_cache->size(3);
  }
  p.q_norm = qn.has_value() ? (const __nv_bfloat16*)qn->data_ptr() : nullptr;
  p.k_norm = kn.has_value() ? (const __nv_bfloat16*)kn->data_ptr() : nullptr;
  TORCH_CHECK(oc::rope_cache_launch(p, cur_stream()) == 0, "rope_and_cache failed");
}

void paged_attention(torch::Tensor q, torch::Tensor kv_cache, torch::Tensor out, c10::optional<torch::Tensor> lse, torch::Tensor qsl,
                     torch::Tensor seq_lens, torch::Tensor block_table, double scale, int64_t mode, int64_t num_q_tiles, int64_t splits,
                     int64_t max_q_len, int64_t short_q_len, c10::optional<torch::Tensor> ws_o, c10::optional<torch::Tensor> ws_ml,
                     int64_t window, double softcap, c10::optional<torch::Tensor> sinks, double k_scale, double v_scale) {
  check_bf16(q, "q");
  TORCH_CHECK(kv_cache.is_cuda() && (kv_cache.scalar_type() == torch::kBFloat16 || kv_cache.scalar_type() == torch::kFloat8_e4m3fn),
              "kv_cache must be a bf16 or float8_e4m3fn CUDA tensor");
  check_bf16(out, "out");
  TORCH_CHECK(q.dim() == 3 && q.stride(2) == 1 && out.is_contiguous(), "q must be [T,Hq,D]; out contiguous");
  TORCH_CHECK(((uintptr_t)q.data_ptr() & 15) == 0 && (q.stride(0) % 8) == 0 && (q.stride(1) % 8) == 0, "q must be 16-byte aligned");
  TORCH_CHECK(kv_cache.is_contiguous() && kv_cache.dim() == 5 && kv_cache.size(1) == 2, "kv_cache must be contiguous [blocks,2,Hkv,bs,D]");
  TORCH_CHECK(qsl.scalar_type() == torch::kInt32 && seq_lens.scalar_type() == torch::kInt32 && block_table.scalar_type() == torch::kInt32,
              "metadata must be int32");
  const c10::cuda::CUDAGuard guard(q.device());
  oc::AttnParams p{};
  p.q = (const __nv_bfloat16*)q.data_ptr();
  p.q_st = q.stride(0);
  p.q_sh = q.stride(1);
  p.kv_cache = (const __nv_bfloat16*)kv_cache.data_ptr();
  p.out = (__nv_bfloat16*)out.data_ptr();
  p.lse = lse.has_value() ? lse->data_ptr<float>() : nullptr;
  p.query_start_loc = qsl.data_ptr<int>();
  p.seq_lens = seq_lens.data_ptr<int>();
  p.block_table = block_table.data_ptr<int>();
  p.bt_stride = (int)block_table.stride(0);
  p.R = (int)seq_lens.size(0);
  p.T = (int)q.size(0);
  p.Hq = (int)q.size(1);
  p.Hkv = (int)kv_cache.size(2);
  p.D = (int)q.size(2);
  p.bs = (int)kv_cache.size(3);
  p.bs_shift = 0;
  while ((1 << p.bs_shift) < p.bs) ++p.bs_shift;
  p.scale = (float)scale;
  p.num_q_tiles = (int)num_q_tiles;
  p.splits = (int)splits;
  p.max_q_len = (int)max_q_len;
  p.short_q_len = (int)short_q_len;
  p.window = (int)window;
  p.softcap = (float)softcap;
  p.kv_fp8 = kv_cache.scalar_type() == torch::kFloat8_e4m3fn;
  p.k_scale = (float)k_scale;
  p.v_scale = (float)v_scale;
  TORCH_CHECK(mode != 2 || !p.kv_fp8, "an fp8 KV cache runs on the mma.sync kernels");
  if (sinks.has_value()) {
    TORCH_CHECK(sinks->is_cuda() && sinks->scalar_type() == torch::kFloat32 && sinks->is_contiguous() && sinks->numel() == q.size(1),
                "sinks must be a contiguous fp32 CUDA tensor with one entry per query head");
    p.sinks = sinks->data_ptr<float>();
  }
  TORCH_CHECK(mode != 2 || (window == 0 && softcap == 0.0 && !sinks.has_value()), "window / softcap / sinks run on the mma.sync kernels");
  if (mode == 1 && splits > 1) {
    TORCH_CHECK(ws_o.has_value() && ws_ml.has_value(), "split-KV needs workspaces");
    TORCH_CHECK((size_t)ws_o->numel() >= (size_t)splits * p.T * p.Hq * p.D && (size_t)ws_ml->numel() >= (size_t)splits * p.T * p.Hq * 2,
                "split-KV workspace too small");
    p.ws_o = ws_o->data_ptr<float>();
    p.ws_ml = ws_ml->data_ptr<float>();
  }
  if (p.T == 0 || p.R == 0) return;
  // mode 0: mma.sync prefill, 1: decode / short verify queries, 2: tcgen05 prefill (D = 128, query tiles of 128 tokens)
  int rc = mode == 2 ? oc::attention_prefill_tc_launch(p, kv_cache.size(0), cur_stream()) : oc::attention_launch(p, (int)mode, cur_stream());
  TORCH_CHECK(rc == 0, "attention launch failed with code ", rc);
}

// LSE-weighted merge of two partial attention results [T, H, D] bf16 with fp32 [T, H] log-sum-exps; returns (merged, merged lse)
std::vector<torch::Tensor> merge_attn_states(torch::Tensor o1, torch::Tensor lse1, torch::Tensor o2, torch::Tensor lse2) {
  check_bf16(o1, "o1");
  check_bf16(o2, "o2");
  TORCH_CHECK(o1.is_contiguous() && o2.is_contiguous() && lse1.is_contiguous() && lse2.is_contiguous() && o1.sizes() == o2.sizes(), "contiguous tensors of one shape");
  TORCH_CHECK(lse1.scalar_type() == torch::kFloat32 && lse2.scalar_type() == torch::kFloat32 && lse1.numel() == lse2.numel(), "lse must be fp32");
  const c10::cuda::CUDAGuard guard(o1.device());
  const int D = (int)o1.size(-1), rows = (int)(o1.numel() / D);
  TORCH_CHECK(lse1.numel() == rows, "one lse per (token, head)");
  auto out = torch::empty_like(o1);
  auto lse = torch::empty_like(lse1);
  TORCH_CHECK(oc::merge_attn_states_launch(o1.data_ptr(), lse1.data_ptr<float>(), o2.data_ptr(), lse2.data_ptr<float>(), out.data_ptr(), lse.data_ptr<float>(),
                                           rows, D, cur_stream()) == 0, "merge_attn_states failed");
  return {out, lse};
}

torch::Tensor argmax(torch::Tensor x) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.stride(1) == 1, "x must be a CUDA [B, V] matrix");
  TORCH_CHECK(x.scalar_type() == torch::kBFloat16 || x.scalar_type() == torch::kFloat32, "argmax supports bf16 and fp32");
  const c10::cuda::CUDAGuard guard(x.device());
  auto out = torch::empty({x.size(0)}, x.options().dtype(torch::kInt64));
  auto packed = torch::zeros({x.size(0)}, x.options().dtype(torch::kInt64));   // one (value key, ~index) word per row, folded with atomicMax
  TORCH_CHECK(oc::argmax_launch(x.data_ptr(), x.scalar_type() == torch::kFloat32, out.data_ptr<int64_t>() ? (long long*)out.data_ptr<int64_t>() : nullptr,
                                (unsigned long long*)packed.data_ptr<int64_t>(), (int)x.size(0), (int)x.size(1), x.stride(0), cur_stream()) == 0,
              "argmax failed");
  return out;
}

// Gated-DeltaNet: conv + SiLU with rolling state, then the gated delta rule with fused gating. `mixed` is the pre-conv [T, 2*Hk*K + Hv*V]
// slice; returns o [T, Hv*V]. spec_state (optional) receives the recurrent state after every token; write_state=false leaves slots alone.
torch::Tensor gdn_forward(torch::Tensor mixed, torch::Tensor b_in, torch::Tensor a_in, torch::Tensor conv_w, torch::Tensor A_log, torch::Tensor dt_bias,
                          torch::Tensor conv_state, torch::Tensor ssm_state, torch::Tensor qsl, torch::Tensor slots, torch::Tensor has_init,
                          int64_t Hk, int64_t Hv, int64_t K, int64_t V, bool write_state, c10::optional<torch::Tensor> spec_state,
                          c10::optional<torch::Tensor> chunk_meta, int64_t num_chunks, int64_t num_long, int64_t chunk_min_len) {
  check_bf16(mixed, "mixed");
  check_bf16(conv_w, "conv_w");
  check_bf16(conv_state, "conv_state");
  TORCH_CHECK(mixed.dim() == 2 && mixed.stride(1) == 1, "mixed must be [T, C] with unit inner stride");
  TORCH_CHECK(ssm_state.scalar_type() == torch::kFloat32 && ssm_state.is_contiguous() && conv_state.is_contiguous(), "states must be contiguous (fp32 recurrent state)");
  TORCH_CHECK(qsl.scalar_type() == torch::kInt32 && slots.scalar_type() == torch::kInt32 && has_init.scalar_type() == torch::kInt32, "metadata must be int32");
  TORCH_CHECK(a_in.stride(1) == 1 && b_in.stride(1) == 1 && a_in.stride(0) == b_in.stride(0), "a/b must share a row pitch");
  const c10::cuda::CUDAGuard guard(mixed.device());
  const int T = (int)mixed.size(0), C = (int)mixed.size(1), R = (int)slots.size(0);
  TORCH_CHECK(C == 2 * Hk * K + Hv * V, "mixed width does not match the head layout");
  auto y = torch::empty({T, C}, mixed.options());
  auto out = torch::empty({T, Hv * V}, mixed.options());
  if (T == 0) return out;
  oc::GdnConvParams cp{};
  cp.x = (const __nv_bfloat16*)mixed.data_ptr();
  cp.ldx = mixed.stride(0);
  cp.w = (const __nv_bfloat16*)conv_w.data_ptr();
  cp.y = (__nv_bfloat16*)y.data_ptr();
  cp.conv_state = (__nv_bfloat16*)conv_state.data_ptr();
  cp.query_start_loc = qsl.data_ptr<int>();
  cp.state_slots = slots.data_ptr<int>();
  cp.has_initial_state = has_init.data_ptr<int>();
  cp.T = T; cp.R = R; cp.C = C; cp.kw = (int)conv_w.size(1);
  TORCH_CHECK(conv_state.size(1) == C && conv_state.size(2) == cp.kw - 1, "conv_state must be [slots, C, kw-1]");
  TORCH_CHECK(oc::gdn_conv_launch(cp, cur_stream()) == 0, "gdn conv launch failed");
  oc::GdnParams p{};
  const __nv_bfloat16* yb = (const __nv_bfloat16*)y.data_ptr();
  p.q = yb; p.k = yb + Hk * K; p.v = yb + 2 * Hk * K;
  p.ld_qkv = C;
  p.a = (const __nv_bfloat16*)a_in.data_ptr();
  p.b = (const __nv_bfloat16*)b_in.data_ptr();
  p.ld_ba = a_in.stride(0);
  p.A_log = A_log.data_ptr<float>();
  p.dt_bias = dt_bias.data_ptr<float>();
  p.state = ssm_state.data_ptr<float>();
  p.out = (__nv_bfloat16*)out.data_ptr();
  p.query_start_loc = cp.query_start_loc; p.state_slots = cp.state_slots; p.has_initial_state = cp.has_initial_state;
  p.R = R; p.Hk = (int)Hk; p.Hv = (int)Hv; p.K = (int)K; p.V = (int)V;
  p.write_state = write_state ? 1 : 0;
  if (spec_state.has_value()) {
    TORCH_CHECK(spec_state->scalar_type() == torch::kFloat32 && spec_state->is_contiguous() && spec_state->dim() == 5 && spec_state->size(0) >= R, "spec_state must be fp32 [R, q, Hv, K, V]");
    p.spec_state = spec_state->data_ptr<float>();
    p.spec_q = (int)spec_state->size(1);
  }
  const bool chunked = chunk_meta.has_value() && num_long > 0 && num_chunks > 0 && !spec_state.has_value();
  p.skip_min_len = chunked ? (int)chunk_min_len : 0;
  int rc = oc::gdn_recurrent_launch(p, cur_stream());
  TORCH_CHECK(rc == 0, "gdn recurrence launch failed: ", rc, " (K and V must be 128)");
  if (chunked) {
    // chunk_meta (int32): [chunk_req (num_chunks) | chunk_t0 (num_chunks) | long_req (num_long) | long_chunk0 (num_long)]
    TORCH_CHECK(chunk_meta->scalar_type() == torch::kInt32 && chunk_meta->is_contiguous() && chunk_meta->numel() >= 2 * num_chunks + 2 * num_long,
                "chunk metadata must be int32 [2 * chunks + 2 * sequences]");
    auto ws = torch::empty({(int64_t)oc::gdn_chunk_workspace_elems((int)num_chunks, (int)Hv)}, mixed.options());
    oc::GdnChunkParams c{};
    c.q = p.q; c.k = p.k; c.v = p.v; c.ld_qkv = p.ld_qkv; c.a = p.a; c.b = p.b; c.ld_ba = p.ld_ba; c.A_log = p.A_log; c.dt_bias = p.dt_bias;
    c.state = p.state; c.out = p.out; c.query_start_loc = p.query_start_loc; c.state_slots = p.state_slots; c.has_initial_state = p.has_initial_state;
    c.Hk = p.Hk; c.Hv = p.Hv; c.K = p.K; c.V = p.V; c.write_state = 1;
    c.ws = (__nv_bfloat16*)ws.data_ptr();
    const int* m = chunk_meta->data_ptr<int>();
    c.chunk_req = m; c.chunk_t0 = m + num_chunks; c.long_req = m + 2 * num_chunks; c.long_chunk0 = m + 2 * num_chunks + num_long;
    c.num_chunks = (int)num_chunks; c.num_long = (int)num_long;
    rc = oc::gdn_chunk_launch(c, cur_stream());
    TORCH_CHECK(rc == 0, "gdn chunked prefill launch failed: ", rc);
  }
  return out;
}

// Speculative commit of the conv state: recompute each slot from the pre-chunk snapshot and the first n_valid inputs of the chunk.
void gdn_conv_commit(torch::Tensor mixed, torch::Tensor conv_state, torch::Tensor prev_state, torch::Tensor n_valid, torch::Tensor qsl,
                     torch::Tensor slots, torch::Tensor has_init, int64_t kw) {
  const c10::cuda::CUDAGuard guard(mixed.device());
  oc::GdnConvParams cp{};
  cp.x = (const __nv_bfloat16*)mixed.data_ptr();
  cp.ldx = mixed.stride(0);
  cp.conv_state = (__nv_bfloat16*)conv_state.data_ptr();
  cp.prev_state = (const __nv_bfloat16*)prev_state.data_ptr();
  cp.n_valid = n_valid.data_ptr<int>();
  cp.query_start_loc = qsl.data_ptr<int>();
  cp.state_slots = slots.data_ptr<int>();
  cp.has_initial_state = has_init.data_ptr<int>();
  cp.T = (int)mixed.size(0); cp.R = (int)slots.size(0); cp.C = (int)mixed.size(1); cp.kw = (int)kw;
  TORCH_CHECK(oc::gdn_conv_commit_launch(cp, cur_stream()) == 0, "gdn conv commit failed");
}

// Temperature / min-p / top-k / top-p / random draw for each row of `logits` in one kernel. Returns the token ids [B] (int64).
torch::Tensor sample(torch::Tensor logits, torch::Tensor temperature, c10::optional<torch::Tensor> top_k, c10::optional<torch::Tensor> top_p,
                     c10::optional<torch::Tensor> min_p, torch::Tensor seeds, c10::optional<torch::Tensor> kept) {
  TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.stride(1) == 1, "logits must be a CUDA [B, V] matrix");
  const bool f32 = logits.scalar_type() == torch::kFloat32;
  TORCH_CHECK(f32 || logits.scalar_type() == torch::kBFloat16, "logits must be fp32 or bf16");
  const int64_t B = logits.size(0);
  auto chk = [&](const torch::Tensor& t, c10::ScalarType ty, const char* name) {
    TORCH_CHECK(t.is_cuda() && t.scalar_type() == ty && t.is_contiguous() && t.numel() == B, name, " must be a contiguous CUDA vector with one entry per row");
  };
  chk(temperature, torch::kFloat32, "temperature");
  chk(seeds, torch::kInt64, "seeds");
  const c10::cuda::CUDAGuard guard(logits.device());
  oc::SampleParams p{};
  p.logits = logits.data_ptr();
  p.is_fp32 = f32;
  p.ld = logits.stride(0);
  p.B = (int)B;
  p.V = (int)logits.size(1);
  p.temperature = temperature.data_ptr<float>();
  if (top_k.has_value()) { chk(*top_k, torch::kInt32, "top_k"); p.top_k = top_k->data_ptr<int>(); }
  if (top_p.has_value()) { chk(*top_p, torch::kFloat32, "top_p"); p.top_p = top_p->data_ptr<float>(); }
  if (min_p.has_value()) { chk(*min_p, torch::kFloat32, "min_p"); p.min_p = min_p->data_ptr<float>(); }
  p.seeds = (const unsigned long long*)seeds.data_ptr<int64_t>();
  auto out = torch::empty({B}, logits.options().dtype(torch::kInt64));
  p.out = (long long*)out.data_ptr<int64_t>();
  if (kept.has_value()) {
    TORCH_CHECK(kept->is_cuda() && kept->scalar_type() == torch::kUInt8 && kept->is_contiguous() && kept->numel() == B * logits.size(1), "kept must be uint8 [B, V]");
    p.kept = kept->data_ptr<uint8_t>();
  }
  TORCH_CHECK(oc::sample_launch(p, cur_stream()) == 0, "sample launch failed");
  return out;
}

torch::Tensor rejection_sample(torch::Tensor draft_ids, torch::Tensor num_draft, torch::Tensor target_logits, torch::Tensor bonus_ids,
                               torch::Tensor uniforms, c10::optional<torch::Tensor> temperature, c10::optional<torch::Tensor> synth_rates,
                               int64_t seed, bool use_noise) {
  TORCH_CHECK(target_logits.is_cuda() && target_logits.dim() == 3 && target_logits.stride(2) == 1, "target_logits must be CUDA [B, k+1, V]");
  TORCH_CHECK(draft_ids.scalar_type() == torch::kInt64 && num_draft.scalar_type() == torch::kInt64 && bonus_ids.scalar_type() == torch::kInt64, "ids must be int64");
  TORCH_CHECK(uniforms.scalar_type() == torch::kFloat64 && uniforms.is_contiguous() && draft_ids.is_contiguous(), "uniforms must be contiguous float64");
  const c10::cuda::CUDAGuard guard(target_logits.device());
  const int B = (int)draft_ids.size(0), k = (int)draft_ids.size(1), V = (int)target_logits.size(2);
  TORCH_CHECK(target_logits.size(0) == B && target_logits.size(1) >= k, "target_logits shape mismatch");
  const bool f32 = target_logits.scalar_type() == torch::kFloat32;
  TORCH_CHECK(f32 || target_logits.scalar_type() == torch::kBFloat16, "logits must be fp32 or bf16");
  auto out = torch::empty({B, k + 1}, draft_ids.options());
  auto stats = torch::empty({std::max(B * k, 1) * (int64_t)sizeof(oc::RowStats)}, draft_ids.options().dtype(torch::kUInt8));
  const float* tp = temperature.has_value() ? temperature->data_ptr<float>() : nullptr;
  const float* sr = synth_rates.has_value() ? synth_rates->data_ptr<float>() : nullptr;
  int rc = oc::rejection_launch(target_logits.data_ptr(), f32, (const long long*)draft_ids.data_ptr<int64_t>(), (const long long*)num_draft.data_ptr<int64_t>(),
                                (const long long*)bonus_ids.data_ptr<int64_t>(), uniforms.data_ptr<double>(), tp, sr, (oc::RowStats*)stats.data_ptr(),
                                (long long*)out.data_ptr<int64_t>(), B, k, V, target_logits.stride(0), target_logits.stride(1), (unsigned long long)seed,
                                use_noise ? 1 : 0, cur_stream());
  TORCH_CHECK(rc == 0, "rejection sampler launch failed");
  return out;
}

std::tuple<torch::Tensor, torch::Tensor> route(torch::Tensor logits, c10::optional<torch::Tensor> bias, int64_t k, int64_t n_group, int64_t topk_group,
                                               bool sigmoid, bool renormalize, double scaling) {
  check_bf16(logits, "router logits");
  TORCH_CHECK(logits.dim() == 2 && logits.stride(1) == 1, "router logits must be [T, E]");
  const c10::cuda::CUDAGuard guard(logits.device());
  const int T = (int)logits.size(0);
  auto w = torch::empty({T, k}, logits.options().dtype(torch::kFloat32));
  auto ids = torch::empty({T, k}, logits.options().dtype(torch::kInt32));
  oc::RouteParams p{};
  p.logits = (const __nv_bfloat16*)logits.data_ptr();
  p.ld = logits.stride(0);
  p.bias = bias.has_value() ? bias->data_ptr<float>() : nullptr;
  p.topk_w = w.data_ptr<float>();
  p.topk_ids = ids.data_ptr<int>();
  p.T = T; p.E = (int)logits.size(1); p.k = (int)k; p.n_group = (int)n_group; p.topk_group = (int)topk_group;
  p.sigmoid = sigmoid ? 1 : 0; p.renormalize = renormalize ? 1 : 0; p.scaling = (float)scaling;
  int rc = oc::route_launch(p, cur_stream());
  TORCH_CHECK(rc == 0, "router launch failed (needs E % 32 == 0, E <= 512, k <= 16)");
  return {w, ids};
}

// One grouped GEMM of the MoE chain over `rows` slot rows, driven by a device-built work list.
static void moe_gemm_run(const torch::Tensor& in, const torch::Tensor& w, const c10::optional<torch::Tensor>& sz, int n_rows, torch::Tensor& out, int Kd,
                         int N, int n_out, int epi, const int4* wl, const int* cnt, int cap, int rows, int tn, int wkind, int group_ktiles,
                         torch::Tensor& counters) {
  oc::GemmParams p{};
  p.T = rows; p.K = Kd; p.N = N; p.n_rows = n_rows; p.n_out = n_out; p.epi = epi; p.group_ktiles = wkind == 0 ? 1 : group_ktiles;
  p.wkind = wkind;
  if (wkind != 0) {
    p.w4 = (const uint8_t*)w.data_ptr();
    p.w4_sz = (const uint32_t*)sz->data_ptr();
    p.n_pad = n_rows;
  }
  p.out = (__nv_bfloat16*)out.data_ptr(); p.ldo = (int)out.stride(0);
  p.ws = nullptr; p.counters = (int*)counters.data_ptr(); p.max_counters = 0;
  p.work = wl; p.work_count = cnt; p.work_capacity = cap;
  p.tn = tn; p.num_t_tiles = 1; p.num_n_tiles = 1; p.splits = 1; p.ktiles_per_split = Kd / 64;
  oc::gemm_plan_stages(p, wkind != 0);
  int r = oc::gemm_launch(p, in.data_ptr(), (int)in.stride(0), wkind == 0 ? w.data_ptr() : nullptr, wkind == 0 ? (int)w.stride(0) : 0, sm_count(),
                          cur_stream());
  TORCH_CHECK(r == 0, "grouped gemm launch failed: ", r);
}

// Routed-expert path of one MoE layer: slots -> grouped GEMM (w13, SiLU*mul) -> grouped GEMM (w2) -> weighted combine.
// w13: bf16 [E_local * 2I, H] with each expert's gate|up rows interleaved in blocks of 16; w2: bf16 [E_local * H, I].
// With `wkind` > 0 the expert weights are packed tiles (see gemm) and w13_sz / w2_sz their scale tables; I2 and group_ktiles
// (64-wide k tiles per scale row of the tables) then come from the caller.
torch::Tensor fused_moe(torch::Tensor x, torch::Tensor w13, torch::Tensor w2, torch::Tensor topk_w, torch::Tensor topk_ids, int64_t E_local,
                        int64_t e_off, torch::Tensor ws, torch::Tensor counters, int64_t wkind, c10::optional<torch::Tensor> w13_sz,
                        c10::optional<torch::Tensor> w2_sz, int64_t I2_packed, int64_t group_ktiles) {
  check_bf16(x, "x");
  if (wkind == 0) {
    check_bf16(w13, "w13");
    check_bf16(w2, "w2");
  } else {
    TORCH_CHECK(wkind >= 1 && wkind <= 3 && w13_sz.has_value() && w2_sz.has_value() && I2_packed > 0 && group_ktiles >= 1, "packed experts need scale tables");
  }
  TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1 && w13.is_contiguous() && w2.is_contiguous(), "bad layouts");
  TORCH_CHECK(topk_ids.scalar_type() == torch::kInt32 && topk_ids.is_contiguous() && topk_w.scalar_type() == torch::kFloat32 && topk_w.is_contiguous(),
              "routing tensors must be contiguous int32 ids / fp32 weights");
  const c10::cuda::CUDAGuard guard(x.device());
  const int T = (int)x.size(0), H = (int)x.size(1), k = (int)topk_ids.size(1);
  const int I2 = wkind == 0 ? (int)(w13.size(0) / E_local) : (int)I2_packed, I = I2 / 2;
  if (wkind == 0) {
    TORCH_CHECK(w13.size(1) == H && w2.size(0) == E_local * H && w2.size(1) == I, "expert weight shapes do not match");
  } else {
    const size_t tb = wkind == 2 ? 8192 : 4096;
    TORCH_CHECK((size_t)w13.numel() * w13.element_size() >= (size_t)(E_local * I2 / 128) * (H / 64) * tb &&
                (size_t)w2.numel() * w2.element_size() >= (size_t)(E_local * H / 128) * (I / 64) * tb, "packed expert weights are too small");
    TORCH_CHECK((size_t)w13_sz->numel() >= (size_t)((H / 64 + group_ktiles - 1) / group_ktiles) * E_local * I2 &&
                (size_t)w2_sz->numel() >= (size_t)((I / 64 + group_ktiles - 1) / group_ktiles) * E_local * H, "expert scale tables are too small");
  }
  TORCH_CHECK(I2 % 128 == 0 && H % 128 == 0 && H % 64 == 0 && I % 64 == 0, "expert dims must be multiples of 128 (rows) and 64 (k)");
  auto y = torch::empty({T, H}, x.options());
  if (T == 0) return y;
  const int n_pairs = T * k;
  const int avg = (n_pairs + (int)E_local - 1) / (int)E_local;
  const int tn = avg <= 32 ? 32 : avg <= 64 ? 64 : (avg <= 128 || wkind != 0) ? 128 : 256;  // packed kinds share TMEM with the weight ring
  const int n1 = I2 / 128, n2 = H / 128;
  const int max_tt = (n_pairs + tn - 1) / tn + (int)E_local;
  auto iopt = x.options().dtype(torch::kInt32);
  auto meta = torch::empty({3 * E_local + 8 + n_pairs}, iopt);
  auto work = torch::empty({(int64_t)max_tt * (n1 + n2) * 4}, iopt);
  auto xs = torch::empty({n_pairs, H}, x.options());
  auto a1 = torch::empty({n_pairs, I}, x.options());
  auto a2 = torch::empty({n_pairs, H}, x.options());
  int* mp = meta.data_ptr<int>();
  oc::MoePlanParams pp{};
  pp.counts = mp; pp.offsets = mp + E_local; pp.cursor = mp + 2 * E_local + 1; pp.total_slots = mp + 3 * E_local + 1; pp.work_count = mp + 3 * E_local + 2;
  int* slot_of = mp + 3 * E_local + 8;
  pp.work1 = (int4*)work.data_ptr<int>();
  pp.work2 = pp.work1 + (size_t)max_tt * n1;
  TORCH_CHECK(((uintptr_t)pp.work2 & 15) == 0, "work list alignment");
  pp.E = (int)E_local; pp.tn = tn; pp.n1 = n1; pp.n2 = n2;
  int rc = oc::moe_prepare_launch(pp, topk_ids.data_ptr<int>(), n_pairs, k, (int)e_off, slot_of, x.data_ptr(), x.stride(0), xs.data_ptr(), H, cur_stream());
  TORCH_CHECK(rc == 0, "moe prepare failed: ", rc);
  auto run = [&](const torch::Tensor& in, const torch::Tensor& w, const c10::optional<torch::Tensor>& sz, int n_rows, torch::Tensor& out, int Kd, int N,
                 int n_out, int epi, const int4* wl, const int* cnt, int cap) {
    moe_gemm_run(in, w, sz, n_rows, out, Kd, N, n_out, epi, wl, cnt, cap, n_pairs, tn, (int)wkind, (int)group_ktiles, counters);
  };
  run(xs, w13, w13_sz, (int)E_local * I2, a1, H, I2, I, oc::EPI_SILU_MUL, pp.work1, pp.work_count, max_tt * n1);
  run(a1, w2, w2_sz, (int)E_local * H, a2, I, H, H, oc::EPI_STORE, pp.work2, pp.work_count + 1, max_tt * n2);
  rc = oc::moe_combine_launch(a2.data_ptr(), slot_of, topk_w.data_ptr<float>(), y.data_ptr(), T, k, H, cur_stream());
  TORCH_CHECK(rc == 0, "moe combine failed");
  return y;
}

// Expert-parallel MoE with the token exchange over peer memory (see ep_a2a.cu): `x`, `topk_w`, `topk_ids` describe this rank's
// own tokens (expert ids are global); `slabs` are every rank's exchange slab and `offs` the six byte offsets of its areas
// (counts, flags, recv rows, recv meta, returned rows, gather); `state` is this rank's int32 scratch [8 + 2 E]. Returns this
// rank's combined rows; with `gather` every rank's rows are also stored into every slab's gather area at row `t_off`.
torch::Tensor fused_moe_a2a(torch::Tensor x, torch::Tensor w13, torch::Tensor w2, torch::Tensor topk_w, torch::Tensor topk_ids, int64_t E_local,
                            torch::Tensor counters, int64_t wkind, c10::optional<torch::Tensor> w13_sz, c10::optional<torch::Tensor> w2_sz,
                            int64_t I2_packed, int64_t group_ktiles, std::vector<int64_t> slabs, std::vector<int64_t> offs, torch::Tensor state,
                            int64_t rank, int64_t cap, int64_t ret_rows, int64_t T_total, int64_t t_off, bool gather, int64_t wait_ns) {
  check_bf16(x, "x");
  const int n = (int)slabs.size();
  TORCH_CHECK(n >= 2 && n <= oc::kMaxRanks && offs.size() == 6 && rank >= 0 && rank < n, "bad rank tables");
  TORCH_CHECK(x.dim() == 2 && (x.size(0) == 0 || x.stride(1) == 1) && w13.is_contiguous() && w2.is_contiguous(), "bad layouts");
  TORCH_CHECK(topk_ids.scalar_type() == torch::kInt32 && topk_ids.is_contiguous() && topk_w.scalar_type() == torch::kFloat32 && topk_w.is_contiguous(),
              "routing tensors must be contiguous int32 ids / fp32 weights");
  const c10::cuda::CUDAGuard guard(x.device());
  const int T = (int)x.size(0), H = (int)x.size(1), k = (int)topk_ids.size(1), E = (int)E_local * n;
  const int I2 = wkind == 0 ? (int)(w13.size(0) / E_local) : (int)I2_packed, I = I2 / 2;
  TORCH_CHECK(I2 % 128 == 0 && H % 128 == 0 && I % 64 == 0, "expert dims must be multiples of 128 (rows) and 64 (k)");
  TORCH_CHECK((int64_t)T * k <= ret_rows && t_off + T <= T_total && cap > 0, "tokens exceed the exchange slab");
  TORCH_CHECK(state.scalar_type() == torch::kInt32 && state.numel() >= 8 + 2 * E, "exchange state too small");
  if (wkind != 0) TORCH_CHECK(w13_sz.has_value() && w2_sz.has_value() && I2_packed > 0 && group_ktiles >= 1, "packed experts need scale tables");
  auto y = torch::empty({T, H}, x.options());
  const int avg = (int)((T_total * k + E - 1) / E);
  const int tn = avg <= 32 ? 32 : avg <= 64 ? 64 : (avg <= 128 || wkind != 0) ? 128 : 256;
  const int n1 = I2 / 128, n2 = H / 128;
  const int max_tt = ((int)cap + tn - 1) / tn + (int)E_local;
  auto iopt = x.options().dtype(torch::kInt32);
  auto meta = torch::empty({3 * E_local + 8}, iopt);
  auto work = torch::empty({(int64_t)max_tt * (n1 + n2) * 4}, iopt);
  auto a1 = torch::empty({cap, I}, x.options());
  auto a2 = torch::empty({cap, H}, x.options());
  int* mp = meta.data_ptr<int>();
  oc::MoePlanParams pp{};
  pp.counts = mp; pp.offsets = mp + E_local; pp.cursor = mp + 2 * E_local + 1; pp.total_slots = mp + 3 * E_local + 1; pp.work_count = mp + 3 * E_local + 2;
  pp.work1 = (int4*)work.data_ptr<int>();
  pp.work2 = pp.work1 + (size_t)max_tt * n1;
  pp.E = (int)E_local; pp.tn = tn; pp.n1 = n1; pp.n2 = n2;
  oc::EpParams ep{};
  for (int i = 0; i < n; ++i) ep.slab[i] = (char*)(uintptr_t)slabs[i];
  ep.off_counts = (size_t)offs[0]; ep.off_flags = (size_t)offs[1]; ep.off_recv_x = (size_t)offs[2]; ep.off_recv_meta = (size_t)offs[3];
  ep.off_ret = (size_t)offs[4]; ep.off_gather = (size_t)offs[5];
  ep.ids = topk_ids.data_ptr<int>();
  ep.x = (const __nv_bfloat16*)x.data_ptr(); ep.ldx = T ? x.stride(0) : H;
  int* sp = state.data_ptr<int>();
  ep.seq = sp; ep.done = sp + 1; ep.send_base = sp + 8; ep.cursor = sp + 8 + E;
  ep.counts_local = pp.counts; ep.total_slots = pp.total_slots;
  ep.n = n; ep.me = (int)rank; ep.E = E; ep.E_local = (int)E_local; ep.k = k; ep.H = H; ep.T = T; ep.n_pairs = T * k; ep.cap = (int)cap;
  ep.ret_rows = (int)ret_rows; ep.gather = gather ? 1 : 0; ep.t_off = (int)t_off; ep.wait_ns = (unsigned long long)wait_ns;
  auto st = cur_stream();
  int rc = oc::ep_count_exchange_launch(ep, st);
  TORCH_CHECK(rc == 0, "expert-parallel count exchange failed: ", rc);
  TORCH_CHECK(oc::moe_plan_launch(pp, st) == 0, "moe plan failed");
  TORCH_CHECK(oc::ep_dispatch_launch(ep, sm_count(), st) == 0, "expert-parallel dispatch failed");
  auto xs = torch::from_blob(ep.slab[rank] + ep.off_recv_x, {cap, (int64_t)H}, x.options());
  moe_gemm_run(xs, w13, w13_sz, (int)E_local * I2, a1, H, I2, I, oc::EPI_SILU_MUL, pp.work1, pp.work_count, max_tt * n1, (int)cap, tn, (int)wkind,
               (int)group_ktiles, counters);
  moe_gemm_run(a1, w2, w2_sz, (int)E_local * H, a2, I, H, H, oc::EPI_STORE, pp.work2, pp.work_count + 1, max_tt * n2, (int)cap, tn, (int)wkind,
               (int)group_ktiles, counters);
  TORCH_CHECK(oc::ep_return_launch(ep, a2.data_ptr(), sm_count(), st) == 0, "expert-parallel return failed");
  TORCH_CHECK(oc::ep_combine_launch(ep, topk_w.data_ptr<float>(), y.data_ptr(), sm_count(), st) == 0, "expert-parallel combine failed");
  return y;
}

torch::Tensor mla_decode(torch::Tensor q_abs, torch::Tensor q_rope, torch::Tensor cache, torch::Tensor qsl, torch::Tensor seq_lens,
                         torch::Tensor block_table, double scale, int64_t max_q_len, int64_t splits, c10::optional<torch::Tensor> ws_o,
                         c10::optional<torch::Tensor> ws_ml) {
  check_bf16(q_abs, "q_abs");
  check_bf16(q_rope, "q_rope");
  check_bf16(cache, "latent cache");
  TORCH_CHECK(q_abs.is_contiguous() && q_rope.is_contiguous() && cache.is_contiguous() && cache.dim() == 3, "q and cache must be contiguous");
  const c10::cuda::CUDAGuard guard(q_abs.device());
  oc::MlaParams p{};
  p.T = (int)q_abs.size(0); p.H = (int)q_abs.size(1); p.kv_lora = (int)q_abs.size(2); p.rope = (int)q_rope.size(2);
  TORCH_CHECK(cache.size(2) == p.kv_lora + p.rope, "cache width must be kv_lora + rope");
  auto out = torch::empty({p.T, p.H, p.kv_lora}, q_abs.options());
  p.q_abs = (const __nv_bfloat16*)q_abs.data_ptr(); p.q_rope = (const __nv_bfloat16*)q_rope.data_ptr();
  p.cache = (const __nv_bfloat16*)cache.data_ptr(); p.out = (__nv_bfloat16*)out.data_ptr();
  p.query_start_loc = qsl.data_ptr<int>(); p.seq_lens = seq_lens.data_ptr<int>(); p.block_table = block_table.data_ptr<int>();
  p.bt_stride = (int)block_table.stride(0); p.R = (int)seq_lens.size(0);
  p.bs = (int)cache.size(1); p.bs_shift = 0;
  while ((1 << p.bs_shift) < p.bs) ++p.bs_shift;
  p.max_q_len = (int)max_q_len; p.splits = (int)splits; p.scale = (float)scale;
  if (splits > 1) {
    TORCH_CHECK(ws_o.has_value() && ws_ml.has_value() && (size_t)ws_o->numel() >= (size_t)splits * p.T * p.H * p.kv_lora &&
                (size_t)ws_ml->numel() >= (size_t)splits * p.T * p.H * 2, "split-KV workspace too small");
    p.ws_o = ws_o->data_ptr<float>(); p.ws_ml = ws_ml->data_ptr<float>();
  }
  int rc = oc::mla_decode_launch(p, cur_stream());
  TORCH_CHECK(rc == 0, "mla decode launch failed: ", rc, " (needs kv_lora 512, rope 64)");
  return out;
}

// Enqueues one small copy per translation unit's status word into `pinned` (int32, >= 16 entries, pinned host memory) on the current
// stream; the caller reads them after an event recorded behind this call (async scheduling: no device-wide synchronisation).
void read_status_async(torch::Tensor pinned) {
  TORCH_CHECK(pinned.scalar_type() == torch::kInt32 && pinned.numel() >= 16 && !pinned.is_cuda() && pinned.is_pinned(), "need 16 pinned int32 words");
  unsigned int* p = reinterpret_cast<unsigned int*>(pinned.data_ptr<int>());
  auto st = cur_stream();
  oc::attention_read_status_async(p + 0, st);
  oc::attention_tc_read_status_async(p + 1, st);
  oc::comm_read_status_async(p + 2, st);
  oc::elementwise_read_status_async(p + 3, st);
  oc::ep_read_status_async(p + 4, st);
  oc::gdn_read_status_async(p + 5, st);
  oc::gemm_read_status_async(p + 6, st);
  oc::mla_read_status_async(p + 7, st);
  oc::moe_read_status_async(p + 8, st);
  oc::sampling_read_status_async(p + 9, st);
}

int64_t read_status(bool clear) {
  return (int64_t)(oc::gemm_read_status(clear) | oc::elementwise_read_status(clear) | oc::attention_read_status(clear) | oc::attention_tc_read_status(clear) |
                   oc::comm_read_status(clear) | oc::gdn_read_status(clear) | oc::sampling_read_status(clear) | oc::moe_read_status(clear) | oc::mla_read_status(clear) | oc::ep_read_status(clear));
}

// ---- symmetric slab + peer-memory reductions
int64_t comm_alloc(int64_t bytes) {
  void* p = nullptr;
  TORCH_CHECK(oc::comm_alloc((size_t)bytes, &p) == 0, "cudaMalloc of the symmetric slab failed");
  return (int64_t)(uintptr_t)p;
}
void comm_free(int64_t ptr) { oc::comm_free((void*)(uintptr_t)ptr); }
py::bytes comm_export(int64_t ptr) {
  char h[64];
  TORCH_CHECK(oc::comm_export((void*)(uintptr_t)ptr, h) == 0, "cudaIpcGetMemHandle failed");
  return py::bytes(h, 64);
}
int64_t comm_import(const std::string& handle) {
  TORCH_CHECK(handle.size() == 64, "an IPC handle is 64 bytes");
  void* p = nullptr;
  TORCH_CHECK(oc::comm_import(handle.data(), &p) == 0, "cudaIpcOpenMemHandle failed (is peer access available?)");
  return (int64_t)(uintptr_t)p;
}
void comm_unimport(int64_t ptr) { oc::comm_unimport((void*)(uintptr_t)ptr); }
torch::Tensor comm_tensor(int64_t ptr, int64_t byte_offset, std::vector<int64_t> shape, int64_t dtype_code, int64_t device) {
  auto dt = dtype_code == 0 ? torch::kBFloat16 : dtype_code == 1 ? torch::kInt32 : torch::kUInt8;
  return torch::from_blob((void*)((uintptr_t)ptr + (uintptr_t)byte_offset), shape, torch::TensorOptions().dtype(dt).device(torch::kCUDA, (int)device));
}

void tp_reduce_norm(std::vector<int64_t> part, std::vector<int64_t> flags, torch::Tensor seq_local, std::vector<int64_t> x_out,
                    c10::optional<torch::Tensor> residual_in, c10::optional<torch::Tensor> residual_out, c10::optional<torch::Tensor> w,
                    int64_t T, int64_t H, int64_t rank, int64_t mode, bool gemma, int64_t phase, double eps, int64_t wait_ns, int64_t grid,
                    std::vector<int64_t> lam, int64_t lam_buf_stride, int64_t lam_src_stride, int64_t lam_ctr, bool lam_pushed) {
  const int tp = (int)part.size();
  TORCH_CHECK(tp >= 2 && tp <= oc::kMaxRanks && (int)flags.size() == tp && (int)x_out.size() == tp, "bad rank tables");
  const c10::cuda::CUDAGuard guard(seq_local.device());
  oc::CommParams p{};
  for (int i = 0; i < tp; ++i) {
    p.part[i] = (const __nv_bfloat16*)(uintptr_t)part[i];
    p.flags[i] = (int*)(uintptr_t)flags[i];
    p.x_out[i] = (__nv_bfloat16*)(uintptr_t)x_out[i];
  }
  p.seq_local = seq_local.data_ptr<int>();
  p.residual_in = residual_in.has_value() ? (const __nv_bfloat16*)residual_in->data_ptr() : nullptr;
  p.residual_out = residual_out.has_value() ? (__nv_bfloat16*)residual_out->data_ptr() : nullptr;
  p.w = w.has_value() ? (const __nv_bfloat16*)w->data_ptr() : nullptr;
  if (residual_in.has_value()) TORCH_CHECK(residual_in->is_contiguous(), "residual must be contiguous");
  p.T = (int)T;
  p.H = (int)H;
  p.tp = tp;
  p.rank = (int)rank;
  p.mode = (int)mode;
  p.gemma = gemma ? 1 : 0;
  p.phase = (int)phase;
  p.eps = (float)eps;
  p.wait_ns = (unsigned long long)wait_ns;
  TORCH_CHECK(lam.empty() || (int)lam.size() == tp, "bad arrival-buffer table");
  for (size_t i = 0; i < lam.size(); ++i) p.lam[i] = (__nv_bfloat16*)(uintptr_t)lam[i];
  p.lam_buf_stride = (long long)lam_buf_stride;
  p.lam_src_stride = (long long)lam_src_stride;
  p.lam_ctr = (int*)(uintptr_t)lam_ctr;
  p.lam_pushed = lam_pushed ? 1 : 0;
  int rc = oc::tp_reduce_norm_launch(p, (int)grid, cur_stream());
  TORCH_CHECK(rc == 0, "tp_reduce_norm launch failed: ", rc);
}

std::vector<int64_t> gemm_kernel_info(int64_t wkind, int64_t small, int64_t smem) {
  int o[6] = {0};
  TORCH_CHECK(oc::gemm_kernel_info((int)wkind, (int)small, (int)smem, o) == 0, "no such kernel variant");
  return {o[0], o[1], o[2], o[3], o[4], o[5]};
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("gemm_kernel_info", &gemm_kernel_info);
  m.def("gemm", &gemm);
  m.def("rms_norm", &rms_norm);
  m.def("rms_norm_gated", &rms_norm_gated);
  m.def("silu_and_mul", &silu_and_mul);
  m.def("rope_and_cache", &rope_and_cache);
  m.def("paged_attention", &paged_attention);
  m.def("argmax", &argmax);
  m.def("merge_attn_states", &merge_attn_states);
  m.def("read_status", &read_status);
  m.def("read_status_async", &read_status_async);
  m.def("mla_decode", &mla_decode);
  m.def("fused_moe", &fused_moe);
  m.def("fused_moe_a2a", &fused_moe_a2a);
  m.def("rejection_sample", &rejection_sample);
  m.def("sample", &sample);
  m.def("route", &route);
  m.def("gdn_forward", &gdn_forward);
  m.def("gdn_conv_commit", &gdn_conv_commit);
  m.def("comm_alloc", &comm_alloc);
  m.def("comm_free", &comm_free);
  m.def("comm_export", &comm_export);
  m.def("comm_import", &comm_import);
  m.def("comm_unimport", &comm_unimport);
  m.def("comm_tensor", &comm_tensor);
  m.def("tp_reduce_norm", &tp_reduce_norm);
}
