"""Multi-head Latent Attention (DeepSeek-V2/V3) in absorbed (MQA-over-latent) form
(reference: models/deepseek_v2.py:870-1075; layers/attention/mla_attention.py:322,1297-1330 ``forward_mqa``;
CPU decode csrc/cpu/mla_decode.cpp). The cache stores one ``kv_lora + rope`` wide latent per token; ``W_UK`` is
folded into the query and ``W_UV`` applied to the attention output, so prefill and decode share one kernel."""
from __future__ import annotations

import torch
import torch.nn as nn

from onecat_vllm.config import ModelConfig
from onecat_vllm.layers.common import RMSNorm, get_rope
from onecat_vllm.layers.linear import ColumnParallelLinear, ReplicatedLinear, RowParallelLinear
from onecat_vllm.ops import ref
from onecat_vllm.parallel.state import get_state


def _rope_interleaved(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """GPT-J style (pairs (2i, 2i+1)), as DeepSeek uses for the rope part."""
    xf = x.float()
    x1, x2 = xf[..., 0::2], xf[..., 1::2]
    c, s = cos.unsqueeze(1), sin.unsqueeze(1)
    return torch.stack([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).flatten(-2).to(x.dtype)


class MLAAttention(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, prefix: str, device):
        super().__init__()
        tp = get_state().tp_size
        self.H = cfg.num_attention_heads // tp
        self.nope, self.rope_d, self.vd, self.lora = cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim, cfg.kv_lora_rank
        self.q_lora = cfg.q_lora_rank
        q, dt = cfg.quant, cfg.dtype
        qk = self.nope + self.rope_d
        if self.q_lora:
            self.q_a_proj = ReplicatedLinear(cfg.hidden_size, self.q_lora, quant=q, prefix=prefix + ".q_a_proj", dtype=dt)
            self.q_a_layernorm = RMSNorm(self.q_lora, cfg.rms_norm_eps, dtype=dt)
            self.q_b_proj = ColumnParallelLinear(self.q_lora, cfg.num_attention_heads * qk, quant=q, prefix=prefix + ".q_b_proj", dtype=dt)
        else:
            self.q_proj = ColumnParallelLinear(cfg.hidden_size, cfg.num_attention_heads * qk, quant=q, prefix=prefix + ".q_proj", dtype=dt)
        self.kv_a_proj_with_mqa = ReplicatedLinear(cfg.hidden_size, self.lora + self.rope_d, quant=q, prefix=prefix + ".kv_a_proj_with_mqa", dtype=dt)
        self.kv_a_layernorm = RMSNorm(self.lora, cfg.rms_norm_eps, dtype=dt)
        self.kv_b_proj = ColumnParallelLinear(self.lora, cfg.num_attention_heads * (self.nope + self.vd), quant=q, prefix=prefix + ".kv_b_proj", dtype=dt)
        self.o_proj = RowParallelLinear(cfg.num_attention_heads * self.vd, cfg.hidden_size, quant=q, prefix=prefix + ".o_proj", dtype=dt)
        self.rope = get_rope(self.rope_d, cfg.max_model_len, cfg.rope_theta, device, cfg.rope_scaling)
        self.scale = qk ** -0.5
        sc = cfg.rope_scaling or {}
        if (sc.get("rope_type") or sc.get("type")) in ("yarn", "deepseek_yarn") and sc.get("mscale_all_dim"):
            # DeepSeek yarn: the softmax scale carries mscale(factor, mscale_all_dim)^2 (reference: models/deepseek_v2.py:483-487)
            from onecat_vllm.ops.ref import yarn_mscale
            m = yarn_mscale(float(sc.get("factor", 1.0)), float(sc["mscale_all_dim"]))
            self.scale *= m * m
        self._wuk = self._wuv = None

    def process_weights_after_loading(self):
        """Runs before the child layers' own repacking (parents come first in ``modules()``): the absorbed ``W_UK`` / ``W_UV`` are
        taken from ``kv_b_proj`` while its checkpoint tensors still exist — a quantised ``kv_b_proj`` is packed for the GEMM
        afterwards and can no longer be dequantised on the host side."""
        self._wuk = self._wuv = None
        self._absorb(self.kv_b_proj.compute_dtype)

    def _absorb(self, dtype):
        if self._wuk is None:
            w = self.kv_b_proj.method.dequantized_weight(self.kv_b_proj).to(dtype).view(self.H, self.nope + self.vd, self.lora)
            self._wuk = w[:, : self.nope, :].contiguous()  # [H, nope, lora]
            self._wuv = w[:, self.nope:, :].contiguous()  # [H, v, lora]
        return self._wuk, self._wuv

    def forward(self, x, md, latent_cache):
        T = x.shape[0]
        if self.q_lora:
            qa, _ = self.q_a_layernorm(self.q_a_proj(x))
            q = self.q_b_proj(qa)
        else:
            q = self.q_proj(x)
        q = q.view(T, self.H, self.nope + self.rope_d)
        kv = self.kv_a_proj_with_mqa(x)
        c, _ = self.kv_a_layernorm(kv[:, : self.lora].contiguous())
        cs = self.rope.cos_sin[md.positions.long()]
        cos, sin = cs[:, : self.rope_d // 2], cs[:, self.rope_d // 2:]
        k_pe = _rope_interleaved(kv[:, self.lora:].unsqueeze(1), cos, sin).squeeze(1)
        q_pe = _rope_interleaved(q[..., self.nope:], cos, sin)
        # insert without a data-dependent shape (no host synchronisation, so the step can be captured in a CUDA graph): tokens
        # without a slot (-1, padding of a captured batch) are routed to slot 0 of block 0, the placeholder block nothing reads
        sm = md.slot_mapping.long().clamp(min=0)
        latent_cache.view(-1, latent_cache.shape[-1]).index_copy_(0, sm, torch.cat([c, k_pe], dim=-1).to(latent_cache.dtype))
        wuk, wuv = self._absorb(x.dtype)
        q_abs = torch.einsum("thn,hnl->thl", q[..., : self.nope], wuk)
        if x.is_cuda:
            from onecat_vllm.ops import cuda as K
            o_lat = K.mla_decode(q_abs, q_pe, latent_cache, md, self.scale, self.lora)
        else:
            o_lat = ref.mla_decode(q_abs, q_pe, latent_cache, md.block_table, md.query_start_loc, md.seq_lens, self.scale, self.lora)
        o = torch.einsum("thl,hvl->thv", o_lat, wuv)
        return self.o_proj(o.reshape(T, self.H * self.vd))
