"""Self-attention block: fused QKV GEMM → (per-head norm) → RoPE + paged-KV insert → paged flash attention
→ (sigmoid output gate) → o_proj (reference: models/llama.py attention; models/qwen3_next.py:505-626 for the
gated variant with per-head q/k RMSNorm and partial rotary)."""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from onecat_vllm import ops
from onecat_vllm.config import ModelConfig
from onecat_vllm.layers.common import get_rope
from onecat_vllm.layers.linear import QKVParallelLinear, RowParallelLinear
from onecat_vllm.parallel.state import get_state


class Attention(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, prefix: str, device, qkv_in: Optional[int] = None):
        super().__init__()
        tp = get_state().tp_size
        self.D = cfg.head_dim
        self.gated = cfg.attn_output_gate
        # qkv_in: width of the projection's input when it is not the hidden size (EAGLE-3 feeds [embedding ; hidden])
        self.qkv_proj = QKVParallelLinear(qkv_in or cfg.hidden_size, cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads,
                                          q_mult=2 if self.gated else 1, bias=cfg.attention_bias, quant=cfg.quant,
                                          prefix=prefix + ".qkv_proj", dtype=cfg.dtype)
        self.Hq, self.Hkv = self.qkv_proj.num_heads, self.qkv_proj.num_kv_heads
        self.o_proj = RowParallelLinear(cfg.num_attention_heads * cfg.head_dim, cfg.hidden_size, bias=cfg.attn_o_bias, quant=cfg.quant,
                                        prefix=prefix + ".o_proj", dtype=cfg.dtype)
        self.sinks = nn.Parameter(torch.zeros(self.Hq, dtype=torch.float32), requires_grad=False) if cfg.attn_sinks else None
        self._tp_rank = get_state().tp_rank
        self.qk_norm, self.gemma, self.eps = cfg.qk_norm, cfg.gemma_norm, cfg.rms_norm_eps
        if cfg.qk_norm:
            init = torch.zeros if cfg.gemma_norm else torch.ones
            self.q_norm = nn.Parameter(init(cfg.head_dim, dtype=cfg.dtype), requires_grad=False)
            self.k_norm = nn.Parameter(init(cfg.head_dim, dtype=cfg.dtype), requires_grad=False)
        self.rotary_dim = 0 if layer_idx in cfg.nope_layers else cfg.rotary_dim
        self.qk_norm_full = cfg.qk_norm_full
        self.norm_after_rope = cfg.qk_norm and cfg.qk_norm_after_rope
        self.mrope_section = getattr(cfg, "mrope_section", None)  # (temporal, height, width) frequency counts; positions are then [3, T]
        if cfg.qk_norm_full:
            if tp > 1:
                raise ValueError("q / k normalisation over the whole projection is served with tensor_parallel_size=1 only")
            self.q_norm = nn.Parameter(torch.ones(cfg.num_attention_heads * cfg.head_dim, dtype=cfg.dtype), requires_grad=False)
            self.k_norm = nn.Parameter(torch.ones(cfg.num_key_value_heads * cfg.head_dim, dtype=cfg.dtype), requires_grad=False)
        # sliding-window layers may rotate with their own base and without the context-extension rule (Gemma3)
        self.window, self.softcap = cfg.layer_window(layer_idx), cfg.attn_softcap
        local = bool(self.window) and cfg.rope_local_theta is not None
        self.rope = get_rope(self.rotary_dim, cfg.max_model_len, cfg.rope_local_theta if local else cfg.rope_theta, device,
                             None if local else cfg.rope_scaling)
        self.scale = cfg.attn_scale if cfg.attn_scale is not None else cfg.head_dim ** -0.5
        self.layer_idx = layer_idx
        self.qkv_clip = cfg.qkv_clip

    def load_weight(self, pname: str, w: torch.Tensor, shard_id=None) -> None:
        """Parameters that belong to the block itself: the per-head sink logits are sharded with the query heads."""
        p = getattr(self, pname)
        if pname == "sinks":
            w = w.narrow(0, self._tp_rank * self.Hq, self.Hq)
        p.data.copy_(w.reshape(p.shape))

    def forward(self, x: torch.Tensor, md, kv_cache: torch.Tensor) -> torch.Tensor:
        T = x.shape[0]
        D, Hq, Hkv = self.D, self.Hq, self.Hkv
        qkv = self.qkv_proj(x)
        if self.qkv_clip is not None:      # OLMo: projections clamped to ±clip before the rotary embedding
            qkv = qkv.clamp(-self.qkv_clip, self.qkv_clip)
        qw = Hq * D * (2 if self.gated else 1)
        if self.gated:
            qg = qkv[:, :qw].view(T, Hq, 2 * D)
            q, gate = qg[..., :D], qg[..., D:]
        else:
            q, gate = qkv[:, :qw].view(T, Hq, D), None
        k = qkv[:, qw:qw + Hkv * D].view(T, Hkv, D)
        v = qkv[:, qw + Hkv * D:].view(T, Hkv, D)
        if self.qk_norm_full:
            q = ops.rms_norm(q.reshape(T, Hq * D), self.q_norm, self.eps)[0].view(T, Hq, D)
            k = ops.rms_norm(k.reshape(T, Hkv * D), self.k_norm, self.eps)[0].view(T, Hkv, D)
        if self.norm_after_rope:
            # rotate first (no cache write), normalise per head, then insert the normalised keys with a zero-width rotation
            q, k = q.contiguous(), k.contiguous()
            ops.rope_and_cache(q, k, v, md.positions, self.rope.cos_sin, None, md.slot_mapping, self.rotary_dim, None, None, self.eps, False)
            q = ops.rms_norm(q.view(T * Hq, D), self.q_norm, self.eps, None, self.gemma)[0].view(T, Hq, D)
            k = ops.rms_norm(k.view(T * Hkv, D), self.k_norm, self.eps, None, self.gemma)[0].view(T, Hkv, D)
            ops.rope_and_cache(q, k, v, md.positions, self.rope.cos_sin[:, :0], kv_cache, md.slot_mapping, 0, None, None, self.eps, False)
        else:
            mrope = self.mrope_section if md.mrope_positions is not None else None
            ops.rope_and_cache(q, k, v, md.mrope_positions if mrope else md.positions, self.rope.cos_sin, kv_cache, md.slot_mapping, self.rotary_dim,
                               self.q_norm if self.qk_norm else None, self.k_norm if self.qk_norm else None, self.eps, self.gemma,
                               mrope_section=mrope)
        o = ops.paged_attention(q, kv_cache, md, self.scale, window=self.window, softcap=self.softcap, sinks=self.sinks)
        if gate is not None:
            o = o * torch.sigmoid(gate.float()).to(o.dtype)
        return self.o_proj(o.reshape(T, Hq * D))
