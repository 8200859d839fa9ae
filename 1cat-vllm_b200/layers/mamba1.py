"""Mamba-1 mixer (selective state-space model) as a state-slot layer of the hybrid decoder
(reference: model_executor/layers/mamba/mamba_mixer.py; models/mamba.py, models/falcon_mamba.py).

x → in_proj → [x | z];  x → depthwise causal conv (bias, SiLU) with a rolling state;  x_proj(x) → [dt_low | B | C];
dt = softplus(dt_proj(dt_low));  A = -exp(A_log) per (channel, state index);  h_t = exp(dt ⊗ A) h_{t-1} + (dt x) ⊗ B,
y = h C + D x;  y * SiLU(z) → out_proj. FalconMamba normalises dt_low, B and C (RMS without weights) first, Jamba with weights.

Runs as PyTorch operations on every device (``ops.ref.mamba1_scan``): no CUDA kernel, tensor_parallel_size 1, no speculative decoding."""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from onecat_vllm.config import ModelConfig
from onecat_vllm.layers.linear import ReplicatedLinear
from onecat_vllm.ops import ref
from onecat_vllm.parallel.state import get_state


class Mamba1Mixer(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, prefix: str):
        super().__init__()
        if get_state().tp_size > 1:
            raise ValueError("the Mamba-1 mixer is served with tensor_parallel_size=1")
        self.d_inner, self.N, self.kw, self.dt_rank = cfg.mamba_n_heads * cfg.mamba_d_head, cfg.mamba_d_state, cfg.mamba_d_conv, cfg.mamba_dt_rank
        self.in_proj = ReplicatedLinear(cfg.hidden_size, 2 * self.d_inner, bias=cfg.mamba_proj_bias, quant=None, prefix=prefix + ".in_proj", dtype=cfg.dtype)
        self.conv_weight = nn.Parameter(torch.zeros(self.d_inner, self.kw, dtype=cfg.dtype), requires_grad=False)
        self.conv_bias = nn.Parameter(torch.zeros(self.d_inner, dtype=cfg.dtype), requires_grad=False) if cfg.mamba_conv_bias else None
        self.x_proj = ReplicatedLinear(self.d_inner, self.dt_rank + 2 * self.N, bias=False, quant=None, prefix=prefix + ".x_proj", dtype=cfg.dtype)
        self.dt_proj = ReplicatedLinear(self.dt_rank, self.d_inner, bias=True, quant=None, prefix=prefix + ".dt_proj", dtype=cfg.dtype)
        self.A_log = nn.Parameter(torch.zeros(self.d_inner, self.N, dtype=torch.float32), requires_grad=False)
        self.D = nn.Parameter(torch.ones(self.d_inner, dtype=torch.float32), requires_grad=False)
        self.out_proj = ReplicatedLinear(self.d_inner, cfg.hidden_size, bias=cfg.mamba_proj_bias, quant=None, prefix=prefix + ".out_proj", dtype=cfg.dtype)
        self.inner_rms_eps = cfg.mamba_inner_rms_eps
        self.inner_norms = cfg.mamba_inner_norm_weights   # Jamba: RMSNorm with weights on dt_low, B and C
        if self.inner_norms:
            from onecat_vllm.layers.common import RMSNorm
            self.dt_layernorm = RMSNorm(self.dt_rank, cfg.rms_norm_eps, False, cfg.dtype)
            self.b_layernorm = RMSNorm(self.N, cfg.rms_norm_eps, False, cfg.dtype)
            self.c_layernorm = RMSNorm(self.N, cfg.rms_norm_eps, False, cfg.dtype)
        self.layer_idx = layer_idx

    def load_weight(self, pname: str, w: torch.Tensor, shard=None) -> None:
        p = getattr(self, pname)
        p.data.copy_(w.reshape(p.shape).to(p.dtype))

    def state_shapes(self):
        return (self.d_inner, self.kw - 1), (1, self.d_inner, self.N)

    def forward(self, x: torch.Tensor, md, state) -> torch.Tensor:
        if getattr(md, "gdn_record", None) is not None:
            raise ValueError("speculative decoding is not served for Mamba-1 layers (their states are not recorded per token)")
        conv_state, ssm_state = state
        xz = self.in_proj(x)
        xs, z = xz[:, : self.d_inner], xz[:, self.d_inner:]
        xs = ref.causal_conv1d(xs.contiguous(), self.conv_weight, self.conv_bias, conv_state, md.query_start_loc, md.state_slots, md.has_initial_state)
        p = self.x_proj(xs)
        dt_low, B, C = p[:, : self.dt_rank], p[:, self.dt_rank: self.dt_rank + self.N], p[:, self.dt_rank + self.N:]
        if self.inner_rms_eps is not None:
            rms = lambda t: (t.float() * torch.rsqrt(t.float().pow(2).mean(-1, keepdim=True) + self.inner_rms_eps)).to(t.dtype)
            dt_low, B, C = rms(dt_low), rms(B), rms(C)
        if self.inner_norms:
            dt_low, B, C = self.dt_layernorm(dt_low.contiguous(), None)[0], self.b_layernorm(B.contiguous(), None)[0], self.c_layernorm(C.contiguous(), None)[0]
        dt = F.softplus(self.dt_proj(dt_low).float())
        y = ref.mamba1_scan(xs, dt, -torch.exp(self.A_log), B, C, self.D, ssm_state, md.query_start_loc, md.state_slots, md.has_initial_state)
        return self.out_proj((y * F.silu(z.float())).to(x.dtype))
