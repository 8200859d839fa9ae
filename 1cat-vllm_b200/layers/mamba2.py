"""Mamba-2 mixer (state-space duality) as a state-slot layer of the hybrid decoder
(reference: model_executor/layers/mamba/mamba_mixer2.py; layers/mamba/ops/ssd_combined.py, causal_conv1d.py, mamba_ssm.py).

x → in_proj → [z | xBC | dt];  xBC → depthwise causal conv (bias, SiLU) with a rolling state → x ``[H, P]``, B / C ``[G, N]``;
dt = softplus(dt + dt_bias) clamped to the time-step limits, A = -exp(A_log);  h_t = exp(dt A) h_{t-1} + dt x ⊗ B,
y = h C + D x;  y → RMSNorm(y * SiLU(z)) over groups of the inner width → out_proj.

The convolution and the scan run as PyTorch operations on every device (the chunked form of ``ops.ref.mamba2_scan``); there is no
CUDA kernel for this mixer, and it is served with tensor_parallel_size = 1 and without speculative decoding."""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from onecat_vllm.config import ModelConfig
from onecat_vllm.layers.linear import ReplicatedLinear
from onecat_vllm.ops import ref
from onecat_vllm.parallel.state import get_state


class Mamba2Mixer(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, prefix: str):
        super().__init__()
        if get_state().tp_size > 1:
            raise ValueError("the Mamba-2 mixer is served with tensor_parallel_size=1")
        self.H, self.P = cfg.mamba_n_heads, cfg.mamba_d_head
        self.G, self.N = cfg.mamba_n_groups, cfg.mamba_d_state
        self.d_inner = self.H * self.P
        self.kw = cfg.mamba_d_conv
        self.conv_dim = self.d_inner + 2 * self.G * self.N
        self.in_proj = ReplicatedLinear(cfg.hidden_size, self.d_inner + self.conv_dim + self.H, bias=cfg.mamba_proj_bias, quant=None,
                                        prefix=prefix + ".in_proj", dtype=cfg.dtype)
        self.conv_weight = nn.Parameter(torch.zeros(self.conv_dim, self.kw, dtype=cfg.dtype), requires_grad=False)
        self.conv_bias = nn.Parameter(torch.zeros(self.conv_dim, dtype=cfg.dtype), requires_grad=False) if cfg.mamba_conv_bias else None
        self.dt_bias = nn.Parameter(torch.ones(self.H, dtype=torch.float32), requires_grad=False)
        self.A_log = nn.Parameter(torch.zeros(self.H, dtype=torch.float32), requires_grad=False)
        self.D = nn.Parameter(torch.ones(self.H, dtype=torch.float32), requires_grad=False)
        self.norm_weight = nn.Parameter(torch.ones(self.d_inner, dtype=cfg.dtype), requires_grad=False)
        self.out_proj = ReplicatedLinear(self.d_inner, cfg.hidden_size, bias=cfg.mamba_proj_bias, quant=None, prefix=prefix + ".out_proj",
                                         dtype=cfg.dtype)
        self.eps = cfg.rms_norm_eps
        self.dt_limit = tuple(cfg.mamba_time_step_limit)
        self.norm_groups = cfg.mamba_norm_groups
        self.layer_idx = layer_idx

    def load_weight(self, pname: str, w: torch.Tensor, shard=None) -> None:
        p = getattr(self, pname)
        p.data.copy_(w.reshape(p.shape).to(p.dtype))

    def state_shapes(self):
        return (self.conv_dim, self.kw - 1), (self.H, self.P, self.N)

    def forward(self, x: torch.Tensor, md, state) -> torch.Tensor:
        """``state`` = (conv_state [slots, conv_dim, kw-1], ssm_state fp32 [slots, H, P, N])."""
        if getattr(md, "gdn_record", None) is not None:
            raise ValueError("speculative decoding is not served for Mamba-2 layers (their states are not recorded per token)")
        conv_state, ssm_state = state
        T = x.shape[0]
        zxbcdt = self.in_proj(x)
        z, xbc, dt = zxbcdt[:, : self.d_inner], zxbcdt[:, self.d_inner: self.d_inner + self.conv_dim], zxbcdt[:, self.d_inner + self.conv_dim:]
        xbc = ref.causal_conv1d(xbc.contiguous(), self.conv_weight, self.conv_bias, conv_state, md.query_start_loc, md.state_slots,
                                md.has_initial_state)
        xs = xbc[:, : self.d_inner].reshape(T, self.H, self.P)
        B = xbc[:, self.d_inner: self.d_inner + self.G * self.N].reshape(T, self.G, self.N)
        C = xbc[:, self.d_inner + self.G * self.N:].reshape(T, self.G, self.N)
        dt = F.softplus(dt.float() + self.dt_bias)
        if self.dt_limit[0] > 0.0 or self.dt_limit[1] != float("inf"):
            dt = dt.clamp(self.dt_limit[0], self.dt_limit[1])
        y = ref.mamba2_scan(xs, dt, -torch.exp(self.A_log), B, C, self.D, ssm_state, md.query_start_loc, md.state_slots, md.has_initial_state)
        y = y.reshape(T, self.d_inner) * F.silu(z.float())
        g = self.norm_groups
        yg = y.view(T, g, self.d_inner // g)
        y = (yg * torch.rsqrt(yg.pow(2).mean(-1, keepdim=True) + self.eps)).view(T, self.d_inner)
        y = (y.to(x.dtype) * self.norm_weight)
        return self.out_proj(y)
