"""Gated short convolution (LFM2's ``conv`` layers) as a state-slot layer of the hybrid decoder
(reference: model_executor/layers/mamba/short_conv.py; models/lfm2.py).

x → in_proj → [B | C | x];  y = C * causal_conv1d(B * x)  (depthwise, kernel ``conv_L_cache``, no activation) → out_proj. The only
state is the convolution's last ``k - 1`` inputs. Runs as PyTorch operations on every device; tensor_parallel_size 1, no
speculative decoding."""
from __future__ import annotations

import torch
import torch.nn as nn

from onecat_vllm.config import ModelConfig
from onecat_vllm.layers.linear import ReplicatedLinear
from onecat_vllm.ops import ref
from onecat_vllm.parallel.state import get_state


class ShortConv(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, prefix: str):
        super().__init__()
        if get_state().tp_size > 1:
            raise ValueError("short-convolution layers are served with tensor_parallel_size=1")
        H = cfg.hidden_size
        self.H, self.kw = H, cfg.mamba_d_conv
        self.in_proj = ReplicatedLinear(H, 3 * H, bias=cfg.mamba_conv_bias, quant=None, prefix=prefix + ".in_proj", dtype=cfg.dtype)
        self.conv_weight = nn.Parameter(torch.zeros(H, self.kw, dtype=cfg.dtype), requires_grad=False)
        self.conv_bias = nn.Parameter(torch.zeros(H, dtype=cfg.dtype), requires_grad=False) if cfg.mamba_conv_bias else None
        self.out_proj = ReplicatedLinear(H, H, bias=cfg.mamba_conv_bias, quant=None, prefix=prefix + ".out_proj", dtype=cfg.dtype)
        self.layer_idx = layer_idx

    def load_weight(self, pname: str, w: torch.Tensor, shard=None) -> None:
        p = getattr(self, pname)
        p.data.copy_(w.reshape(p.shape).to(p.dtype))

    def state_shapes(self):
        return (self.H, self.kw - 1), (1, 1, 1)

    def forward(self, x: torch.Tensor, md, state) -> torch.Tensor:
        if getattr(md, "gdn_record", None) is not None:
            raise ValueError("speculative decoding is not served for short-convolution layers (their state is not recorded per token)")
        conv_state, _ = state
        bcx = self.in_proj(x)
        B, C, xx = bcx[:, : self.H], bcx[:, self.H: 2 * self.H], bcx[:, 2 * self.H:]
        conv = ref.causal_conv1d((B * xx).contiguous(), self.conv_weight, self.conv_bias, conv_state, md.query_start_loc, md.state_slots,
                                 md.has_initial_state, activation=False)
        return self.out_proj(C * conv)
