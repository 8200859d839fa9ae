"""Gated-DeltaNet linear-attention block (reference: layers/mamba/gdn/qwen_gdn_linear_attn.py:2057-2180 layer,
:6945-7013 gating; recurrence flash_qla/.../gdn_forward.cu:131-215).

x → [q|k|v|z] and [b|a] projections → depthwise causal conv (k=4, SiLU) over [q|k|v] with a rolling state →
g = -exp(A_log)·softplus(a+dt_bias), β = sigmoid(b) → gated delta rule with fp32 state per (sequence, v-head)
→ RMSNormGated(o, z) per head → row-parallel out_proj. V heads (and their K-head groups) are split over TP ranks."""
from __future__ import annotations

import torch
import torch.nn as nn

from onecat_vllm import ops
from onecat_vllm.config import ModelConfig
from onecat_vllm.layers.linear import MergedColumnParallelLinear, RowParallelLinear
from onecat_vllm.ops import ref
from onecat_vllm.parallel.state import get_state


class GatedDeltaNet(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, prefix: str):
        super().__init__()
        tp = get_state().tp_size
        self.Hk, self.Hv = cfg.linear_num_key_heads // tp, cfg.linear_num_value_heads // tp
        self.K, self.V = cfg.linear_key_head_dim, cfg.linear_value_head_dim
        key_dim, val_dim = cfg.linear_num_key_heads * self.K, cfg.linear_num_value_heads * self.V
        self.key_dim, self.val_dim = key_dim // tp, val_dim // tp
        self.kw = cfg.linear_conv_kernel_dim
        self.in_proj_qkvz = MergedColumnParallelLinear(cfg.hidden_size, [key_dim, key_dim, val_dim, val_dim], quant=cfg.quant,
                                                       prefix=prefix + ".in_proj_qkvz", dtype=cfg.dtype)
        self.in_proj_ba = MergedColumnParallelLinear(cfg.hidden_size, [cfg.linear_num_value_heads, cfg.linear_num_value_heads],
                                                     quant=None, prefix=prefix + ".in_proj_ba", dtype=cfg.dtype)
        self.conv_dim = 2 * self.key_dim + self.val_dim
        self.conv_weight = nn.Parameter(torch.zeros(self.conv_dim, self.kw, dtype=cfg.dtype), requires_grad=False)
        self.A_log = nn.Parameter(torch.zeros(self.Hv, dtype=torch.float32), requires_grad=False)
        self.dt_bias = nn.Parameter(torch.ones(self.Hv, dtype=torch.float32), requires_grad=False)
        self.norm_weight = nn.Parameter(torch.ones(self.V, dtype=cfg.dtype), requires_grad=False)
        self.out_proj = RowParallelLinear(val_dim, cfg.hidden_size, quant=cfg.quant, prefix=prefix + ".out_proj", dtype=cfg.dtype)
        self.eps = cfg.rms_norm_eps
        self.layer_idx = layer_idx

    def deinterleave(self, which: str, w: torch.Tensor) -> torch.Tensor:
        """Checkpoints with a fused ``in_proj_qkvz`` / ``in_proj_ba`` (Qwen3-Next) store the rows per key-head group —
        ``[q_g | k_g | v_g | z_g]`` resp. ``[b_g | a_g]`` for group g — while this layer keeps ``[q | k | v | z]`` and ``[b | a]`` over all
        heads (reference: models/qwen3_next.py ``fix_query_key_value_ordering``). ``w`` is the full (unsharded) tensor."""
        cfg_hk = self.Hk * get_state().tp_size
        r = self.Hv // self.Hk
        if which == "in_proj_qkvz":
            parts = [self.K, self.K, r * self.V, r * self.V]
        else:
            parts = [r, r]
        g = w.reshape(cfg_hk, sum(parts), *w.shape[1:])
        outs, o = [], 0
        for n in parts:
            outs.append(g[:, o:o + n].reshape(cfg_hk * n, *w.shape[1:]))
            o += n
        return torch.cat(outs, 0)

    def load_weight(self, pname: str, w: torch.Tensor, shard=None) -> None:
        """Per-head and per-channel parameters, sharded like the heads: conv channels are ``[q | k | v]`` segments."""
        st = get_state()
        tp, r = st.tp_size, st.tp_rank
        p = getattr(self, pname)
        if pname == "conv_weight":
            w = w.reshape(w.shape[0], -1)
            kd, vd = self.key_dim * tp, self.val_dim * tp
            segs = [w[:kd], w[kd:2 * kd], w[2 * kd:2 * kd + vd]]
            w = torch.cat([s.chunk(tp, 0)[r] for s in segs], 0)
        elif pname in ("A_log", "dt_bias"):
            w = w.reshape(-1).chunk(tp, 0)[r]
        p.data.copy_(w.reshape(p.shape).to(p.dtype))

    def state_shapes(self):
        return (self.conv_dim, self.kw - 1), (self.Hv, self.K, self.V)

    def forward(self, x: torch.Tensor, md, state) -> torch.Tensor:
        """``state`` = (conv_state [slots, conv_dim, kw-1], ssm_state fp32 [slots, Hv, K, V])."""
        conv_state, ssm_state = state
        T = x.shape[0]
        qkvz = self.in_proj_qkvz(x)
        ba = self.in_proj_ba(x)
        mixed, z = qkvz[:, : self.conv_dim], qkvz[:, self.conv_dim:]
        b, a = ba[:, : self.Hv], ba[:, self.Hv:]
        if x.is_cuda:
            from onecat_vllm.ops import cuda as K
            o = K.gdn_forward(mixed, b, a, self.conv_weight, self.A_log, self.dt_bias, conv_state, ssm_state, md,
                              self.Hk, self.Hv, self.K, self.V)
        else:
            rec = getattr(md, "gdn_record", None)
            pre = mixed.contiguous()
            prev = conv_state[md.state_slots.long()].clone() if rec is not None else None
            mixed = ref.causal_conv1d(pre, self.conv_weight, None, conv_state, md.query_start_loc, md.state_slots, md.has_initial_state)
            q = mixed[:, : self.key_dim].reshape(T, self.Hk, self.K)
            k = mixed[:, self.key_dim: 2 * self.key_dim].reshape(T, self.Hk, self.K)
            v = mixed[:, 2 * self.key_dim:].reshape(T, self.Hv, self.V)
            g, beta = ref.gdn_gating(a, b, self.A_log, self.dt_bias)
            spec = None
            if rec is not None:
                spec = torch.zeros(md.num_reqs, md.spec_q, self.Hv, self.K, self.V, dtype=torch.float32)
                rec.append(dict(conv_state=conv_state, ssm_state=ssm_state, spec=spec, prev=prev, mixed=pre, kw=self.kw))
            o = ref.gated_delta_rule(q, k, v, g, beta, ssm_state, md.query_start_loc, md.state_slots, md.has_initial_state, token_states=spec)
        o = ops.rms_norm_gated(o.reshape(T, self.Hv * self.V), z, self.norm_weight, self.eps, self.Hv)
        return self.out_proj(o)
