"""Sparse MoE block: router → top-k → expert SwiGLU FFNs → weighted sum (+ shared expert)
(reference: models/qwen3_next.py:319-466 Qwen block; models/deepseek_v2.py:245-388 DeepSeek block;
layers/fused_moe/layer.py:70 ``FusedMoE``; routers layers/fused_moe/router/*.py).

Expert placement: with expert parallelism each rank owns ``E / ep`` whole experts; otherwise every rank holds
a 1/tp slice of every expert's intermediate dimension. Both produce *partial* outputs that the caller reduces
together with the residual add and norm."""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from onecat_vllm.config import ModelConfig
from onecat_vllm.layers.linear import ReplicatedLinear
from onecat_vllm.layers.mlp import MLP
from onecat_vllm.ops import ref
from onecat_vllm.parallel.state import get_state


class FusedMoE(nn.Module):
    """Holds stacked expert weights ``w13 [E_local, 2I_local, H]`` and ``w2 [E_local, H, I_local]``
    (bf16, or quantised storage + scales that dequantise to that)."""

    def __init__(self, cfg: ModelConfig, prefix: str):
        super().__init__()
        st = get_state()
        self.E, self.k = cfg.num_experts, cfg.num_experts_per_tok
        self.ep = st.ep_size > 1
        if self.ep:
            assert self.E % st.ep_size == 0
            self.E_local, self.e_off, self.I = self.E // st.ep_size, st.ep_rank * (self.E // st.ep_size), cfg.moe_intermediate_size
        else:
            self.E_local, self.e_off, self.I = self.E, 0, cfg.moe_intermediate_size // st.tp_size
        self.I_global, self.H = cfg.moe_intermediate_size, cfg.hidden_size
        self.tp, self.tp_rank = st.tp_size, st.tp_rank
        q = cfg.quant
        self.qmethod = (q.expert_method or q.method) if q and q.method != "none" else "none"
        self.block = q.weight_block_size if q else None
        dt = cfg.dtype
        E, I, H = self.E_local, self.I, self.H
        if self.qmethod == "fp8":
            bn, bk = self.block or (128, 128)
            self.w13 = nn.Parameter(torch.zeros(E, 2 * I, H, dtype=torch.float8_e4m3fn), requires_grad=False)
            self.w2 = nn.Parameter(torch.zeros(E, H, I, dtype=torch.float8_e4m3fn), requires_grad=False)
            self.w13_scale = nn.Parameter(torch.ones(E, -(-2 * I // bn), -(-H // bk), dtype=torch.float32), requires_grad=False)
            self.w2_scale = nn.Parameter(torch.ones(E, -(-H // bn), -(-I // bk), dtype=torch.float32), requires_grad=False)
        elif self.qmethod == "mxfp4":
            self.w13 = nn.Parameter(torch.zeros(E, 2 * I, H // 2, dtype=torch.uint8), requires_grad=False)
            self.w2 = nn.Parameter(torch.zeros(E, H, I // 2, dtype=torch.uint8), requires_grad=False)
            self.w13_scale = nn.Parameter(torch.full((E, 2 * I, H // 32), 127, dtype=torch.uint8), requires_grad=False)
            self.w2_scale = nn.Parameter(torch.full((E, H, I // 32), 127, dtype=torch.uint8), requires_grad=False)
        else:
            self.qmethod = "none"
            self.w13 = nn.Parameter(torch.zeros(E, 2 * I, H, dtype=dt), requires_grad=False)
            self.w2 = nn.Parameter(torch.zeros(E, H, I, dtype=dt), requires_grad=False)
        self.act = cfg.moe_act
        if cfg.expert_bias:
            self.w13_bias = nn.Parameter(torch.zeros(E, 2 * I, dtype=dt), requires_grad=False)
            self.w2_bias = nn.Parameter(torch.zeros(E, H, dtype=dt), requires_grad=False)
        else:
            self.w13_bias = self.w2_bias = None
        self._dq = None
        self.kernel_state = None

    # ---- loading: expert_id is global; proj in {"gate_proj","up_proj","down_proj"}
    def load_expert_weight(self, expert_id: int, proj: str, pname: str, w: torch.Tensor) -> None:
        e = expert_id - self.e_off
        if not 0 <= e < self.E_local:
            return
        I, r = self.I, (0 if self.ep else self.tp_rank)
        if pname == "bias":
            if proj in ("gate_proj", "up_proj"):
                src = w.narrow(0, r * I, I) if not self.ep and self.tp > 1 else w
                self.w13_bias.data[e, (0 if proj == "gate_proj" else I):(I if proj == "gate_proj" else 2 * I)].copy_(src)
            elif self.ep or self.tp_rank == 0:
                self.w2_bias.data[e].copy_(w)   # the down bias joins the partial sums once
            return
        scale = pname != "weight"
        tgt13, tgt2 = (self.w13_scale, self.w2_scale) if scale else (self.w13, self.w2)
        if proj in ("gate_proj", "up_proj"):
            rows = tgt13.shape[1] // 2
            src = w.narrow(0, r * rows, rows) if not self.ep and self.tp > 1 else w
            tgt13.data[e, (0 if proj == "gate_proj" else rows):(rows if proj == "gate_proj" else 2 * rows)].copy_(src)
        else:
            cols = tgt2.shape[2]
            src = w.narrow(1, r * cols, cols) if not self.ep and self.tp > 1 else w
            tgt2.data[e].copy_(src)

    def dequantized(self):
        if self._dq is None:
            if self.qmethod == "fp8":
                blk = self.block or (128, 128)
                self._dq = (ref.fp8_block_dequantize(self.w13, self.w13_scale, blk), ref.fp8_block_dequantize(self.w2, self.w2_scale, blk))
            elif self.qmethod == "mxfp4":
                self._dq = (ref.mxfp4_dequantize(self.w13, self.w13_scale), ref.mxfp4_dequantize(self.w2, self.w2_scale))
            else:
                self._dq = (self.w13, self.w2)
        return self._dq

    def process_weights_after_loading(self):
        self._dq = None
        if self.w13.is_cuda and self.act == "silu" and self.w13_bias is None:
            from onecat_vllm.ops import cuda as K
            K.prepare_moe(self)

    def forward(self, x, topk_w, topk_ids):
        if self.act != "silu" or self.w13_bias is not None:
            # experts with biases or the GPT-OSS activation: one pair of dense GEMMs per active expert (the grouped kernel's
            # epilogue implements SiLU·mul without bias only)
            if getattr(self, "_dq_model", None) is None or self._dq_model[0].dtype != x.dtype:
                self._dq_model = tuple(t.to(x.dtype) for t in self.dequantized())   # packed experts are widened once for this path
            w13, w2 = self._dq_model
            mm = None
            if x.is_cuda:
                from onecat_vllm.ops import cuda as K
                K.TORCH_STANDINS.add("moe_expert_loop")
                mm = K.gemm_bf16 if x.dtype == torch.bfloat16 else None
            return ref.fused_experts(x, w13, w2, topk_w, topk_ids, self.e_off, self.w13_bias, self.w2_bias, self.act, mm)
        if x.is_cuda:
            from onecat_vllm.ops import cuda as K
            return K.fused_moe(self, x, topk_w, topk_ids)
        w13, w2 = self.dequantized()
        return ref.fused_experts(x, w13, w2, topk_w, topk_ids, self.e_off)


class SparseMoeBlock(nn.Module):
    def __init__(self, cfg: ModelConfig, prefix: str):
        super().__init__()
        self.cfg = cfg
        self.gate = ReplicatedLinear(cfg.hidden_size, cfg.num_experts, bias=cfg.router_linear_bias, quant=None, prefix=prefix + ".gate",
                                     dtype=cfg.dtype)
        self.experts = FusedMoE(cfg, prefix + ".experts")
        self.deepseek = cfg.scoring_func == "sigmoid" or cfg.n_group > 1 or cfg.router_bias
        if self.deepseek:
            self.e_score_correction_bias = nn.Parameter(torch.zeros(cfg.num_experts, dtype=torch.float32), requires_grad=False)
        self.shared_expert: Optional[MLP] = None
        if cfg.shared_expert_intermediate_size > 0:
            self.shared_expert = MLP(cfg.hidden_size, cfg.shared_expert_intermediate_size, cfg.quant if cfg.quant.expert_method is None else
                                     cfg.quant, prefix + ".shared_expert", cfg.dtype)
            if cfg.shared_expert_gate:
                self.shared_expert_gate = ReplicatedLinear(cfg.hidden_size, 1, quant=None, prefix=prefix + ".shared_expert_gate", dtype=cfg.dtype)

    def route(self, x):
        c = self.cfg
        logits = self.gate(x)
        if x.is_cuda:
            from onecat_vllm.ops import cuda as K
            return K.route(logits, c, getattr(self, "e_score_correction_bias", None))
        if self.deepseek:
            return ref.grouped_topk(logits, c.num_experts_per_tok, c.n_group, c.topk_group, self.e_score_correction_bias,
                                    c.scoring_func, c.norm_topk_prob, c.routed_scaling_factor)
        return ref.topk_softmax(logits, c.num_experts_per_tok, c.norm_topk_prob)

    def _forward_a2a(self, x, mgr):
        """Token-exchange expert parallelism on a replicated batch: this rank routes its slice of the rows, the manager returns
        every rank's finished rows; rank 0 alone adds them to its partial sum so that the reduction that follows counts them once."""
        from onecat_vllm.parallel.all2all import token_slice
        st = get_state()
        T = x.shape[0]
        lo, hi = token_slice(T, st.ep_size, st.ep_rank)
        xl = x[lo:hi]
        if hi > lo:
            w, ids = self.route(xl)
        else:
            k = self.cfg.num_experts_per_tok
            w, ids = x.new_zeros(0, k, dtype=torch.float32), torch.zeros(0, k, dtype=torch.int32, device=x.device)
        y = mgr.moe(self.experts, xl, w.to(torch.float32), ids, t_off=lo, T_total=T, gather=True)
        return y.clone() if st.ep_rank == 0 else torch.zeros_like(x)

    def forward(self, x):
        from onecat_vllm import envs
        mgr = get_state().ep_a2a
        if mgr is not None and self.experts.ep and x.shape[0] >= envs.ONECAT_EP_A2A_MIN_TOKENS and \
                (not x.is_cuda or self.experts.kernel_state is not None):
            out = self._forward_a2a(x, mgr)
        else:
            w, ids = self.route(x)
            out = self.experts(x, w.to(torch.float32), ids)
        if self.shared_expert is not None:
            s = self.shared_expert(x)
            if self.cfg.shared_expert_gate:
                s = s * torch.sigmoid(self.shared_expert_gate(x).float()).to(s.dtype)
            out = out + s
        return out
