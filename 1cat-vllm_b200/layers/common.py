"""Norm, rotary and embedding layers (reference: layers/layernorm.py:157,252; layers/rotary_embedding/;
layers/vocab_parallel_embedding.py:400,686; layers/logits_processor.py:179-247)."""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from onecat_vllm import ops
from onecat_vllm.ops import ref
from onecat_vllm.parallel import state as ps


class RMSNorm(nn.Module):
    def __init__(self, hidden: int, eps: float, gemma: bool = False, dtype=torch.float32):
        super().__init__()
        self.weight = nn.Parameter(torch.zeros(hidden, dtype=dtype) if gemma else torch.ones(hidden, dtype=dtype), requires_grad=False)
        self.eps, self.gemma = eps, gemma

    def forward(self, x, residual: Optional[torch.Tensor] = None):
        """Returns (normed, residual_out); the add is fused."""
        return ops.rms_norm(x, self.weight, self.eps, residual, self.gemma)

    def load_weight(self, pname, w, shard_id=None):
        self.weight.data.copy_(w)


class LayerNorm(nn.Module):
    """Mean-and-variance normalisation with the interface of ``RMSNorm`` (returns ``(normed, residual_out)``), for the families that
    predate RMSNorm or keep it: OLMo (no learned parameters), StableLM / Starcoder2 / Jais-2 (weight and bias), Nemotron (weight
    stored minus one, reference: models/nemotron.py ``NemotronLayerNorm1P``). It runs as PyTorch operations on every device and is
    not folded into the tensor-parallel reduction kernel (``plain`` tells ``reduce_add_norm`` to reduce first and call it after)."""

    plain = True

    def __init__(self, hidden: int, eps: float, affine: bool = True, bias: bool = True, plus_one: bool = False, dtype=torch.float32):
        super().__init__()
        self.hidden, self.eps, self.gemma = hidden, eps, plus_one
        self.weight = nn.Parameter(torch.zeros(hidden, dtype=dtype) if plus_one else torch.ones(hidden, dtype=dtype), requires_grad=False) \
            if affine else None
        self.bias = nn.Parameter(torch.zeros(hidden, dtype=dtype), requires_grad=False) if affine and bias else None

    def forward(self, x, residual: Optional[torch.Tensor] = None):
        if residual is not None:
            x = x + residual
        w = self.weight
        if w is not None:
            w = w.float() + 1.0 if self.gemma else w.float()
        y = torch.nn.functional.layer_norm(x.float(), (self.hidden,), w, None if self.bias is None else self.bias.float(), self.eps)
        return y.to(x.dtype), x

    def load_weight(self, pname, w, shard_id=None):
        getattr(self, pname).data.copy_(w)


def make_norm(cfg, hidden: Optional[int] = None) -> nn.Module:
    """The normalisation a model's blocks use: RMSNorm unless its configuration names the mean-and-variance form."""
    hidden = hidden or cfg.hidden_size
    if cfg.norm_type == "layernorm":
        return LayerNorm(hidden, cfg.rms_norm_eps, cfg.norm_affine, cfg.norm_bias, cfg.gemma_norm, cfg.dtype)
    return RMSNorm(hidden, cfg.rms_norm_eps, cfg.gemma_norm, cfg.dtype)


class RotaryEmbedding:
    """NeoX-style rotary with a precomputed fp32 cos|sin table."""

    def __init__(self, rotary_dim: int, max_pos: int, theta: float, device, scaling: Optional[dict] = None):
        self.rotary_dim = rotary_dim
        self.cos_sin = ref.build_cos_sin_cache(rotary_dim, max_pos, theta, device, scaling)


_ROPE_CACHE: dict = {}


def get_rope(rotary_dim: int, max_pos: int, theta: float, device, scaling: Optional[dict] = None) -> RotaryEmbedding:
    key = (rotary_dim, max_pos, theta, str(device), repr(sorted(scaling.items())) if scaling else None)
    if key not in _ROPE_CACHE:
        _ROPE_CACHE[key] = RotaryEmbedding(rotary_dim, max_pos, theta, device, scaling)
    return _ROPE_CACHE[key]


def pad_vocab(v: int, tp: int, mult: int = 64) -> int:
    per = -(-v // tp)
    return -(-per // mult) * mult * tp


class VocabParallelEmbedding(nn.Module):
    """Rows are split over TP ranks (padded to 64 per shard); out-of-shard ids contribute zeros and the
    partial results are summed across ranks."""

    def __init__(self, vocab: int, hidden: int, dtype=torch.float32):
        super().__init__()
        st = ps.get_state()
        self.tp, self.rank = st.tp_size, st.tp_rank
        self.vocab, self.padded = vocab, pad_vocab(vocab, self.tp)
        self.per = self.padded // self.tp
        self.lo = self.rank * self.per
        self.weight = nn.Parameter(torch.zeros(self.per, hidden, dtype=dtype), requires_grad=False)

    def load_weight(self, pname, w, shard_id=None):
        hi = min(self.lo + self.per, w.shape[0])
        if hi > self.lo:
            self.weight.data[: hi - self.lo].copy_(w[self.lo:hi])

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        if self.tp == 1:
            return F.embedding(ids.long(), self.weight)
        local = ids.long() - self.lo
        ok = (local >= 0) & (local < self.per)
        out = F.embedding(local.clamp(0, self.per - 1), self.weight) * ok.unsqueeze(-1).to(self.weight.dtype)
        from onecat_vllm.parallel.tp_ops import reduce_only
        return reduce_only(out)


class ParallelLMHead(VocabParallelEmbedding):
    """Vocab-sharded output projection; ``compute_logits`` gathers the shards."""

    def compute_logits(self, hidden: torch.Tensor) -> torch.Tensor:
        if hidden.is_cuda:
            from onecat_vllm.ops import cuda as K
            local = K.gemm_bf16(hidden, self.weight)
        else:
            local = F.linear(hidden, self.weight)
        full = ps.all_gather_last_dim(local)
        return full[..., : self.vocab]

    def greedy_tokens(self, hidden: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
        """Arg-max over the whole vocabulary without gathering the logits: each rank takes the maximum of its own shard and the
        ranks exchange one (value, index) pair per row; ties go to the lowest token id, as ``argmax`` over the gathered logits would
        (reference: model_executor/layers/logits_processor.py:363,711 fused top-1 across tensor-parallel ranks)."""
        if hidden.is_cuda:
            from onecat_vllm.ops import cuda as K
            local = K.gemm_bf16(hidden, self.weight)
        else:
            local = F.linear(hidden, self.weight)
        valid = max(min(self.per, self.vocab - self.lo), 0)      # the last shard is padded with rows that are not tokens
        B = hidden.shape[0]
        if valid > 0:
            lf = local[:, :valid].float()
            if scale < 0:
                lf = lf * scale
            val, idx = lf.max(dim=-1)
            pair = torch.stack([val, (idx + self.lo).float()], dim=-1)   # token ids are below 2^24: exact in fp32
        else:
            pair = torch.stack([torch.full((B,), -float("inf"), device=hidden.device), torch.zeros(B, device=hidden.device)], dim=-1)
        if self.tp == 1:
            return pair[:, 1].long()
        import torch.distributed as dist
        pairs = [torch.empty_like(pair) for _ in range(self.tp)]
        dist.all_gather(pairs, pair.contiguous(), group=ps.get_state().tp_group)
        allp = torch.stack(pairs, 0)                                # [tp, B, 2]
        best = allp[..., 0].argmax(dim=0)                           # first rank holding the maximum = lowest token id among ties
        return allp[best, torch.arange(B, device=hidden.device), 1].long()
