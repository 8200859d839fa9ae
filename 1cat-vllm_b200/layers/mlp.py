"""SwiGLU feed-forward: merged gate|up column-parallel GEMM with the SiLU·mul applied in its epilogue,
then the row-parallel down projection (reference: models/llama.py ``LlamaMLP``; layers/activation.py ``SiluAndMul``)."""
from __future__ import annotations

import torch.nn as nn

from onecat_vllm.layers.linear import ColumnParallelLinear, MergedColumnParallelLinear, RowParallelLinear


class MLP(nn.Module):
    def __init__(self, hidden: int, inter: int, quant, prefix: str, dtype, parallel: bool = True, fuse_act: bool = True, act: str = "silu",
                 bias: bool = False):
        """``fuse_act=False`` (LoRA-enabled models) keeps gate|up as a plain GEMM so adapter deltas can be added before SiLU·mul.
        ``act="gelu_tanh"`` (Gemma GeGLU) always takes the unfused form: the GEMM epilogue implements SiLU·mul only."""
        super().__init__()
        fuse_act = fuse_act and act == "silu" and not bias   # the fused epilogue has no bias input
        self.fuse_act, self.act = fuse_act, act
        self.gate_up_proj = MergedColumnParallelLinear(hidden, [inter, inter], bias=bias, quant=quant, prefix=prefix + ".gate_up_proj",
                                                       dtype=dtype, fuse_silu_mul=fuse_act)
        self.down_proj = RowParallelLinear(inter, hidden, bias=bias, quant=quant, prefix=prefix + ".down_proj", dtype=dtype)

    def forward(self, x):
        h = self.gate_up_proj(x)
        if not self.fuse_act:
            from onecat_vllm import ops
            h = ops.silu_and_mul(h) if self.act == "silu" else ops.gelu_tanh_and_mul(h)
        return self.down_proj(h)


class PlainMLP(nn.Module):
    """Feed-forward without a gate: ``down(act(up(x)))`` with ``act`` = squared ReLU (Arcee) or GELU
    (reference: models/arcee.py ``ArceeMLP``; layers/activation.py ``ReLUSquaredActivation``). The activation is an elementwise
    PyTorch operation between the two GEMMs."""

    def __init__(self, hidden: int, inter: int, quant, prefix: str, dtype, act: str = "relu2", bias: bool = False):
        super().__init__()
        self.act = act
        self.up_proj = ColumnParallelLinear(hidden, inter, bias=bias, quant=quant, prefix=prefix + ".up_proj", dtype=dtype)
        self.down_proj = RowParallelLinear(inter, hidden, bias=bias, quant=quant, prefix=prefix + ".down_proj", dtype=dtype)

    def forward(self, x):
        import torch
        import torch.nn.functional as F
        h = self.up_proj(x)
        if self.act == "relu2":
            h = torch.square(F.relu(h))
        elif self.act == "gelu_tanh":
            h = F.gelu(h, approximate="tanh")
        elif self.act == "gelu":
            h = F.gelu(h)
        else:
            h = F.silu(h)
        return self.down_proj(h)


class FeedForwardBlock(PlainMLP):
    """An ungated feed-forward that is a block of its own (NemotronH: every block is ``h + mixer(norm(h))`` and the mixer is a
    Mamba-2 layer, an attention layer or this; reference: models/nemotron_h.py ``NemotronHMLPDecoderLayer``). It takes the place of a
    state-slot mixer in the decoder and declares a one-element state, so the runner and the scheduler need no third kind of layer."""

    def __init__(self, cfg, layer_idx: int, prefix: str):
        super().__init__(cfg.hidden_size, cfg.intermediate_size, cfg.quant, prefix, cfg.dtype, act=cfg.hidden_act, bias=cfg.mlp_bias)

    def state_shapes(self):
        return (1, 1), (1, 1, 1)

    def forward(self, x, md=None, state=None):
        return super().forward(x)
