"""SwiGLU feed-forward: merged gate|up column-parallel GEMM with the SiLU·mul applied in its epilogue,
then the row-parallel down projection (reference: models/llama.py ``LlamaMLP``; layers/activation.py ``SiluAndMul``)."""
from __future__ import annotations

import torch.nn as nn

from onecat_vllm.layers.linear import MergedColumnParallelLinear, RowParallelLinear


class MLP(nn.Module):
    def __init__(self, hidden: int, inter: int, quant, prefix: str, dtype, parallel: bool = True):
        super().__init__()
        self.gate_up_proj = MergedColumnParallelLinear(hidden, [inter, inter], quant=quant, prefix=prefix + ".gate_up_proj",
                                                       dtype=dtype, fuse_silu_mul=True)
        self.down_proj = RowParallelLinear(inter, hidden, quant=quant, prefix=prefix + ".down_proj", dtype=dtype)

    def forward(self, x):
        return self.down_proj(self.gate_up_proj(x))
