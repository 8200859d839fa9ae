"""Tensor-parallel reductions as the model sees them.

The reference all-reduces after every row-parallel GEMM and then runs a separate add+RMSNorm kernel, or
fuses both through FlashInfer / custom kernels (reference: layers/linear.py:1800-1805;
compilation/passes/fusion/allreduce_rms_fusion.py:199; csrc/custom_all_reduce.cuh:436). Here the model always
calls ``reduce_add_norm``: with one rank it is the fused add+norm kernel, with several it is the
peer-memory kernel that sums the ranks' partials, adds the residual and normalises in one pass
(``tp_comm="fused"``) or NCCL all-reduce followed by the norm (``tp_comm="nccl"``, the baseline).
"""
from __future__ import annotations

from typing import Optional

import torch

from onecat_vllm.parallel import state as ps


def reduce_add_norm(partial: torch.Tensor, residual: Optional[torch.Tensor], norm) -> tuple[torch.Tensor, torch.Tensor]:
    st = ps.get_state()
    if st.tp_size == 1:
        return norm(partial, residual)
    if getattr(norm, "plain", False):      # a normalisation the fused kernel does not compute: reduce, then normalise
        return norm(reduce_only(partial), residual)
    if st.fused is not None and partial.is_cuda and st.tp_comm == "fused":
        return st.fused.reduce_add_norm(partial, residual, norm.weight, norm.eps, norm.gemma, pushed=getattr(partial, "_tp_pushed", False))
    ps.all_reduce(partial)
    return norm(partial, residual)


def reduce_only(partial: torch.Tensor) -> torch.Tensor:
    st = ps.get_state()
    if st.tp_size == 1:
        return partial
    if st.fused is not None and partial.is_cuda and st.tp_comm == "fused":
        return st.fused.all_reduce(partial)
    return ps.all_reduce(partial)


def row_parallel_out(num_tokens: int, hidden: int, dtype, device) -> Optional[torch.Tensor]:
    """Where a row-parallel GEMM should write its partial sums: a slice of the symmetric heap in fused mode."""
    st = ps.get_state()
    if st.tp_size > 1 and st.fused is not None and st.tp_comm == "fused" and device.type == "cuda":
        return st.fused.partial_buffer(num_tokens, hidden, dtype)
    return None
