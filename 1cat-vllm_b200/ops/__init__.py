"""Op entry points. CUDA tensors go to the hand-written sm_100a kernels in the in-tree extension
(``onecat_vllm.ops.cuda``); CPU tensors go to the PyTorch restatements in ``onecat_vllm.ops.ref``.
There is no silent fallback: a CUDA tensor without the extension raises."""
from __future__ import annotations

from typing import Optional

import torch

from onecat_vllm.ops import ref

_ext = None


def ext():
    global _ext
    if _ext is None:
        from onecat_vllm.ops import cuda as _c
        _ext = _c
    return _ext


def rms_norm(x, w, eps, residual=None, gemma=False):
    if x.is_cuda:
        return ext().rms_norm(x, w, eps, residual, gemma)
    return ref.rms_norm(x, w, eps, residual, gemma)


def silu_and_mul(x):
    if x.is_cuda:
        return ext().silu_and_mul(x)
    return ref.silu_and_mul(x)


def gelu_tanh_and_mul(x):
    """GeGLU activation; an elementwise PyTorch expression on either device (Gemma-family models only)."""
    return ref.gelu_tanh_and_mul(x)


def rope_and_cache(q, k, v, positions, cos_sin, kv_cache, slot_mapping, rotary_dim, q_norm_w=None, k_norm_w=None,
                   eps=1e-6, gemma=False, mrope_section=None):
    """``mrope_section`` (three frequency counts summing to ``rotary_dim / 2``) with ``positions`` of shape ``[3, T]``: frequency i
    rotates by the temporal, height or width position according to the section it falls in (Qwen2-VL family)."""
    if q.is_cuda:
        return ext().rope_and_cache(q, k, v, positions, cos_sin, kv_cache, slot_mapping, rotary_dim, q_norm_w, k_norm_w, eps, gemma, mrope_section)
    return ref.rope_and_cache(q, k, v, positions, cos_sin, kv_cache, slot_mapping, rotary_dim, q_norm_w, k_norm_w, eps, gemma, mrope_section)


def paged_attention(q, kv_cache, md, scale, out=None, window=0, softcap=0.0, sinks=None):
    """``md`` is the step's AttentionMetadata. ``window``: sliding window in tokens (0 = full causal); ``softcap``: tanh soft-capping
    of the scaled scores (0 = off); ``sinks``: fp32 ``[Hq]`` sink logits that join the softmax denominator."""
    if q.is_cuda:
        return ext().paged_attention(q, kv_cache, md, scale, out, window=window, softcap=softcap, sinks=sinks)
    from onecat_vllm import envs
    if envs.ONECAT_CPU_ATTENTION == "native" and kv_cache.dtype in (torch.float32, torch.bfloat16) and q.dtype in (torch.float32, torch.bfloat16):
        return cpu_paged_attention(q, kv_cache, md.block_table, md.query_start_loc, md.seq_lens, scale, out, window=window, softcap=softcap, sinks=sinks)
    return ref.paged_attention(q, kv_cache, md.block_table, md.query_start_loc, md.seq_lens, scale, out, window=window, softcap=softcap,
                               sinks=sinks)


def cpu_paged_attention(q, kv_cache, block_table, query_start_loc, seq_lens, scale, out=None, return_lse=False, window=0, softcap=0.0, sinks=None,
                        threads: int = 0):
    """The C++ paged attention of the CPU backend (``csrc/native/cpu_attention.cpp``): same contract as ``ref.paged_attention`` for fp32 /
    bf16 queries and caches."""
    from onecat_vllm.utils import _native
    T, Hq, D = q.shape
    if q.stride(2) != 1:
        q = q.contiguous()
    o = torch.empty(T, Hq, D, dtype=q.dtype) if out is None else out
    assert o.stride(2) == 1 and kv_cache.is_contiguous() and o.dtype == q.dtype
    lse = torch.full((T, Hq), -float("inf"), dtype=torch.float32) if return_lse else None
    bt = block_table if block_table.dtype == torch.int32 else block_table.to(torch.int32)
    qsl = query_start_loc.to(torch.int32).contiguous()
    sl = seq_lens.to(torch.int32).contiguous()
    sk = sinks.float().contiguous() if sinks is not None else None
    _native.cpu_paged_attention(q.data_ptr(), kv_cache.data_ptr(), o.data_ptr(), lse.data_ptr() if lse is not None else 0, bt.data_ptr(), qsl.data_ptr(),
                                sl.data_ptr(), sk.data_ptr() if sk is not None else 0, q.stride(0), q.stride(1), o.stride(0), o.stride(1), bt.stride(0),
                                sl.shape[0], Hq, kv_cache.shape[2], D, kv_cache.shape[3], float(scale), int(window), float(softcap),
                                int(q.dtype == torch.bfloat16), int(kv_cache.dtype == torch.bfloat16), int(threads))
    return (o, lse) if return_lse else o


def rms_norm_gated(x, z, w, eps, heads):
    """x, z ``[T, heads*D]`` (column slices allowed) → ``[T, heads*D]``: per-head RMSNorm(x) * w * silu(z)."""
    if x.is_cuda:
        return ext().rms_norm_gated(x, z, w, eps, heads)
    T, D = x.shape[0], x.shape[1] // heads
    return ref.rms_norm_gated(x.reshape(T * heads, D), z.reshape(T * heads, D), w, eps).reshape(T, heads * D)


def merge_attn_states(o1, lse1, o2, lse2):
    """LSE-weighted merge of two partial attention results over disjoint key sets."""
    if o1.is_cuda:
        return ext().merge_attn_states(o1, lse1, o2, lse2)
    return ref.merge_attn_states(o1, lse1, o2, lse2)


def argmax(logits):
    if logits.is_cuda:
        return ext().argmax(logits)
    return logits.argmax(-1)
