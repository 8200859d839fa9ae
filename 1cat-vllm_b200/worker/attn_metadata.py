"""Per-step attention metadata shared by all layers
(reference: vllm/v1/attention/backend.py:549 ``AttentionMetadataBuilder``; fields of flash_attn.py ``FlashAttentionMetadata``)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch


@dataclass
class AttentionMetadata:
    num_reqs: int
    num_tokens: int
    query_start_loc: torch.Tensor  # int32 [R+1]
    seq_lens: torch.Tensor  # int32 [R]  context length including this step's tokens
    block_table: torch.Tensor  # int32 [R, max_blocks]
    slot_mapping: torch.Tensor  # int32 [T]
    positions: torch.Tensor  # int32 [T]
    max_query_len: int
    max_seq_len: int
    # hybrid models
    state_slots: Optional[torch.Tensor] = None  # int32 [R]
    has_initial_state: Optional[torch.Tensor] = None  # bool/int32 [R]
    # host copies (cheap control decisions without a device sync)
    query_lens_cpu: Optional[list] = None
    seq_lens_cpu: Optional[list] = None
    # split-KV decode plan (filled by the GPU runner)
    num_kv_splits: int = 1
    is_uniform_decode: bool = False
    uniform_query_len: int = 1
    mrope_positions: Optional[torch.Tensor] = None  # int32 [3, T] (temporal, height, width) for models with rotary sections
