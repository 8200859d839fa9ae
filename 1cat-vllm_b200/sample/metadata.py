"""Batched sampling state (reference: vllm/v1/sample/metadata.py)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch


@dataclass
class SamplingMetadata:
    temperature: Optional[torch.Tensor]  # [B] fp32; None when all greedy
    all_greedy: bool
    all_random: bool
    top_p: Optional[torch.Tensor]
    top_k: Optional[torch.Tensor]
    min_p: Optional[torch.Tensor]
    generators: dict  # row -> torch.Generator
    max_num_logprobs: Optional[int]
    no_penalties: bool
    presence_penalties: Optional[torch.Tensor] = None
    frequency_penalties: Optional[torch.Tensor] = None
    repetition_penalties: Optional[torch.Tensor] = None
    prompt_token_ids: Optional[list] = None  # per row list[int] (for penalties)
    output_token_ids: list = field(default_factory=list)  # per row list[int]
    min_tokens: dict = field(default_factory=dict)  # row -> (min_tokens, stop_ids)
    logit_bias: list = field(default_factory=list)  # per row dict | None
    allowed_token_ids: list = field(default_factory=list)  # per row list | None
    bad_words_token_ids: dict = field(default_factory=dict)  # row -> list[list[int]]
    grammar_bitmask: Optional[torch.Tensor] = None
    thinking: dict = field(default_factory=dict)  # row -> (budget, think-start id, think-end id)
    custom_processors: list = field(default_factory=list)  # engine-level user logits processors (objects with ``apply``)
    row_info: list = field(default_factory=list)  # per row: request id, prompt / output token ids, SamplingParams.extra_args
