"""Prompt input types (reference: vllm/inputs/)."""
from __future__ import annotations

from typing import Optional, TypedDict, Union


class TextPrompt(TypedDict, total=False):
    prompt: str
    cache_salt: Optional[str]


class TokensPrompt(TypedDict, total=False):
    prompt_token_ids: list[int]
    prompt: Optional[str]
    cache_salt: Optional[str]


class EmbedsPrompt(TypedDict, total=False):
    """Precomputed input embeddings ``[num_tokens, hidden_size]`` instead of token ids: the output of an external encoder (for
    instance a vision tower) or of the model's own embedding table (reference: vllm/inputs/data.py ``EmbedsPrompt``)."""

    prompt_embeds: object
    cache_salt: Optional[str]


PromptType = Union[str, list[int], TextPrompt, TokensPrompt, EmbedsPrompt]


def parse_prompt(p: PromptType) -> tuple[Optional[str], Optional[list[int]], Optional[str]]:
    """Returns (text, token_ids, cache_salt)."""
    if isinstance(p, str):
        return p, None, None
    if isinstance(p, (list, tuple)):
        return None, [int(t) for t in p], None
    if isinstance(p, dict):
        if "prompt_token_ids" in p:
            return p.get("prompt"), [int(t) for t in p["prompt_token_ids"]], p.get("cache_salt")
        if "prompt" in p:
            return p["prompt"], None, p.get("cache_salt")
    raise TypeError(f"unsupported prompt type: {type(p)}")
