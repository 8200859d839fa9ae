"""Request / response schemas of the OpenAI-compatible API (reference: vllm/entrypoints/openai/*/protocol.py)."""
from __future__ import annotations

import time
import uuid
from typing import Any, Literal, Optional, Union

from pydantic import BaseModel, ConfigDict, Field

from onecat_vllm.sampling_params import RepetitionDetectionParams, RequestOutputKind, SamplingParams, StructuredOutputsParams


class _Base(BaseModel):
    model_config = ConfigDict(extra="allow")


class _SamplingMixin(_Base):
    model: Optional[str] = None
    max_tokens: Optional[int] = None
    temperature: Optional[float] = None
    top_p: Optional[float] = None
    top_k: Optional[int] = None
    min_p: Optional[float] = None
    n: int = 1
    seed: Optional[int] = None
    stop: Optional[Union[str, list[str]]] = None
    stop_token_ids: Optional[list[int]] = None
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    repetition_penalty: float = 1.0
    logit_bias: Optional[dict[str, float]] = None
    ignore_eos: bool = False
    min_tokens: int = 0
    skip_special_tokens: bool = True
    stream: bool = False
    stream_options: Optional[dict] = None
    priority: int = 0
    response_format: Optional[dict] = None
    structured_outputs: Optional[dict] = None
    allowed_token_ids: Optional[list[int]] = None
    bad_words: Optional[list[str]] = None
    thinking_token_budget: Optional[int] = None
    repetition_detection: Optional[dict] = None
    prompt_logprobs: Optional[int] = None
    truncate_prompt_tokens: Optional[int] = None
    include_stop_str_in_output: bool = False
    guided_json: Optional[Union[str, dict]] = None       # earlier spellings of structured_outputs
    guided_regex: Optional[str] = None
    guided_choice: Optional[list[str]] = None
    guided_grammar: Optional[str] = None
    user: Optional[str] = None

    def to_sampling_params(self, default_max_tokens: int, logprobs: Optional[int] = None) -> SamplingParams:
        so = None
        if self.structured_outputs:
            so = StructuredOutputsParams(**self.structured_outputs)
        elif self.guided_json is not None or self.guided_regex or self.guided_choice or self.guided_grammar:
            so = StructuredOutputsParams(json=self.guided_json, regex=self.guided_regex, choice=self.guided_choice, grammar=self.guided_grammar)
        elif self.response_format and self.response_format.get("type") == "json_object":
            so = StructuredOutputsParams(json_object=True)
        elif self.response_format and self.response_format.get("type") == "json_schema":
            so = StructuredOutputsParams(json=self.response_format.get("json_schema", {}).get("schema"))
        return SamplingParams(
            n=self.n, presence_penalty=self.presence_penalty, frequency_penalty=self.frequency_penalty,
            repetition_penalty=self.repetition_penalty, temperature=1.0 if self.temperature is None else self.temperature,
            top_p=1.0 if self.top_p is None else self.top_p, top_k=self.top_k or 0, min_p=self.min_p or 0.0, seed=self.seed,
            stop=self.stop, stop_token_ids=self.stop_token_ids, ignore_eos=self.ignore_eos,
            max_tokens=self.max_tokens if self.max_tokens is not None else default_max_tokens, min_tokens=self.min_tokens,
            logprobs=logprobs, skip_special_tokens=self.skip_special_tokens,
            logit_bias={int(k): float(v) for k, v in self.logit_bias.items()} if self.logit_bias else None,
            allowed_token_ids=self.allowed_token_ids, bad_words=self.bad_words, structured_outputs=so,
            thinking_token_budget=self.thinking_token_budget, prompt_logprobs=self.prompt_logprobs,
            truncate_prompt_tokens=self.truncate_prompt_tokens, include_stop_str_in_output=self.include_stop_str_in_output,
            repetition_detection=RepetitionDetectionParams(**self.repetition_detection) if self.repetition_detection else None,
            output_kind=RequestOutputKind.DELTA if self.stream else RequestOutputKind.FINAL_ONLY)


class CompletionRequest(_SamplingMixin):
    prompt: Union[str, list[int], list[str], list[list[int]]]
    echo: bool = False
    logprobs: Optional[int] = None


class ChatMessage(_Base):
    role: str
    content: Optional[Union[str, list[dict]]] = None
    name: Optional[str] = None
    tool_calls: Optional[list[dict]] = None
    tool_call_id: Optional[str] = None
    reasoning_content: Optional[str] = None


class ChatCompletionRequest(_SamplingMixin):
    messages: list[ChatMessage]
    max_completion_tokens: Optional[int] = None
    logprobs: bool = False
    top_logprobs: Optional[int] = None
    tools: Optional[list[dict]] = None
    tool_choice: Optional[Union[str, dict]] = "auto"
    add_generation_prompt: bool = True
    chat_template: Optional[str] = None
    chat_template_kwargs: Optional[dict] = None


class TokenizeRequest(_Base):
    model: Optional[str] = None
    prompt: Optional[str] = None
    messages: Optional[list[ChatMessage]] = None
    add_special_tokens: bool = True


class DetokenizeRequest(_Base):
    model: Optional[str] = None
    tokens: list[int]


class UsageInfo(_Base):
    prompt_tokens: int = 0
    completion_tokens: int = 0
    total_tokens: int = 0
    prompt_tokens_details: Optional[dict] = None


def new_id(prefix: str) -> str:
    return f"{prefix}-{uuid.uuid4().hex}"


def error_body(message: str, typ: str = "BadRequestError", code: int = 400) -> dict:
    return {"error": {"message": message, "type": typ, "param": None, "code": code}}


def now() -> int:
    return int(time.time())
