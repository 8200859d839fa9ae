"""Sampling parameters of a request.

Same field names and defaults as the reference's msgspec struct
(reference: vllm/sampling_params.py:198-346); greedy iff ``temperature < 1e-5``
(reference: vllm/sampling_params.py:26).
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from enum import IntEnum
from typing import Any, Optional, Union

_SAMPLING_EPS = 1e-5
_MAX_TEMP = 1e-2


class SamplingType(IntEnum):
    GREEDY = 0
    RANDOM = 1
    RANDOM_SEED = 2


class RequestOutputKind(IntEnum):
    CUMULATIVE = 0  # whole output so far on every update
    DELTA = 1  # only new tokens/text
    FINAL_ONLY = 2  # nothing until the request is finished


@dataclass
class StructuredOutputsParams:
    json: Optional[Union[str, dict]] = None
    regex: Optional[str] = None
    choice: Optional[list[str]] = None
    grammar: Optional[str] = None
    json_object: Optional[bool] = None

    def kind(self) -> str:
        for k in ("json", "regex", "choice", "grammar", "json_object"):
            if getattr(self, k):
                return k
        return "none"


@dataclass
class RepetitionDetectionParams:
    """Stop a request whose output ends in an n-gram (``min_pattern_size`` .. ``max_pattern_size`` tokens) repeated ``min_count`` times
    in a row (reference: vllm/sampling_params.py:145 ``RepetitionDetectionParams``). ``max_pattern_size = 0`` disables it."""

    max_pattern_size: int = 0
    min_pattern_size: int = 0
    min_count: int = 0

    def __post_init__(self) -> None:
        if self.max_pattern_size < 0 or self.min_pattern_size < 0 or self.min_pattern_size > self.max_pattern_size:
            raise ValueError("need 0 <= min_pattern_size <= max_pattern_size")
        if self.max_pattern_size > 0 and self.min_count < 2:
            raise ValueError("min_count must be >= 2 when repetition detection is on")

    def hit(self, tokens: list) -> bool:
        if self.max_pattern_size <= 0:
            return False
        for p in range(max(self.min_pattern_size, 1), self.max_pattern_size + 1):
            need = p * self.min_count
            if len(tokens) < need:
                break
            tail = tokens[-need:]
            if all(tail[i] == tail[i % p] for i in range(p, need)):
                return True
        return False


@dataclass
class SamplingParams:
    n: int = 1
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    repetition_penalty: float = 1.0
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = 0
    min_p: float = 0.0
    seed: Optional[int] = None
    stop: Optional[Union[str, list[str]]] = None
    stop_token_ids: Optional[list[int]] = None
    ignore_eos: bool = False
    max_tokens: Optional[int] = 16
    min_tokens: int = 0
    logprobs: Optional[int] = None
    prompt_logprobs: Optional[int] = None
    detokenize: bool = True
    skip_special_tokens: bool = True
    spaces_between_special_tokens: bool = True
    include_stop_str_in_output: bool = False
    truncate_prompt_tokens: Optional[int] = None  # keep only the last k prompt tokens (-1: as many as max_model_len allows)
    logit_bias: Optional[dict[int, float]] = None
    allowed_token_ids: Optional[list[int]] = None
    bad_words: Optional[list[str]] = None
    bad_words_token_ids: Optional[list[list[int]]] = None
    structured_outputs: Optional[StructuredOutputsParams] = None
    thinking_token_budget: Optional[int] = None  # at most this many tokens between the think-start and think-end tokens
    repetition_detection: Optional[RepetitionDetectionParams] = None
    output_kind: RequestOutputKind = RequestOutputKind.CUMULATIVE
    extra_args: Optional[dict[str, Any]] = None
    # internal: eos ids resolved by the input processor
    _eos_token_id: Optional[int] = field(default=None, repr=False)
    _think_ids: Optional[tuple] = field(default=None, repr=False)  # (think-start id, think-end id), resolved by the input processor
    _all_stop_token_ids: set = field(default_factory=set, repr=False)

    def __post_init__(self) -> None:
        if isinstance(self.stop, str):
            self.stop = [self.stop]
        elif self.stop is None:
            self.stop = []
        if self.stop_token_ids is None:
            self.stop_token_ids = []
        if 0 < self.temperature < _MAX_TEMP:
            self.temperature = max(self.temperature, _MAX_TEMP)
        if self.top_k is None or self.top_k < 0:
            self.top_k = 0
        if self.temperature < _SAMPLING_EPS:  # greedy: neutralise the random knobs
            self.top_p, self.top_k, self.min_p = 1.0, 0, 0.0
        self._verify()
        self._all_stop_token_ids = set(self.stop_token_ids)

    def _verify(self) -> None:
        if not isinstance(self.n, int) or self.n < 1:
            raise ValueError(f"n must be an int >= 1, got {self.n}")
        if not -2.0 <= self.presence_penalty <= 2.0:
            raise ValueError("presence_penalty must be in [-2, 2]")
        if not -2.0 <= self.frequency_penalty <= 2.0:
            raise ValueError("frequency_penalty must be in [-2, 2]")
        if self.repetition_penalty <= 0.0:
            raise ValueError("repetition_penalty must be > 0")
        if self.temperature < 0.0:
            raise ValueError("temperature must be non-negative")
        if not 0.0 < self.top_p <= 1.0:
            raise ValueError("top_p must be in (0, 1]")
        if not 0.0 <= self.min_p <= 1.0:
            raise ValueError("min_p must be in [0, 1]")
        if self.max_tokens is not None and self.max_tokens < 1:
            raise ValueError("max_tokens must be at least 1")
        if self.min_tokens < 0:
            raise ValueError("min_tokens must be >= 0")
        if self.max_tokens is not None and self.min_tokens > self.max_tokens:
            raise ValueError("min_tokens must be <= max_tokens")
        if self.logprobs is not None and self.logprobs < -1:
            raise ValueError("logprobs must be >= -1")
        if self.stop and not self.detokenize:
            raise ValueError("stop strings need detokenize=True")
        if self.n > 1 and self.temperature < _SAMPLING_EPS:
            raise ValueError("n > 1 needs temperature > 0 (greedy would repeat one sample)")

    @property
    def sampling_type(self) -> SamplingType:
        if self.temperature < _SAMPLING_EPS:
            return SamplingType.GREEDY
        if self.seed is not None:
            return SamplingType.RANDOM_SEED
        return SamplingType.RANDOM

    @property
    def all_stop_token_ids(self) -> set:
        return self._all_stop_token_ids

    def update_from_generation_config(self, eos_token_id: Optional[int], extra_eos: Optional[list[int]] = None) -> None:
        self._eos_token_id = eos_token_id
        if extra_eos and not self.ignore_eos:
            self._all_stop_token_ids.update(e for e in extra_eos if e != eos_token_id)

    def clone(self) -> "SamplingParams":
        return copy.deepcopy(self)

    def to_dict(self) -> dict:
        d = {k: v for k, v in self.__dict__.items() if not k.startswith("_")}
        d["output_kind"] = int(self.output_kind)
        if self.structured_outputs is not None:
            d["structured_outputs"] = dict(self.structured_outputs.__dict__)
        if self.repetition_detection is not None:
            d["repetition_detection"] = dict(self.repetition_detection.__dict__)
        if self._think_ids is not None:
            d["_think_ids"] = list(self._think_ids)
        return d

    @classmethod
    def from_dict(cls, d: dict) -> "SamplingParams":
        d = dict(d)
        d["output_kind"] = RequestOutputKind(d.get("output_kind", 0))
        so = d.get("structured_outputs")
        if isinstance(so, dict):
            d["structured_outputs"] = StructuredOutputsParams(**so)
        if isinstance(d.get("repetition_detection"), dict):
            d["repetition_detection"] = RepetitionDetectionParams(**d["repetition_detection"])
        think = d.pop("_think_ids", None)
        sp = cls(**d)
        sp._think_ids = tuple(think) if think else None
        return sp


@dataclass
class BeamSearchParams:
    """Parameters of ``LLM.beam_search`` (reference: vllm/sampling_params.py ``BeamSearchParams``)."""

    beam_width: int
    max_tokens: int
    ignore_eos: bool = False
    temperature: float = 0.0
    length_penalty: float = 1.0


@dataclass
class PoolingParams:
    """Parameters of an embedding / classify request (reference: vllm/pooling_params.py)."""

    task: str = "embed"  # embed | encode (raw hidden state) | score | classify (needs a sequence-classification checkpoint)
    normalize: bool = True
    use_activation: bool = True  # classify: softmax over the labels (sigmoid for a single label) instead of raw logits
    dimensions: Optional[int] = None  # matryoshka truncation
    pooling_type: str = "last"  # last | mean | cls

    def __post_init__(self) -> None:
        if self.pooling_type not in ("last", "mean", "cls"):
            raise ValueError(f"unknown pooling_type '{self.pooling_type}'")

    def to_dict(self) -> dict:
        return dict(task=self.task, normalize=self.normalize, dimensions=self.dimensions, pooling_type=self.pooling_type,
                    use_activation=self.use_activation)
