"""Engine-side request state (reference: vllm/v1/request.py, v1/engine/__init__.py:42-238)."""
from __future__ import annotations

import enum
import time
from dataclasses import dataclass, field
from typing import Any, Optional

from onecat_vllm.sampling_params import SamplingParams


class FinishReason(enum.IntEnum):
    STOP = 0
    LENGTH = 1
    ABORT = 2
    ERROR = 3

    def __str__(self) -> str:
        return ("stop", "length", "abort", "error")[int(self)]


class RequestStatus(enum.IntEnum):
    WAITING = 0
    RUNNING = 1
    PREEMPTED = 2
    FINISHED_STOPPED = 3
    FINISHED_LENGTH_CAPPED = 4
    FINISHED_ABORTED = 5
    FINISHED_ERROR = 6

    @staticmethod
    def is_finished(s: "RequestStatus") -> bool:
        return s >= RequestStatus.FINISHED_STOPPED

    @staticmethod
    def finish_reason(s: "RequestStatus") -> Optional[FinishReason]:
        return {RequestStatus.FINISHED_STOPPED: FinishReason.STOP, RequestStatus.FINISHED_LENGTH_CAPPED: FinishReason.LENGTH,
                RequestStatus.FINISHED_ABORTED: FinishReason.ABORT, RequestStatus.FINISHED_ERROR: FinishReason.ERROR}.get(s)


@dataclass
class EngineCoreRequest:
    """What crosses the frontend → engine-core boundary (reference: v1/engine/__init__.py:82-131)."""

    request_id: str
    prompt_token_ids: list[int]
    sampling_params: Optional[SamplingParams]
    arrival_time: float = 0.0
    eos_token_id: Optional[int] = None
    priority: int = 0
    cache_salt: Optional[str] = None
    client_index: int = 0
    data_parallel_rank: Optional[int] = None
    pooling_params: Any = None
    lora_request: Any = None
    trace_headers: Optional[dict] = None
    prompt_embeds: Any = None  # [num_prompt_tokens, hidden] tensor replacing the embedding lookup of the prompt
    mm_features: Any = None    # list[MultiModalFeature]: placeholder ranges of the prompt and their encoder inputs

    def to_wire(self) -> dict:
        return {"request_id": self.request_id, "prompt_token_ids": self.prompt_token_ids,
                "sampling_params": self.sampling_params.to_dict() if self.sampling_params else None,
                "arrival_time": self.arrival_time, "eos_token_id": self.eos_token_id, "priority": self.priority,
                "cache_salt": self.cache_salt, "client_index": self.client_index,
                "pooling_params": self.pooling_params.to_dict() if self.pooling_params is not None else None,
                "lora_request": self.lora_request.to_dict() if self.lora_request is not None else None,
                "prompt_embeds": self.prompt_embeds, "mm_features": [f.to_wire() for f in self.mm_features] if self.mm_features else None}

    @classmethod
    def from_wire(cls, d: dict) -> "EngineCoreRequest":
        sp = d.get("sampling_params")
        pp = d.get("pooling_params")
        if pp is not None:
            from onecat_vllm.sampling_params import PoolingParams
            pp = PoolingParams(**pp)
        return cls(d["request_id"], list(d["prompt_token_ids"]), SamplingParams.from_dict(sp) if sp else None,
                   d.get("arrival_time", 0.0), d.get("eos_token_id"), d.get("priority", 0), d.get("cache_salt"),
                   d.get("client_index", 0), pooling_params=pp, lora_request=_lora_from(d.get("lora_request")),
                   prompt_embeds=d.get("prompt_embeds"), mm_features=_mm_from(d.get("mm_features")))


@dataclass
class EngineCoreOutput:
    """Per-request delta produced by one engine step (reference: v1/engine/__init__.py:169-195)."""

    request_id: str
    new_token_ids: list[int]
    finish_reason: Optional[FinishReason] = None
    stop_reason: Optional[int | str] = None
    new_logprobs: Optional[list] = None  # per new token: (token_ids, logprobs, ranks)
    prompt_logprobs: Optional[list] = None
    num_cached_tokens: int = 0
    events: Optional[list] = None
    pooling_output: Optional[list] = None  # pooled hidden state of an embedding request (floats)

    @property
    def finished(self) -> bool:
        return self.finish_reason is not None

    def to_wire(self) -> dict:
        return {"request_id": self.request_id, "new_token_ids": self.new_token_ids,
                "finish_reason": None if self.finish_reason is None else int(self.finish_reason),
                "stop_reason": self.stop_reason, "new_logprobs": self.new_logprobs,
                "prompt_logprobs": self.prompt_logprobs, "num_cached_tokens": self.num_cached_tokens,
                "pooling_output": self.pooling_output}

    @classmethod
    def from_wire(cls, d: dict) -> "EngineCoreOutput":
        fr = d.get("finish_reason")
        return cls(d["request_id"], list(d["new_token_ids"]), None if fr is None else FinishReason(fr), d.get("stop_reason"),
                   d.get("new_logprobs"), d.get("prompt_logprobs"), d.get("num_cached_tokens", 0),
                   pooling_output=d.get("pooling_output"))


@dataclass
class EngineCoreOutputs:
    """One step's outputs for one client (reference: v1/engine/__init__.py:214-238)."""

    outputs: list[EngineCoreOutput] = field(default_factory=list)
    scheduler_stats: Any = None
    timestamp: float = 0.0
    engine_index: int = 0
    finished_requests: Optional[set] = None
    utility_output: Any = None

    def __post_init__(self) -> None:
        if not self.timestamp:
            self.timestamp = time.monotonic()


def _lora_from(d):
    if not d:
        return None
    from onecat_vllm.lora import LoRARequest
    return LoRARequest.from_dict(d)


def _mm_from(lst):
    if not lst:
        return None
    from onecat_vllm.multimodal import MultiModalFeature
    return [f if isinstance(f, MultiModalFeature) else MultiModalFeature.from_wire(f) for f in lst]


class Request:
    """Scheduler-side request. Tokens = prompt + outputs; ``num_computed_tokens`` chases
    ``num_tokens_with_spec`` (reference: v1/core/sched/scheduler.py:459-468)."""

    def __init__(self, request_id: str, prompt_token_ids: list[int], sampling_params: Optional[SamplingParams],
                 eos_token_id: Optional[int] = None, arrival_time: Optional[float] = None, priority: int = 0,
                 cache_salt: Optional[str] = None, client_index: int = 0, block_hasher=None, pooling_params=None, lora_request=None,
                 prompt_embeds=None, mm_features=None) -> None:
        self.request_id = request_id
        self.prompt_embeds = prompt_embeds
        self.mm_features = list(mm_features or [])
        self.mm_cached: set = set()  # indices of the items whose encoder output this request holds a reference to
        if self.mm_features:  # the same placeholder ids stand for different images: the items' hashes salt the prefix cache
            cache_salt = f"{cache_salt or ''}|mm:" + ",".join(f.mm_hash[:16] for f in self.mm_features)
        if prompt_embeds is not None:  # placeholder ids say nothing about the content: never share KV blocks with another request
            cache_salt = f"{cache_salt or ''}|embeds:{request_id}"
        self.lora_request = lora_request
        if lora_request is not None:  # KV computed under an adapter is only reusable under the same adapter
            cache_salt = f"{cache_salt or ''}|lora:{lora_request.lora_int_id}"
        self.prompt_token_ids = list(prompt_token_ids)
        self.sampling_params = sampling_params
        self.pooling_params = pooling_params
        self.eos_token_id = eos_token_id
        self.arrival_time = time.time() if arrival_time is None else arrival_time
        self.priority = priority
        self.cache_salt = cache_salt
        self.client_index = client_index
        self.status = RequestStatus.WAITING
        self.stop_reason: Optional[int | str] = None
        self.num_prompt_tokens = len(self.prompt_token_ids)
        self._output_token_ids: list[int] = []
        self._all_token_ids: list[int] = list(self.prompt_token_ids)
        self.spec_token_ids: list[int] = []
        self.num_computed_tokens = 0
        self.num_cached_tokens = -1
        self.num_preemptions = 0
        self.num_output_placeholders = 0  # async scheduling
        self.max_tokens = sampling_params.max_tokens if sampling_params and sampling_params.max_tokens is not None else 1 << 30
        self.block_hashes: list[bytes] = []
        self._block_hasher = block_hasher
        self.events: list = []
        so = sampling_params.structured_outputs if sampling_params is not None else None
        self.use_structured_output = so is not None and so.kind() != "none"
        # Draft tokens are verified against softmax(logits / temperature) only. A request whose sampling also filters or edits the
        # logits (top-k / top-p / min-p, penalties, bias, allowed ids, bad words, min_tokens, a thinking budget, its own seed) is
        # decoded without drafts, like a structured-output request, so that its tokens come from exactly the distribution the
        # non-speculative sampler would use (reference: v1/sample/rejection_sampler.py applies the processors to all k+1 rows).
        sp = sampling_params
        if sp is None:
            self.spec_decode_ok = not self.use_structured_output
        else:
            edits = bool(sp.logit_bias or sp.allowed_token_ids or sp.bad_words or sp.bad_words_token_ids or sp.min_tokens > 0
                         or sp.thinking_token_budget is not None or sp.presence_penalty or sp.frequency_penalty or sp.repetition_penalty != 1.0
                         or (sp.extra_args or {}).get("logits_processors"))
            filters = sp.top_k > 0 or sp.top_p < 1.0 or sp.min_p > 0.0 or sp.seed is not None
            greedy = sp.temperature < 1e-5  # arg-max is unchanged by the filters
            self.spec_decode_ok = not self.use_structured_output and not edits and (greedy or not filters)
        self.first_scheduled_time: Optional[float] = None
        if block_hasher is not None:
            self.block_hashes = block_hasher(self)

    @classmethod
    def from_engine_core_request(cls, r: EngineCoreRequest, block_hasher=None) -> "Request":
        return cls(r.request_id, r.prompt_token_ids, r.sampling_params, r.eos_token_id, r.arrival_time, r.priority,
                   r.cache_salt, r.client_index, block_hasher, r.pooling_params, r.lora_request, r.prompt_embeds, r.mm_features)

    def append_output_token_ids(self, ids: int | list[int]) -> None:
        if isinstance(ids, int):
            ids = [ids]
        self._output_token_ids.extend(ids)
        self._all_token_ids.extend(ids)
        if self._block_hasher is not None:
            self.block_hashes.extend(self._block_hasher(self))

    @property
    def output_token_ids(self) -> list[int]:
        return self._output_token_ids

    @property
    def all_token_ids(self) -> list[int]:
        return self._all_token_ids

    @property
    def num_tokens(self) -> int:
        return len(self._all_token_ids)

    @property
    def num_tokens_with_spec(self) -> int:
        return len(self._all_token_ids) + len(self.spec_token_ids)

    @property
    def num_output_tokens(self) -> int:
        return len(self._output_token_ids)

    def is_finished(self) -> bool:
        return RequestStatus.is_finished(self.status)

    def get_finished_reason(self) -> Optional[FinishReason]:
        return RequestStatus.finish_reason(self.status)

    def __lt__(self, other: "Request") -> bool:  # priority queue order (reference: request_queue.py:131)
        return (self.priority, self.arrival_time, self.request_id) < (other.priority, other.arrival_time, other.request_id)
