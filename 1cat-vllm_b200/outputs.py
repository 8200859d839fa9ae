"""Result objects returned to API users (reference: vllm/outputs.py)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional


@dataclass
class Logprob:
    logprob: float
    rank: Optional[int] = None
    decoded_token: Optional[str] = None


@dataclass
class CompletionOutput:
    index: int
    text: str
    token_ids: list[int]
    cumulative_logprob: Optional[float] = None
    logprobs: Optional[list[dict[int, Logprob]]] = None
    finish_reason: Optional[str] = None
    stop_reason: Optional[int | str] = None

    def finished(self) -> bool:
        return self.finish_reason is not None


@dataclass
class RequestMetrics:
    arrival_time: float = 0.0
    first_scheduled_time: Optional[float] = None
    first_token_time: Optional[float] = None
    last_token_time: Optional[float] = None
    finished_time: Optional[float] = None
    num_cached_tokens: int = 0
    num_prompt_tokens: int = 0
    num_generation_tokens: int = 0
    max_tokens: Optional[int] = None
    finish_reason: Optional[str] = None


@dataclass
class RequestOutput:
    request_id: str
    prompt: Optional[str]
    prompt_token_ids: list[int]
    outputs: list[CompletionOutput]
    finished: bool
    prompt_logprobs: Optional[list] = None
    metrics: Optional[RequestMetrics] = None
    num_cached_tokens: int = 0

    def add(self, nxt: "RequestOutput", aggregate: bool) -> None:
        """Merge a later output of the same request (reference: vllm/outputs.py RequestOutput.add)."""
        self.finished |= nxt.finished
        for o in nxt.outputs:
            for mine in self.outputs:
                if mine.index == o.index:
                    if aggregate:
                        mine.text += o.text
                        mine.token_ids.extend(o.token_ids)
                        if o.logprobs:
                            mine.logprobs = (mine.logprobs or []) + o.logprobs
                        mine.cumulative_logprob = o.cumulative_logprob
                    else:
                        mine.text, mine.token_ids, mine.logprobs = o.text, o.token_ids, o.logprobs
                        mine.cumulative_logprob = o.cumulative_logprob
                    mine.finish_reason, mine.stop_reason = o.finish_reason, o.stop_reason
                    break
            else:
                self.outputs.append(o)


@dataclass
class PoolingOutput:
    data: list[float] = field(default_factory=list)

    @property
    def embedding(self) -> list[float]:
        return self.data


@dataclass
class PoolingRequestOutput:
    request_id: str
    outputs: PoolingOutput
    prompt_token_ids: list[int]
    finished: bool = True
