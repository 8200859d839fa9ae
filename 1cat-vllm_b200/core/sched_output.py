"""Structures exchanged between scheduler and model runner
(reference: vllm/v1/core/sched/output.py; v1/outputs.py ``ModelRunnerOutput``)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional

from onecat_vllm.sampling_params import SamplingParams


@dataclass
class NewRequestData:
    req_id: str
    prompt_token_ids: list[int]
    sampling_params: Optional[SamplingParams]
    block_ids: list[int]
    num_computed_tokens: int
    state_slot: int = -1
    eos_token_id: Optional[int] = None
    pooling_params: Any = None
    lora_request: Any = None
    prompt_embeds: Any = None
    mm_features: Any = None


@dataclass
class CachedRequestData:
    """Requests the runner already knows: only deltas travel."""

    req_ids: list[str] = field(default_factory=list)
    resumed_from_preemption: list[bool] = field(default_factory=list)
    new_token_ids: list[list[int]] = field(default_factory=list)  # for resumed requests: all tokens
    new_block_ids: list[Optional[list[int]]] = field(default_factory=list)
    num_computed_tokens: list[int] = field(default_factory=list)
    state_slots: list[int] = field(default_factory=list)

    @property
    def num_reqs(self) -> int:
        return len(self.req_ids)


@dataclass
class SchedulerOutput:
    scheduled_new_reqs: list[NewRequestData] = field(default_factory=list)
    scheduled_cached_reqs: CachedRequestData = field(default_factory=CachedRequestData)
    num_scheduled_tokens: dict[str, int] = field(default_factory=dict)
    total_num_scheduled_tokens: int = 0
    scheduled_spec_decode_tokens: dict[str, list[int]] = field(default_factory=dict)
    finished_req_ids: set = field(default_factory=set)
    preempted_req_ids: set = field(default_factory=set)
    num_common_prefix_blocks: int = 0
    grammar_bitmask: Any = None  # numpy int32 [rows, ceil(vocab/32)], bit set = token allowed
    structured_rows: dict[str, int] = field(default_factory=dict)  # request id -> row of grammar_bitmask
    kv_swap_out: list = field(default_factory=list)  # (GPU block, CPU block): save before the step's forward
    kv_swap_in: list = field(default_factory=list)   # (CPU block, GPU block): restore before the step's forward
    scheduled_encoder_inputs: dict[str, list[int]] = field(default_factory=dict)  # request id -> indices of its multimodal items to encode
    free_encoder_mm_hashes: list = field(default_factory=list)  # encoder outputs the workers may drop

    @property
    def is_empty(self) -> bool:
        return self.total_num_scheduled_tokens == 0


@dataclass
class LogprobsLists:
    """Per sampled token: top-k ids, their logprobs, and the rank of the sampled token."""

    token_ids: list[list[int]]
    logprobs: list[list[float]]
    ranks: list[int]


@dataclass
class ModelRunnerOutput:
    req_ids: list[str] = field(default_factory=list)
    sampled_token_ids: list[list[int]] = field(default_factory=list)  # per request; >1 with spec decode
    spec_token_ids: Optional[list[list[int]]] = None  # drafts for the next step
    logprobs: Optional[list[Optional[LogprobsLists]]] = None
    prompt_logprobs: Optional[dict] = None
    num_nans_in_logits: Optional[dict] = None
    pooler_output: Optional[list] = None  # per request: pooled vector (list of floats) once its prompt is complete, else None
    device_time_ms: float = 0.0  # CUDA-event time of the step (0 when not measured)
    status: int = 0  # non-zero: a bounded device wait expired


EMPTY_MODEL_RUNNER_OUTPUT = ModelRunnerOutput()
