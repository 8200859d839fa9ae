"""Frontend request/response processing (reference: vllm/v1/engine/input_processor.py:36,
output_processor.py:417, parallel_sampling.py, logprobs.py).

``InputProcessor`` validates and tokenises a prompt into an ``EngineCoreRequest``. ``OutputProcessor`` turns the
engine core's token deltas into ``RequestOutput`` objects: incremental detokenisation, stop strings (reported
back so the engine aborts the request), logprob assembly, n>1 fan-in, and per-request timing for metrics."""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Optional

from onecat_vllm.config import VllmConfig
from onecat_vllm.engine.tokenizer import IncrementalDetokenizer
from onecat_vllm.inputs import PromptType, parse_prompt
from onecat_vllm.outputs import CompletionOutput, Logprob, PoolingOutput, PoolingRequestOutput, RequestMetrics, RequestOutput
from onecat_vllm.request import EngineCoreOutput, EngineCoreRequest, FinishReason
from onecat_vllm.sampling_params import PoolingParams, RequestOutputKind, SamplingParams


class InputProcessor:
    def __init__(self, cfg: VllmConfig, tokenizer):
        self.cfg, self.tok = cfg, tokenizer

    def _think_token_ids(self):
        if self.tok is None:
            return None
        if not hasattr(self, "_think_cache"):
            a, b = _single_token(self.tok, "<think>"), _single_token(self.tok, "</think>")
            self._think_cache = (a, b) if a is not None and b is not None else None
        return self._think_cache

    def process(self, request_id: str, prompt: PromptType, params: SamplingParams, arrival_time: Optional[float] = None,
                priority: int = 0, lora_request=None) -> tuple[EngineCoreRequest, Optional[str]]:
        if lora_request is not None and not self.cfg.model_config.enable_lora:
            raise ValueError("this engine was started without enable_lora")
        embeds = prompt.get("prompt_embeds") if isinstance(prompt, dict) else None
        if embeds is not None:
            import torch
            embeds = torch.as_tensor(embeds)
            if embeds.dim() != 2 or embeds.shape[1] != self.cfg.model_config.hidden_size:
                raise ValueError(f"prompt_embeds must be [num_tokens, {self.cfg.model_config.hidden_size}]")
            text, ids, salt = None, [0] * embeds.shape[0], prompt.get("cache_salt")
        else:
            text, ids, salt = parse_prompt(prompt)
        if ids is None:
            if self.tok is None:
                raise ValueError("text prompts need a tokenizer; pass token ids or set tokenizer=")
            ids = list(self.tok.encode(text))
        mc = self.cfg.model_config
        k = getattr(params, "truncate_prompt_tokens", None)
        if k is not None and embeds is None:
            if k == -1:
                k = mc.max_model_len - 1
            if k < 1:
                raise ValueError("truncate_prompt_tokens must be a positive integer or -1")
            ids = list(ids)[-k:]   # left truncation, as the reference does
        mm_features = None
        mm_data = prompt.get("multi_modal_data") if isinstance(prompt, dict) else None
        if mm_data:
            if embeds is not None:
                raise ValueError("multi_modal_data cannot be combined with prompt_embeds")
            if getattr(self, "_mm_processor", None) is None:
                from onecat_vllm.multimodal import MULTIMODAL_REGISTRY
                self._mm_processor = MULTIMODAL_REGISTRY.create_processor(mc)
            if self._mm_processor is None:
                raise ValueError("this model takes no multimodal inputs (its config names no image / video / audio token)")
            done = self._mm_processor.apply(list(ids), mm_data)
            ids, mm_features = done.token_ids, done.features
        if not ids:
            raise ValueError("the prompt is empty")
        if len(ids) >= mc.max_model_len:
            raise ValueError(f"prompt has {len(ids)} tokens but max_model_len is {mc.max_model_len}")
        bad = [t for t in ids if not 0 <= t < mc.vocab_size]
        if bad:
            raise ValueError(f"token id {bad[0]} is outside the vocabulary (size {mc.vocab_size})")
        pooling = None
        if isinstance(params, PoolingParams):
            if params.task == "classify" and mc.num_labels <= 0:
                raise ValueError("classify needs a *ForSequenceClassification checkpoint (this model has no score head)")
            # an embedding request runs its prompt, "generates" one token that nobody reads, and returns the pooled state
            pooling, params = params, SamplingParams(temperature=0.0, max_tokens=1, detokenize=False,
                                                     output_kind=RequestOutputKind.FINAL_ONLY)
        sp = params.clone()
        if sp.max_tokens is None:
            sp.max_tokens = mc.max_model_len - len(ids)
        if sp.logprobs is not None and sp.logprobs > 20 and sp.logprobs != -1:
            raise ValueError("at most 20 logprobs per token can be requested")
        eos = mc.eos_token_id if mc.eos_token_id is not None else getattr(self.tok, "eos_token_id", None)
        sp.update_from_generation_config(eos)
        if sp.thinking_token_budget is not None:
            if sp.thinking_token_budget < 0:
                raise ValueError("thinking_token_budget must be a non-negative integer")
            sp._think_ids = self._think_token_ids()
            if sp._think_ids is None:
                raise ValueError("thinking_token_budget needs a tokenizer in which <think> and </think> are single tokens")
        if sp.bad_words and self.tok is not None and not sp.bad_words_token_ids:
            sp.bad_words_token_ids = [self.tok.encode(w, add_special_tokens=False) for w in sp.bad_words]
        if sp.allowed_token_ids is not None and any(not 0 <= t < mc.vocab_size for t in sp.allowed_token_ids):
            raise ValueError("allowed_token_ids contains an id outside the vocabulary")
        req = EngineCoreRequest(request_id, ids, sp, arrival_time or time.time(), eos, priority, salt, pooling_params=pooling,
                                lora_request=lora_request, prompt_embeds=embeds, mm_features=mm_features)
        return req, text


def _single_token(tok, text: str):
    try:
        ids = tok.encode(text, add_special_tokens=False)
    except TypeError:
        ids = tok.encode(text)
    return ids[0] if len(ids) == 1 else None


@dataclass
class _ReqState:
    request_id: str
    parent_id: Optional[str]
    index: int
    prompt: Optional[str]
    prompt_ids: list
    params: SamplingParams
    detok: IncrementalDetokenizer
    arrival: float
    logprobs: Optional[list] = None
    cum_logprob: float = 0.0
    sent_tokens: int = 0
    sent_chars: int = 0
    metrics: RequestMetrics = field(default_factory=RequestMetrics)
    queue: Optional[object] = None  # asyncio queue for streaming clients
    pooling: bool = False
    prompt_logprobs: Optional[list] = None


class OutputProcessor:
    def __init__(self, tokenizer, log_stats: bool = False):
        self.tok = tokenizer
        self.states: dict[str, _ReqState] = {}
        self.parents: dict[str, dict] = {}
        self.finished_stats: list = []

    def add_request(self, req: EngineCoreRequest, prompt: Optional[str], parent_id: Optional[str] = None, index: int = 0, queue=None) -> None:
        sp = req.sampling_params
        st = _ReqState(req.request_id, parent_id, index, prompt, req.prompt_token_ids, sp,
                       IncrementalDetokenizer(self.tok if sp.detokenize else None, req.prompt_token_ids, sp.skip_special_tokens,
                                              sp.stop, sp.include_stop_str_in_output), req.arrival_time, queue=queue)
        st.metrics.arrival_time = req.arrival_time
        st.pooling = req.pooling_params is not None
        if sp.logprobs is not None:
            st.logprobs = []
        if sp.prompt_logprobs is not None:
            st.prompt_logprobs = [None]  # the first prompt token has no predecessor
        self.states[req.request_id] = st
        if parent_id is not None:
            self.parents.setdefault(parent_id, {"n": sp.n, "done": {}, "prompt": prompt, "prompt_ids": req.prompt_token_ids})

    def abort(self, request_ids: list[str]) -> list[str]:
        out = []
        for rid in request_ids:
            if self.states.pop(rid, None) is not None:
                out.append(rid)
            for cid in [c for c, s in self.states.items() if s.parent_id == rid]:
                self.states.pop(cid)
                out.append(cid)
        return out

    def has_unfinished(self) -> bool:
        return bool(self.states)

    def process_outputs(self, outs: list[EngineCoreOutput], now: Optional[float] = None) -> tuple[list[RequestOutput], list[str]]:
        """Returns (request outputs to hand to the caller, ids the engine must abort because a stop string hit)."""
        now = now or time.time()
        results: list[RequestOutput] = []
        to_abort: list[str] = []
        for o in outs:
            st = self.states.get(o.request_id)
            if st is None:
                continue
            if st.metrics.first_token_time is None and o.new_token_ids:
                st.metrics.first_token_time = now
            st.metrics.last_token_time = now
            st.metrics.num_generation_tokens += len(o.new_token_ids)
            st.metrics.num_cached_tokens = o.num_cached_tokens
            finish, stop_reason = o.finish_reason, o.stop_reason
            stop_str = st.detok.update(o.new_token_ids, finished=finish is not None)
            if stop_str is not None and finish is None:
                finish, stop_reason = FinishReason.STOP, stop_str
                to_abort.append(o.request_id)
            if st.prompt_logprobs is not None and o.prompt_logprobs:
                for ids, lps, rank in o.prompt_logprobs:
                    d = {}
                    for j, (tid, lp) in enumerate(zip(ids, lps)):
                        if tid not in d:
                            d[tid] = Logprob(lp, rank if j == 0 else j, self.tok.decode([tid]) if self.tok is not None else None)
                    st.prompt_logprobs.append(d)
            if st.logprobs is not None and o.new_logprobs:
                for ids, lps, rank in o.new_logprobs:
                    d = {}
                    for j, (tid, lp) in enumerate(zip(ids, lps)):
                        if tid not in d:
                            d[tid] = Logprob(lp, rank if j == 0 else j, self.tok.decode([tid]) if self.tok is not None else None)
                    st.logprobs.append(d)
                    st.cum_logprob += lps[0]
            if st.pooling:
                ro = PoolingRequestOutput(st.request_id, PoolingOutput(list(o.pooling_output or [])), st.prompt_ids, True) \
                    if finish is not None else None
            else:
                ro = self._make_output(st, finish, stop_reason, o.num_cached_tokens)
            if finish is not None:
                st.metrics.finished_time = now
                st.metrics.num_prompt_tokens = len(st.prompt_ids)
                st.metrics.max_tokens = getattr(st.params, "max_tokens", None)
                st.metrics.finish_reason = str(finish)
                self.finished_stats.append(st.metrics)
                self.states.pop(o.request_id, None)
            if ro is not None:
                if st.queue is not None:
                    st.queue.put_nowait(ro)
                else:
                    results.append(ro)
        return results, to_abort

    def _make_output(self, st: _ReqState, finish, stop_reason, num_cached) -> Optional[RequestOutput]:
        kind = st.params.output_kind
        finished = finish is not None
        if kind == RequestOutputKind.FINAL_ONLY and not finished:
            return None
        ids, text = st.detok.ids, st.detok.text
        if kind == RequestOutputKind.DELTA:
            d_ids, d_text = ids[st.sent_tokens:], text[st.sent_chars:]
            lps = st.logprobs[st.sent_tokens:] if st.logprobs is not None else None
            st.sent_tokens, st.sent_chars = len(ids), len(text)
        else:
            d_ids, d_text, lps = list(ids), text, st.logprobs
        co = CompletionOutput(st.index, d_text, d_ids, st.cum_logprob if st.logprobs is not None else None, lps,
                              str(finish) if finished else None, stop_reason)
        if st.parent_id is None:
            return RequestOutput(st.request_id, st.prompt, st.prompt_ids, [co], finished, metrics=st.metrics, num_cached_tokens=num_cached,
                                 prompt_logprobs=st.prompt_logprobs)
        # n > 1: gather children under the parent id
        par = self.parents[st.parent_id]
        if finished:
            par["done"][st.index] = co
        if kind == RequestOutputKind.FINAL_ONLY:
            if len(par["done"]) < par["n"]:
                return None
            outs = [par["done"][i] for i in sorted(par["done"])]
            self.parents.pop(st.parent_id)
            return RequestOutput(st.parent_id, st.prompt, st.prompt_ids, outs, True, metrics=st.metrics)
        all_done = len(par["done"]) == par["n"]
        if all_done:
            self.parents.pop(st.parent_id, None)
        return RequestOutput(st.parent_id, st.prompt, st.prompt_ids, [co], all_done, metrics=st.metrics)
