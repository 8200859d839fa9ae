"""Unified token-budget scheduler.

Semantics follow the reference's v1 scheduler (reference: vllm/v1/core/sched/scheduler.py:75 class,
:458 ``schedule``, :1174 preemption, :1528 ``update_from_output``, :1936 ``update_draft_token_ids``;
stop checks v1/core/sched/utils.py ``check_stop``): there is no prefill/decode phase — each step gives
every request up to ``num_tokens_with_spec - num_computed_tokens`` tokens out of one budget, RUNNING
first, then WAITING; when blocks run out the lowest-priority running request is preempted.
"""
from __future__ import annotations

import heapq
import time
from collections import deque
from dataclasses import dataclass, field
from typing import Iterable, Optional

from onecat_vllm.config import VllmConfig
from onecat_vllm.core.kv_cache_manager import KVCacheManager
from onecat_vllm.core.kv_cache_utils import make_block_hasher
from onecat_vllm.core.sched_output import CachedRequestData, ModelRunnerOutput, NewRequestData, SchedulerOutput
from onecat_vllm.request import EngineCoreOutput, EngineCoreOutputs, FinishReason, Request, RequestStatus


@dataclass
class SchedulerStats:
    """Per-step gauges (reference: v1/metrics/stats.py:171)."""

    num_running_reqs: int = 0
    num_waiting_reqs: int = 0
    kv_cache_usage: float = 0.0
    prefix_cache_queries: int = 0
    prefix_cache_hits: int = 0
    num_preemptions: int = 0
    num_scheduled_tokens: int = 0
    spec_num_drafts: int = 0
    spec_num_draft_tokens: int = 0
    spec_num_accepted_tokens: int = 0
    step_device_ms: float = 0.0


class RequestQueue:
    """FCFS deque or priority heap behind one interface (reference: v1/core/sched/request_queue.py:75,131)."""

    def __init__(self, policy: str) -> None:
        self.policy = policy
        self._dq: deque = deque()
        self._heap: list = []

    def add(self, r: Request) -> None:
        if self.policy == "priority":
            heapq.heappush(self._heap, r)
        else:
            self._dq.append(r)

    def prepend(self, rs: Iterable[Request]) -> None:
        if self.policy == "priority":
            for r in rs:
                heapq.heappush(self._heap, r)
        else:
            self._dq.extendleft(reversed(list(rs)))

    def peek(self) -> Request:
        return self._heap[0] if self.policy == "priority" else self._dq[0]

    def pop(self) -> Request:
        return heapq.heappop(self._heap) if self.policy == "priority" else self._dq.popleft()

    def remove(self, r: Request) -> None:
        if self.policy == "priority":
            self._heap.remove(r)
            heapq.heapify(self._heap)
        else:
            self._dq.remove(r)

    def __len__(self) -> int:
        return len(self._heap) if self.policy == "priority" else len(self._dq)

    def __bool__(self) -> bool:
        return len(self) > 0

    def __iter__(self):
        return iter(sorted(self._heap) if self.policy == "priority" else self._dq)


def check_stop(request: Request, max_model_len: int) -> bool:
    """min_tokens gate → EOS → stop ids → length (reference: v1/core/sched/utils.py)."""
    sp = request.sampling_params
    if sp is not None and request.num_output_tokens >= sp.min_tokens:
        last = request.output_token_ids[-1]
        if not sp.ignore_eos and request.eos_token_id is not None and last == request.eos_token_id:
            request.status = RequestStatus.FINISHED_STOPPED
            return True
        if last in sp.all_stop_token_ids:
            request.status = RequestStatus.FINISHED_STOPPED
            request.stop_reason = last
            return True
    if request.num_tokens >= max_model_len or request.num_output_tokens >= request.max_tokens:
        request.status = RequestStatus.FINISHED_LENGTH_CAPPED
        return True
    if sp is not None and sp.repetition_detection is not None and sp.repetition_detection.hit(request.output_token_ids):
        request.status = RequestStatus.FINISHED_STOPPED
        request.stop_reason = "repetition"
        return True
    return False


class Scheduler:
    def __init__(self, vllm_config: VllmConfig, num_gpu_blocks: int, num_state_slots: int = 0, log_stats: bool = True) -> None:
        self.cfg = vllm_config
        sc, cc = vllm_config.scheduler_config, vllm_config.cache_config
        self.max_num_scheduled_tokens = sc.max_num_batched_tokens
        self.max_num_running_reqs = sc.max_num_seqs
        self.max_model_len = vllm_config.model_config.max_model_len
        self.block_size = cc.block_size
        self.policy = sc.policy
        spec = vllm_config.speculative_config
        mc = vllm_config.model_config
        self.num_spec_tokens = spec.num_speculative_tokens if spec.enabled else 0
        self.num_lookahead_tokens = self.num_spec_tokens if spec.method in ("mtp", "eagle", "eagle3", "draft_model") else 0
        self.kv_cache_manager = KVCacheManager(num_gpu_blocks, cc.block_size, self.max_model_len, cc.enable_prefix_caching,
                                               num_state_slots, use_eagle=spec.method in ("mtp", "eagle", "eagle3", "draft_model"),
                                               dcp_world_size=vllm_config.parallel_config.decode_context_parallel_size,
                                               log_stats=log_stats,
                                               sliding_window=(mc.sliding_window if mc.sliding_window and len(mc.sliding_layers) == mc.num_hidden_layers
                                                               and not spec.enabled else 0))
        from onecat_vllm.core.encoder_cache_manager import EncoderCacheManager
        self.max_num_encoder_input_tokens = sc.max_num_encoder_input_tokens
        self.encoder_cache_manager = EncoderCacheManager(sc.encoder_cache_size)
        if cc.kv_transfer_config:
            self.kv_cache_manager.enable_kv_connector(cc.kv_transfer_config)
        elif cc.num_cpu_blocks > 0:
            self.kv_cache_manager.enable_cpu_offload(cc.num_cpu_blocks, cc.kv_offloading_policy)
        self.block_hasher = make_block_hasher(self.kv_cache_manager.block_size, cc.prefix_caching_hash_algo) \
            if self.kv_cache_manager.enable_caching else None
        self.requests: dict[str, Request] = {}
        self.waiting = RequestQueue(self.policy)
        self.running: list[Request] = []
        self.finished_req_ids: set = set()
        self.log_stats = log_stats
        self._num_preemptions = 0
        self._spec_stats = [0, 0, 0]
        self.use_pp = vllm_config.parallel_config.pipeline_parallel_size > 1
        self.async_scheduling = False  # set by the engine core when it keeps a step in flight
        self.max_loras = vllm_config.model_config.max_loras if vllm_config.model_config.enable_lora else 0

    # ------------------------------------------------------------------ admission
    def add_request(self, request: Request | object) -> None:
        if not isinstance(request, Request):
            request = Request.from_engine_core_request(request, self.block_hasher)
        if request.request_id in self.requests:
            raise ValueError(f"duplicate request id {request.request_id}")
        if request.num_prompt_tokens >= self.max_model_len:
            raise ValueError(f"prompt of {request.num_prompt_tokens} tokens does not fit max_model_len={self.max_model_len}")
        if request.num_prompt_tokens == 0:
            raise ValueError("empty prompt")
        self.requests[request.request_id] = request
        self.waiting.add(request)

    def finish_requests(self, request_ids: str | Iterable[str], status: RequestStatus = RequestStatus.FINISHED_ABORTED) -> None:
        """Abort path: called for client disconnects and frontend stop strings."""
        assert RequestStatus.is_finished(status)
        if isinstance(request_ids, str):
            request_ids = [request_ids]
        for rid in list(request_ids):
            r = self.requests.get(rid)
            if r is None or r.is_finished():
                continue
            if r.status == RequestStatus.RUNNING:
                self.running.remove(r)
            else:
                self.waiting.remove(r)
            r.status = status
            self._free_request(r)

    def _try_schedule_encoder_inputs(self, r: Request, num_computed: int, n: int, encoder_budget: int) -> tuple[list[int], int, int]:
        """Which multimodal items of ``r`` must be encoded for the tokens [num_computed, num_computed + n) to run. An item whose
        placeholder range overlaps that window needs its encoder output in the cache: already there (this or another request put it
        there), or scheduled now if the step's encoder budget and the cache have room; otherwise the window is cut just before the
        item. Returns (item indices to encode, tokens to schedule, remaining encoder budget)
        (reference: v1/core/sched/scheduler.py:1936 ``_try_schedule_encoder_inputs``)."""
        todo: list[int] = []
        if not r.mm_features:
            return todo, n, encoder_budget
        pending = 0
        for i, f in enumerate(r.mm_features):
            if f.offset >= num_computed + n:
                break
            if f.offset + f.length <= num_computed:
                continue  # fully consumed already
            if i in r.mm_cached or self.encoder_cache_manager.check_and_update_cache(r, i):
                r.mm_cached.add(i)
                continue
            if self.encoder_cache_manager.can_allocate(r, i, encoder_budget, pending):
                todo.append(i)
                pending += f.length
                encoder_budget -= f.length
                continue
            # no room: run only the tokens before this item (none, if the window starts inside it)
            n = max(f.offset - num_computed, 0)
            break
        return todo, n, encoder_budget

    def _free_request(self, r: Request) -> None:
        assert r.is_finished()
        self.encoder_cache_manager.free(r)
        self.kv_cache_manager.free(r)
        self.finished_req_ids.add(r.request_id)
        del self.requests[r.request_id]

    # ------------------------------------------------------------------ schedule
    def schedule(self) -> SchedulerOutput:
        out = SchedulerOutput()
        budget = self.max_num_scheduled_tokens
        scheduled_running: list[Request] = []
        scheduled_new: list[Request] = []
        scheduled_resumed: list[Request] = []
        new_blocks_of: dict[str, list[int]] = {}
        preempted: list[Request] = []
        sc = self.cfg.scheduler_config
        encoder_budget = self.max_num_encoder_input_tokens

        # 1. running requests
        i = 0
        while i < len(self.running) and budget > 0:
            r = self.running[i]
            n = r.num_tokens_with_spec + r.num_output_placeholders - r.num_computed_tokens
            if r.num_output_placeholders and r.sampling_params is not None and (
                    r.num_output_tokens + r.num_output_placeholders >= r.sampling_params.max_tokens
                    or r.num_tokens + r.num_output_placeholders >= self.max_model_len):
                n = 0  # the token in flight is the request's last: nothing more to compute for it
            if sc.long_prefill_token_threshold > 0:
                n = min(n, sc.long_prefill_token_threshold)
            n = min(n, budget, self.max_model_len - 1 - r.num_computed_tokens)
            enc_todo: list[int] = []
            if n > 0 and r.mm_features:
                enc_todo, n, enc_left = self._try_schedule_encoder_inputs(r, r.num_computed_tokens, n, encoder_budget)
            if n <= 0:
                i += 1
                continue
            while True:
                new_blocks = self.kv_cache_manager.allocate_slots(r, n, num_lookahead_tokens=self.num_lookahead_tokens)
                if new_blocks is not None:
                    break
                victim = max(self.running, key=lambda q: (q.priority, q.arrival_time)) if self.policy == "priority" else self.running[-1]
                vi = self.running.index(victim)
                self.running.pop(vi)
                if vi < i:
                    i -= 1
                if victim in scheduled_running:
                    scheduled_running.remove(victim)
                    budget += out.num_scheduled_tokens.pop(victim.request_id)
                    out.scheduled_spec_decode_tokens.pop(victim.request_id, None)
                    new_blocks_of.pop(victim.request_id, None)
                self._preempt(victim)
                preempted.append(victim)
                if victim is r:
                    new_blocks = None
                    break
            if new_blocks is None:
                break  # r itself was preempted: nothing below it can run either
            scheduled_running.append(r)
            new_blocks_of[r.request_id] = [b.block_id for b in new_blocks]
            out.num_scheduled_tokens[r.request_id] = n
            budget -= n
            if enc_todo:
                encoder_budget = enc_left
                out.scheduled_encoder_inputs[r.request_id] = enc_todo
                for k in enc_todo:
                    self.encoder_cache_manager.allocate(r, k)
                    r.mm_cached.add(k)
            if r.spec_token_ids:
                num_spec = n + r.num_computed_tokens - r.num_tokens
                if num_spec > 0:
                    del r.spec_token_ids[num_spec:]
                    out.scheduled_spec_decode_tokens[r.request_id] = list(r.spec_token_ids)
                else:
                    r.spec_token_ids = []
            i += 1

        # 2. waiting requests (none in a step that preempted)
        if not preempted:
            skipped: list[Request] = []
            while self.waiting and budget > 0 and len(self.running) < self.max_num_running_reqs:
                r = self.waiting.peek()
                if r.lora_request is not None and self.max_loras > 0:
                    # a step may not touch more adapters than the workers hold (reference: scheduler.py ``scheduled_loras``)
                    live = {x.lora_request.lora_int_id for x in self.running if x.lora_request is not None}
                    if r.lora_request.lora_int_id not in live and len(live) >= self.max_loras:
                        self.waiting.pop()
                        skipped.append(r)
                        continue
                if r.num_computed_tokens == 0:
                    hit_blocks, num_hit = self.kv_cache_manager.get_computed_blocks(r)
                else:
                    hit_blocks, num_hit = [], 0
                n = r.num_tokens - (r.num_computed_tokens + num_hit)
                if sc.long_prefill_token_threshold > 0:
                    n = min(n, sc.long_prefill_token_threshold)
                if not sc.enable_chunked_prefill and n > budget:
                    break
                n = min(n, budget)
                assert n > 0
                enc_todo = []
                if r.mm_features:
                    enc_todo, n, enc_left = self._try_schedule_encoder_inputs(r, r.num_computed_tokens + num_hit, n, encoder_budget)
                    if n <= 0:
                        break  # the encoder budget or cache is exhausted for this step
                new_blocks = self.kv_cache_manager.allocate_slots(r, n, num_hit, hit_blocks, self.num_lookahead_tokens)
                if new_blocks is None:
                    break
                if enc_todo:
                    encoder_budget = enc_left
                    out.scheduled_encoder_inputs[r.request_id] = enc_todo
                    for k in enc_todo:
                        self.encoder_cache_manager.allocate(r, k)
                        r.mm_cached.add(k)
                self.waiting.pop()
                self.running.append(r)
                if r.status == RequestStatus.PREEMPTED:
                    scheduled_resumed.append(r)
                else:
                    scheduled_new.append(r)
                    if r.first_scheduled_time is None:
                        r.first_scheduled_time = time.time()
                r.status = RequestStatus.RUNNING
                r.num_computed_tokens += num_hit
                if r.num_cached_tokens < 0:
                    r.num_cached_tokens = num_hit
                new_blocks_of[r.request_id] = self.kv_cache_manager.get_block_ids(r.request_id)
                out.num_scheduled_tokens[r.request_id] = n
                budget -= n
            if skipped:
                self.waiting.prepend(skipped)

        out.total_num_scheduled_tokens = self.max_num_scheduled_tokens - budget
        assert out.total_num_scheduled_tokens == sum(out.num_scheduled_tokens.values())
        km = self.kv_cache_manager
        out.scheduled_new_reqs = [
            NewRequestData(r.request_id, r.prompt_token_ids, r.sampling_params, new_blocks_of[r.request_id],
                           r.num_computed_tokens, km.get_state_slot(r.request_id), r.eos_token_id, r.pooling_params, r.lora_request, r.prompt_embeds,
                           r.mm_features or None)
            for r in scheduled_new]
        cached = CachedRequestData()
        for r in scheduled_resumed + scheduled_running:
            resumed = r in scheduled_resumed
            cached.req_ids.append(r.request_id)
            cached.resumed_from_preemption.append(resumed)
            if resumed:
                cached.new_token_ids.append(list(r.all_token_ids))
            elif self.use_pp:  # stages that do not sample learn the tokens from here (reference: scheduler.py ``use_pp`` branch)
                cached.new_token_ids.append(list(r.all_token_ids[r.num_computed_tokens:]))
            else:
                cached.new_token_ids.append([])
            cached.new_block_ids.append(new_blocks_of[r.request_id])
            cached.num_computed_tokens.append(r.num_computed_tokens)
            cached.state_slots.append(km.get_state_slot(r.request_id))
        out.scheduled_cached_reqs = cached
        out.finished_req_ids, self.finished_req_ids = self.finished_req_ids, set()
        out.preempted_req_ids = {r.request_id for r in preempted}
        out.free_encoder_mm_hashes = self.encoder_cache_manager.get_freed_mm_hashes()
        if self.running:
            out.num_common_prefix_blocks = km.get_num_common_prefix_blocks(self.running[0].request_id, len(self.running))
        if self.kv_cache_manager.offload is not None:
            out.kv_swap_out, out.kv_swap_in = self.kv_cache_manager.offload.take_ops()
        # advance: the runner computes these tokens in this step
        for rid, n in out.num_scheduled_tokens.items():
            r = self.requests[rid]
            r.num_computed_tokens += n
            if self.async_scheduling and r.num_computed_tokens >= r.num_tokens + r.num_output_placeholders:
                r.num_output_placeholders += 1   # this step samples a token the next schedule() will not have seen yet
        return out

    def may_preempt(self) -> bool:
        """Whether the next schedule() could run out of KV blocks (and so preempt a request whose step is still in flight)."""
        need = len(self.running) * (1 + self.num_lookahead_tokens // max(self.block_size, 1) + 1) + 8
        return self.kv_cache_manager.block_pool.get_num_free_blocks() < need

    def all_plain(self) -> bool:
        """Every live request samples from the untouched logits and reports nothing but its tokens: the condition under which a
        step may be scheduled before the previous step's tokens are known."""
        for q in (self.running, self.waiting):
            for r in q:
                sp = r.sampling_params
                if sp is None or r.pooling_params is not None or r.spec_token_ids:
                    return False
                if (sp.logprobs is not None or sp.prompt_logprobs is not None or sp.presence_penalty or sp.frequency_penalty
                        or sp.repetition_penalty != 1.0 or sp.min_tokens or sp.logit_bias or sp.allowed_token_ids or sp.bad_words
                        or getattr(sp, "structured_outputs", None) is not None or getattr(sp, "thinking_token_budget", None) is not None
                        or getattr(sp, "repetition_detection", None) is not None):
                    return False
        return True

    def _preempt(self, r: Request) -> None:
        self.kv_cache_manager.free(r)
        self.encoder_cache_manager.free(r)  # the recomputation will ask for the encoder outputs again
        r.mm_cached.clear()
        r.status = RequestStatus.PREEMPTED
        r.num_computed_tokens = 0
        r.num_output_placeholders = 0
        r.spec_token_ids = []
        r.num_preemptions += 1
        self._num_preemptions += 1
        self.waiting.prepend([r])

    # ------------------------------------------------------------------ results
    def _release_consumed_encoder_inputs(self, sched_out: SchedulerOutput) -> None:
        """An item's encoder output is needed until the last of its placeholder positions has been computed."""
        for rid in sched_out.num_scheduled_tokens:
            r = self.requests.get(rid)
            if r is None or not r.mm_cached:
                continue
            for i in [i for i in r.mm_cached if r.mm_features[i].offset + r.mm_features[i].length <= r.num_computed_tokens]:
                self.encoder_cache_manager.free_encoder_input(r, i)
                r.mm_cached.discard(i)

    def update_from_output(self, sched_out: SchedulerOutput, mro: ModelRunnerOutput) -> dict[int, EngineCoreOutputs]:
        self._release_consumed_encoder_inputs(sched_out)
        idx = {rid: i for i, rid in enumerate(mro.req_ids)}
        outputs: dict[int, list[EngineCoreOutput]] = {}
        stopped: list[Request] = []
        for rid, n_sched in sched_out.num_scheduled_tokens.items():
            r = self.requests.get(rid)
            if r is None or r.is_finished():
                continue  # aborted while the step was in flight
            i = idx.get(rid)
            generated = mro.sampled_token_ids[i] if i is not None and mro.sampled_token_ids else []
            drafts = sched_out.scheduled_spec_decode_tokens.get(rid)
            if drafts:
                # rejected drafts were counted as computed: take them back
                n_rej = len(drafts) + 1 - len(generated) if generated else len(drafts)
                r.num_computed_tokens -= n_rej
                self._spec_stats[0] += 1
                self._spec_stats[1] += len(drafts)
                self._spec_stats[2] += max(len(generated) - 1, 0)
            new_ids: list[int] = []
            stop = False
            for t in generated:
                if r.num_output_placeholders > 0:
                    r.num_output_placeholders -= 1
                r.append_output_token_ids(t)
                new_ids.append(t)
                if check_stop(r, self.max_model_len):
                    stop = True
                    break
            if new_ids and len(new_ids) < len(generated):
                # tokens after the stop point were computed but are dropped
                r.num_computed_tokens = min(r.num_computed_tokens, r.num_tokens)
            if mro.spec_token_ids is not None and i is not None and not stop and r.spec_decode_ok:
                r.spec_token_ids = list(mro.spec_token_ids[i])[: self.num_spec_tokens] if r.num_computed_tokens >= r.num_tokens - 1 else []
            lp = None
            if mro.logprobs is not None and i is not None and mro.logprobs[i] is not None and new_ids:
                l = mro.logprobs[i]
                lp = [(l.token_ids[k], l.logprobs[k], l.ranks[k]) for k in range(len(new_ids))]
            plp = mro.prompt_logprobs.get(rid) if mro.prompt_logprobs else None
            pooled = mro.pooler_output[i] if mro.pooler_output is not None and i is not None else None
            if new_ids or plp is not None or stop:
                outputs.setdefault(r.client_index, []).append(EngineCoreOutput(
                    rid, new_ids, r.get_finished_reason() if stop else None, r.stop_reason if stop else None, lp, plp,
                    max(r.num_cached_tokens, 0), pooling_output=pooled))
            if stop:
                stopped.append(r)
        for r in stopped:
            if r in self.running:
                self.running.remove(r)
            else:
                self.waiting.remove(r)   # preempted while its last step was in flight
            self._free_request(r)
        stats = self.make_stats(sched_out, mro)
        result = {c: EngineCoreOutputs(outs, stats) for c, outs in outputs.items()}
        if not result and stats is not None:
            result[0] = EngineCoreOutputs([], stats)
        return result

    def update_draft_token_ids(self, req_ids: list[str], drafts: list[list[int]]) -> None:
        for rid, d in zip(req_ids, drafts):
            r = self.requests.get(rid)
            if r is not None and not r.is_finished() and r.spec_decode_ok:
                r.spec_token_ids = list(d)

    # ------------------------------------------------------------------ introspection
    def get_num_unfinished_requests(self) -> int:
        return len(self.waiting) + len(self.running)

    def has_unfinished_requests(self) -> bool:
        return self.get_num_unfinished_requests() > 0

    def has_finished_requests(self) -> bool:
        return bool(self.finished_req_ids)

    def has_requests(self) -> bool:
        return self.has_unfinished_requests() or self.has_finished_requests()

    def reset_prefix_cache(self) -> bool:
        return self.kv_cache_manager.reset_prefix_cache()

    def make_stats(self, sched_out: Optional[SchedulerOutput] = None, mro: Optional[ModelRunnerOutput] = None) -> Optional[SchedulerStats]:
        if not self.log_stats:
            return None
        pc = self.kv_cache_manager.make_prefix_cache_stats()
        s = SchedulerStats(len(self.running), len(self.waiting), self.kv_cache_manager.usage, pc.queries if pc else 0,
                           pc.hits if pc else 0, self._num_preemptions,
                           sched_out.total_num_scheduled_tokens if sched_out else 0, *self._spec_stats,
                           step_device_ms=mro.device_time_ms if mro else 0.0)
        self._num_preemptions = 0
        self._spec_stats = [0, 0, 0]
        return s
