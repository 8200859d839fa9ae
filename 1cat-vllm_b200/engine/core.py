"""Engine core: owns the scheduler and the executor; one ``step`` = schedule → execute → update
(reference: vllm/v1/engine/core.py:94 ``EngineCore``, :241 ``_initialize_kv_caches``, :445 ``step``, :786-804 utility
calls; the process wrapper with ZMQ sockets lives in ``onecat_vllm.engine.core_proc``)."""
from __future__ import annotations

import time
from typing import Optional

from onecat_vllm.config import VllmConfig
from onecat_vllm.core.scheduler import Scheduler
from onecat_vllm.executor.uniproc import Executor
from onecat_vllm.logger import init_logger
from onecat_vllm.request import EngineCoreOutputs, EngineCoreRequest, Request, RequestStatus

log = init_logger(__name__)


class EngineDeadError(RuntimeError):
    """Raised to API callers once the engine core or a worker has failed (reference: v1/engine/exceptions.py:9)."""


class CollectiveTimeout(RuntimeError):
    """A bounded device-side wait on a peer expired; the step's outputs are not trustworthy."""


class EngineCore:
    def __init__(self, vllm_config: VllmConfig, executor_class=None, log_stats: bool = True):
        self.cfg = vllm_config
        from onecat_vllm.utils.plugins import load_general_plugins
        load_general_plugins()
        executor_class = executor_class or Executor.get_class(vllm_config)
        t0 = time.time()
        self.executor = executor_class(vllm_config)
        self._failed = False
        self.executor.register_failure_callback(self._on_executor_failure)
        num_blocks, num_slots = self.executor.initialize_kv_cache()
        self.scheduler = Scheduler(vllm_config, num_blocks, num_slots, log_stats)
        self.step_count = 0
        self.paused = False
        # async scheduling: one step may be in flight on the device while the next one is scheduled and staged. Not with drafts
        # (their acceptance decides what the next step computes) nor with pipeline stages (tokens reach them through the scheduler).
        pc, sc = vllm_config.parallel_config, vllm_config.scheduler_config
        from onecat_vllm import envs
        want = bool(sc.async_scheduling) if envs.ONECAT_ASYNC_SCHEDULING == "" else envs.ONECAT_ASYNC_SCHEDULING == "1"
        self.async_scheduling = want and pc.pipeline_parallel_size == 1 and \
            not (vllm_config.speculative_config and vllm_config.speculative_config.method) and \
            not vllm_config.model_config.logits_processors   # user processors may read the tokens produced so far
        self.scheduler.async_scheduling = self.async_scheduling
        self._stalled = 0      # consecutive idle schedules that placed nothing (see _unschedulable)
        self._inflight = None  # SchedulerOutput of the launched, uncollected step
        self._overlap = True   # set_overlap(False): finish what is in flight without launching behind it (drains the pipeline)
        self._structured = None  # built on the first request that asks for a grammar
        from onecat_vllm.core.kv_events import make_publisher
        self._kv_events = make_publisher(vllm_config.cache_config.kv_events_config)
        log.info_once(f"engine core ready: {num_blocks} KV blocks, {num_slots} state slots, init {time.time() - t0:.1f}s")

    def _on_executor_failure(self) -> None:
        self._failed = True

    # ---- requests
    def add_request(self, req: EngineCoreRequest | Request) -> None:
        sp = req.sampling_params
        if sp is not None and sp.structured_outputs is not None and sp.structured_outputs.kind() != "none":
            self.structured_output_manager().grammar_init(req.request_id, sp.structured_outputs)
        self.scheduler.add_request(req)

    def structured_output_manager(self):
        if self._structured is None:
            from onecat_vllm.engine.tokenizer import get_tokenizer
            from onecat_vllm.structured import StructuredOutputManager
            mc = self.cfg.model_config
            tok = get_tokenizer(mc.tokenizer)
            self._structured = StructuredOutputManager(tok, mc.vocab_size, backend=self.cfg.structured_outputs_backend)
        return self._structured

    def abort_requests(self, request_ids: list[str]) -> None:
        if self._structured is not None:
            for rid in request_ids:
                self._structured.free(rid)
        self.scheduler.finish_requests(request_ids, RequestStatus.FINISHED_ABORTED)

    # ---- the step
    def step(self) -> tuple[dict[int, EngineCoreOutputs], bool]:
        """Returns (outputs per client, whether a model step ran)."""
        if self._failed:
            raise EngineDeadError("a worker failed")
        if self.async_scheduling:
            return self._step_async()
        if not self.scheduler.has_requests() or self.paused:
            return {}, False
        so = self.scheduler.schedule()
        stuck = self._unschedulable(so)
        if stuck is not None:
            return stuck, False
        if self._structured is not None and self._structured.grammars:
            so.grammar_bitmask, so.structured_rows = self._structured.grammar_bitmask(list(so.num_scheduled_tokens))
        mro = self._guarded(so, lambda: self.executor.execute_model(so))
        return self._finish_step(so, mro)

    def _unschedulable(self, so) -> Optional[dict]:
        """An idle engine (nothing running, nothing in flight, no block copies pending) that schedules no token of its first waiting
        request, sixteen times in a row, will never schedule it: the request asks for more than the engine can ever give (an encoder
        input larger than the encoder cache, more blocks than the pool holds). It is finished with an error instead of spinning."""
        sch = self.scheduler
        idle = (so.total_num_scheduled_tokens == 0 and not sch.running and sch.waiting and self._inflight is None and not so.kv_swap_in
                and not so.kv_swap_out)
        if not idle:
            self._stalled = 0
            return None
        self._stalled += 1
        if self._stalled < 16:
            return None
        self._stalled = 0
        r = sch.waiting.peek()
        log.error(f"request {r.request_id} can never be scheduled on this engine ({r.num_tokens} tokens, {len(r.mm_features or ())} multimodal items): "
                  "finished with an error")
        from onecat_vllm.request import EngineCoreOutput, FinishReason
        out = EngineCoreOutput(r.request_id, [], FinishReason.ERROR if hasattr(FinishReason, "ERROR") else FinishReason.ABORT,
                               "the request does not fit this engine (KV blocks or encoder cache)")
        sch.finish_requests(r.request_id, RequestStatus.FINISHED_ERROR)
        if self._structured is not None:
            self._structured.free(r.request_id)
        return {r.client_index: EngineCoreOutputs([out])}

    def _guarded(self, so, call):
        try:
            mro = call()
        except Exception as e:
            self._failed = True
            log.error(f"model step failed; scheduler state: running={len(self.scheduler.running)} waiting={len(self.scheduler.waiting)} "
                      f"tokens={so.total_num_scheduled_tokens}: {e!r}")
            raise
        if mro is not None and mro.status != 0:
            self._failed = True
            raise CollectiveTimeout(f"device wait expired (status {mro.status:#x})")
        return mro

    def _step_async(self) -> tuple[dict[int, EngineCoreOutputs], bool]:
        """One step stays in flight: while the device runs step n, step n+1 is scheduled (counting the token each sampling request
        of step n will produce as a placeholder), staged and enqueued behind it; only then is step n's result read and applied.
        Falls back to the plain schedule-run-update order whenever a request needs its tokens on the host between steps, a grammar
        is active or the KV cache is close to full (a preemption must not hit a request whose step is in flight)."""
        sch = self.scheduler
        overlap_ok = self._overlap and not self.paused and not (self._structured is not None and self._structured.grammars) and sch.all_plain() and \
            not sch.may_preempt()
        if self._inflight is None:
            if not sch.has_requests() or self.paused:
                return {}, False
            so = sch.schedule()
            stuck = self._unschedulable(so)
            if stuck is not None:
                return stuck, False
            if not overlap_ok or so.total_num_scheduled_tokens == 0:
                if self._structured is not None and self._structured.grammars:
                    so.grammar_bitmask, so.structured_rows = self._structured.grammar_bitmask(list(so.num_scheduled_tokens))
                mro = self._guarded(so, lambda: self.executor.execute_model(so))
                return self._finish_step(so, mro)
            self._guarded(so, lambda: self.executor.launch_model(so))
            self._inflight = so
        nxt = None
        if overlap_ok and sch.has_unfinished_requests():
            nxt = sch.schedule()
            self._guarded(nxt, lambda: self.executor.launch_model(nxt))
        cur, self._inflight = self._inflight, nxt
        mro = self._guarded(cur, lambda: self.executor.collect_model())
        return self._finish_step(cur, mro)

    def set_overlap(self, on: bool) -> None:
        """With ``False`` the next steps only finish work that is in flight (or run in the plain order when nothing is): a caller
        that needs every launched step accounted for, e.g. to time an exact number of steps, turns overlap off for the last one."""
        self._overlap = bool(on)

    def _finish_step(self, so, mro) -> tuple[dict[int, EngineCoreOutputs], bool]:
        outs = self.scheduler.update_from_output(so, mro)
        ev = self.scheduler.kv_cache_manager.block_pool.take_events()  # also bounds the list when nobody listens
        if self._kv_events is not None:
            self._kv_events.publish(ev)
        if self._structured is not None and self._structured.grammars:
            for eco in outs.values():
                for o in eco.outputs:
                    if self._structured.has(o.request_id):
                        self._structured.accept_tokens(o.request_id, o.new_token_ids)
                        if o.finished:
                            self._structured.free(o.request_id)
        self.step_count += 1
        return outs, so.total_num_scheduled_tokens > 0

    # ---- utility calls
    def has_unfinished_requests(self) -> bool:
        return self.scheduler.has_unfinished_requests()

    def reset_prefix_cache(self) -> bool:
        return self.scheduler.reset_prefix_cache()

    def reset_encoder_cache(self) -> int:
        return self.scheduler.encoder_cache_manager.reset()

    def sleep(self, level: int = 1) -> None:
        self.paused = True
        self.executor.collective_rpc("sleep", (level,))
        self.scheduler.reset_prefix_cache()

    def wake_up(self, tags=None) -> None:
        """``tags`` (sleep mode only): wake just these pools, e.g. ``["weights"]`` to push new weights before the KV cache returns."""
        self.executor.collective_rpc("wake_up", (tags,))
        if tags is None or "kv_cache" in tags:
            self.paused = False

    def pause_generation(self) -> None:
        """Stop scheduling steps; queued and running requests keep their state and KV (reference: v1/engine/core.py pause)."""
        self.paused = True

    def resume_generation(self) -> None:
        self.paused = False

    def is_paused(self) -> bool:
        return self.paused

    def profile(self, start: bool = True) -> None:
        self.executor.collective_rpc("profile", (start,))

    def save_sharded_state(self, path: str) -> None:
        self.executor.collective_rpc("save_sharded_state", (path,))

    def add_lora(self, req) -> bool:
        return all(self.executor.collective_rpc("add_lora", (req,)))

    def remove_lora(self, lora_id: int) -> bool:
        return all(self.executor.collective_rpc("remove_lora", (lora_id,)))

    def list_loras(self) -> list:
        return self.executor.collective_rpc("list_loras")[0]

    def collective_rpc(self, method, args=(), kwargs=None):
        return self.executor.collective_rpc(method, args, kwargs)

    def shutdown(self) -> None:
        if getattr(self, "executor", None) is not None:
            self.executor.shutdown()
            self.executor = None
