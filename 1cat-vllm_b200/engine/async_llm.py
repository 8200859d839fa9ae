"""Asyncio engine for the API server (reference: vllm/v1/engine/async_llm.py:70 class, :280 ``add_request``, :524
``generate``, :637 output handler). One background task pulls engine-core outputs, runs the output processor and feeds
per-request queues; ``generate`` is an async generator over ``RequestOutput`` deltas. Stop strings found by the
detokenizer abort the request in the core; a dead core surfaces as ``EngineDeadError`` in every pending stream."""
from __future__ import annotations

import asyncio
import time
from typing import AsyncGenerator, Optional

from onecat_vllm.config import EngineArgs, VllmConfig
from onecat_vllm.engine.core import EngineDeadError
from onecat_vllm.engine.processors import InputProcessor, OutputProcessor
from onecat_vllm.engine.tokenizer import get_tokenizer
from onecat_vllm.inputs import PromptType
from onecat_vllm.logger import init_logger
from onecat_vllm.outputs import RequestOutput
from onecat_vllm.sampling_params import RequestOutputKind, SamplingParams

log = init_logger(__name__)


class AsyncLLM:
    def __init__(self, vllm_config: VllmConfig, log_stats: bool = True):
        self.cfg = vllm_config
        self.tokenizer = get_tokenizer(vllm_config.model_config.tokenizer)
        self.input_processor = InputProcessor(vllm_config, self.tokenizer)
        self.output_processor = OutputProcessor(self.tokenizer, log_stats)
        from onecat_vllm.engine.core_proc import AsyncMPClient
        self.engine_core = AsyncMPClient(vllm_config, log_stats)
        self.stat_loggers = []
        if log_stats:
            from onecat_vllm.metrics.loggers import make_stat_loggers
            self.stat_loggers = make_stat_loggers(vllm_config, prometheus=True)
        self._handler: Optional[asyncio.Task] = None
        self.errored: Optional[BaseException] = None
        self.last_scheduler_stats = None

    @classmethod
    def from_engine_args(cls, args: EngineArgs) -> "AsyncLLM":
        return cls(args.create_engine_config(), log_stats=not args.disable_log_stats)

    @property
    def is_running(self) -> bool:
        return self.errored is None and not self.engine_core.dead

    def _ensure_handler(self) -> None:
        if self._handler is None or self._handler.done():
            self._handler = asyncio.get_running_loop().create_task(self._output_loop())

    async def _utility(self, method: str, *args):
        """Utility replies arrive on the output socket, which only the output task reads: start it before the first call."""
        self._ensure_handler()
        return await self.engine_core.call_utility_async(method, *args)

    async def _output_loop(self) -> None:
        try:
            while True:
                outs = await self.engine_core.get_output_async()
                self.last_scheduler_stats = outs.scheduler_stats
                # process in chunks so one huge batch does not starve the event loop (reference: async_llm.py:656-703)
                items = outs.outputs
                for i in range(0, max(len(items), 1), 128):
                    _, to_abort = self.output_processor.process_outputs(items[i:i + 128], time.time())
                    if to_abort:
                        await self.engine_core.abort_requests_async(to_abort)
                    if i + 128 < len(items):
                        await asyncio.sleep(0)
                if self.stat_loggers and outs.scheduler_stats is not None:
                    for l in self.stat_loggers:
                        l.record(outs.scheduler_stats, outs.outputs, self.output_processor.finished_stats)
                    self.output_processor.finished_stats.clear()
        except asyncio.CancelledError:
            raise
        except BaseException as e:  # engine death: wake every waiting stream
            self.errored = e
            for st in list(self.output_processor.states.values()):
                if st.queue is not None:
                    st.queue.put_nowait(e)
            log.error(f"output handler stopped: {e!r}")

    async def add_request(self, request_id: str, prompt: PromptType, params: SamplingParams, priority: int = 0, lora_request=None) -> asyncio.Queue:
        if self.errored is not None:
            raise EngineDeadError(str(self.errored))
        self._ensure_handler()
        req, text = self.input_processor.process(request_id, prompt, params, None, priority, lora_request)
        q: asyncio.Queue = asyncio.Queue()
        n = getattr(params, "n", 1)
        if n == 1:
            self.output_processor.add_request(req, text, queue=q)
            await self.engine_core.add_request_async(req)
            return q
        for i in range(n):
            child = type(req)(**{**req.__dict__})
            child.request_id = f"{i}_{request_id}"
            sp = req.sampling_params.clone()
            if sp.seed is not None:
                sp.seed += i
            child.sampling_params = sp
            self.output_processor.add_request(child, text, parent_id=request_id, index=i, queue=q)
            sp2 = sp.clone()
            sp2.n = 1
            child.sampling_params = sp2
            await self.engine_core.add_request_async(child)
        return q

    async def generate(self, prompt: PromptType, sampling_params: SamplingParams, request_id: str, priority: int = 0,
                       lora_request=None) -> AsyncGenerator[RequestOutput, None]:
        q = await self.add_request(request_id, prompt, sampling_params, priority, lora_request)
        finished_children = 0
        try:
            while True:
                out = await q.get()
                if isinstance(out, BaseException):
                    raise EngineDeadError(str(out))
                yield out
                if out.finished:
                    break
        except (asyncio.CancelledError, GeneratorExit):
            await self.abort(request_id)
            raise

    async def encode(self, prompt: PromptType, pooling_params, request_id: str, priority: int = 0):
        """Run one pooling request to completion and return its ``PoolingRequestOutput``."""
        q = await self.add_request(request_id, prompt, pooling_params, priority)
        try:
            out = await q.get()
        except asyncio.CancelledError:
            await self.abort(request_id)
            raise
        if isinstance(out, BaseException):
            raise EngineDeadError(str(out))
        return out

    async def abort(self, request_id: str) -> None:
        ids = self.output_processor.abort([request_id])
        await self.engine_core.abort_requests_async(ids)

    async def check_health(self) -> None:
        if not self.is_running:
            raise EngineDeadError("engine is not running")

    async def reset_prefix_cache(self) -> bool:
        return await self._utility("reset_prefix_cache")

    async def reset_mm_cache(self) -> int:
        return await self._utility("reset_encoder_cache")

    async def sleep(self, level: int = 1) -> None:
        await self._utility("sleep", level)

    async def wake_up(self) -> None:
        await self._utility("wake_up")

    async def pause_generation(self) -> None:
        await self._utility("pause_generation")

    async def resume_generation(self) -> None:
        await self._utility("resume_generation")

    async def is_paused(self) -> bool:
        return bool(await self._utility("is_paused"))

    async def profile(self, start: bool) -> None:
        await self._utility("profile", start)

    async def add_lora(self, lora_request) -> bool:
        return await self._utility("add_lora", lora_request.to_dict())

    async def remove_lora(self, lora_id: int) -> bool:
        return await self._utility("remove_lora", lora_id)

    async def collective_rpc(self, method: str, args=(), kwargs=None):
        return await self._utility("collective_rpc", method, list(args), kwargs)

    def shutdown(self) -> None:
        if self._handler is not None:
            self._handler.cancel()
        self.engine_core.shutdown()
