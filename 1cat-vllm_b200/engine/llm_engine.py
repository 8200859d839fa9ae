"""Synchronous engine used by the offline API (reference: vllm/v1/engine/llm_engine.py:47; ``add_request`` :209,
``step`` :287). The engine core runs in-process (``InprocClient``) or in its own process behind ZMQ
(``ONECAT_ENABLE_MULTIPROCESSING=1``)."""
from __future__ import annotations

import time
from typing import Optional

from onecat_vllm import envs
from onecat_vllm.config import EngineArgs, VllmConfig
from onecat_vllm.engine.processors import InputProcessor, OutputProcessor
from onecat_vllm.engine.tokenizer import get_tokenizer
from onecat_vllm.inputs import PromptType
from onecat_vllm.outputs import RequestOutput
from onecat_vllm.sampling_params import RequestOutputKind, SamplingParams


class LLMEngine:
    def __init__(self, vllm_config: VllmConfig, log_stats: bool = False, multiprocess: Optional[bool] = None):
        self.cfg = vllm_config
        self.tokenizer = get_tokenizer(vllm_config.model_config.tokenizer)
        self.input_processor = InputProcessor(vllm_config, self.tokenizer)
        self.output_processor = OutputProcessor(self.tokenizer, log_stats)
        mp = envs.ONECAT_ENABLE_MULTIPROCESSING if multiprocess is None else multiprocess
        from onecat_vllm.engine.core_client import make_client
        self.engine_core = make_client(vllm_config, multiprocess=mp, asyncio_mode=False, log_stats=log_stats)
        self.log_stats = log_stats
        self.stat_loggers = []
        if log_stats:
            from onecat_vllm.metrics.loggers import make_stat_loggers
            self.stat_loggers = make_stat_loggers(vllm_config)

    @classmethod
    def from_engine_args(cls, args: EngineArgs, **kw) -> "LLMEngine":
        return cls(args.create_engine_config(), log_stats=not args.disable_log_stats, **kw)

    def add_request(self, request_id: str, prompt: PromptType, params: SamplingParams, arrival_time: Optional[float] = None,
                    priority: int = 0, lora_request=None) -> None:
        req, text = self.input_processor.process(request_id, prompt, params, arrival_time, priority, lora_request)
        n = getattr(params, "n", 1)
        if n == 1:
            self.output_processor.add_request(req, text)
            self.engine_core.add_request(req)
            return
        for i in range(n):  # fan out: child requests with distinct seeds (reference: parallel_sampling.py)
            child = type(req)(**{**req.__dict__})
            child.request_id = f"{i}_{request_id}"
            sp = req.sampling_params.clone()
            sp.n = n
            if sp.seed is not None:
                sp.seed += i
            child.sampling_params = sp
            self.output_processor.add_request(child, text, parent_id=request_id, index=i)
            sp2 = sp.clone()
            sp2.n = 1
            child.sampling_params = sp2
            self.engine_core.add_request(child)

    def abort_request(self, request_ids: list[str]) -> None:
        ids = self.output_processor.abort(request_ids)
        self.engine_core.abort_requests(ids)

    def step(self) -> list[RequestOutput]:
        outs = self.engine_core.get_output()
        now = time.time()
        self.last_scheduler_stats = outs.scheduler_stats
        results, to_abort = self.output_processor.process_outputs(outs.outputs, now)
        if to_abort:
            self.engine_core.abort_requests(to_abort)
        if self.stat_loggers and outs.scheduler_stats is not None:
            for l in self.stat_loggers:
                l.record(outs.scheduler_stats, outs.outputs, self.output_processor.finished_stats)
            self.output_processor.finished_stats.clear()
        return results

    def has_unfinished_requests(self) -> bool:
        return self.output_processor.has_unfinished()

    def get_num_unfinished_requests(self) -> int:
        return len(self.output_processor.states)

    def reset_prefix_cache(self) -> bool:
        return self.engine_core.call_utility("reset_prefix_cache")

    def sleep(self, level: int = 1) -> None:
        self.engine_core.call_utility("sleep", level)

    def wake_up(self, tags=None) -> None:
        self.engine_core.call_utility("wake_up", tags)

    def add_lora(self, lora_request) -> bool:
        return self.engine_core.call_utility("add_lora", lora_request.to_dict())

    def remove_lora(self, lora_id: int) -> bool:
        return self.engine_core.call_utility("remove_lora", lora_id)

    def list_loras(self) -> list:
        return self.engine_core.call_utility("list_loras")

    def collective_rpc(self, method, args=(), kwargs=None):
        return self.engine_core.call_utility("collective_rpc", method, args, kwargs)

    def get_metrics(self) -> dict:
        from onecat_vllm.metrics.loggers import snapshot
        return snapshot(self.stat_loggers)

    def shutdown(self) -> None:
        if getattr(self, "engine_core", None) is not None:
            self.engine_core.shutdown()
            self.engine_core = None

    def __del__(self):
        try:
            self.shutdown()
        except Exception:
            pass
