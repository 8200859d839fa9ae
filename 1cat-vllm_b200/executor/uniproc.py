"""Executors fan engine-core calls out to workers (reference: vllm/v1/executor/abstract.py:37 ``Executor``,
uniproc_executor.py:46,155). ``UniProcExecutor`` drives one in-process worker; ``ExternalLauncherExecutor`` is the
torchrun form: every rank runs the whole engine deterministically and owns one worker."""
from __future__ import annotations

import os
from typing import Any, Callable, Optional

from onecat_vllm.config import VllmConfig
from onecat_vllm.core.kv_cache_utils import get_kv_cache_config
from onecat_vllm.worker.worker import Worker


class Executor:
    uses_processes = False

    @staticmethod
    def get_class(cfg: VllmConfig):
        b = cfg.parallel_config.distributed_executor_backend
        ws = cfg.parallel_config.world_size
        if b == "external_launcher" or (b is None and ws > 1 and "RANK" in os.environ and int(os.environ.get("WORLD_SIZE", 1)) == ws):
            return ExternalLauncherExecutor
        if b == "mp" or (b is None and ws > 1):
            from onecat_vllm.executor.multiproc import MultiprocExecutor
            return MultiprocExecutor
        return UniProcExecutor

    def __init__(self, cfg: VllmConfig):
        self.cfg = cfg
        self.is_failed = False
        self.failure_callback: Optional[Callable] = None
        self._init_executor()

    def _init_executor(self) -> None:
        raise NotImplementedError

    def collective_rpc(self, method: str, args: tuple = (), kwargs: Optional[dict] = None, timeout: Optional[float] = None) -> list:
        raise NotImplementedError

    def register_failure_callback(self, cb: Callable) -> None:
        if self.is_failed:
            cb()
        else:
            self.failure_callback = cb

    # ---- engine-facing API
    def initialize_kv_cache(self) -> tuple[int, int]:
        """Profile → size → allocate → warm up. Returns (num_blocks, num_state_slots)."""
        cfg = self.cfg
        all_specs = self.collective_rpc("get_kv_cache_specs")
        all_avail = self.collective_rpc("determine_available_memory")
        # every rank sizes its own layers (pipeline stages own different ones); the pool takes the smallest block count
        kvcs = [get_kv_cache_config(s, a, cfg.cache_config.block_size, cfg.scheduler_config.max_num_seqs,
                                    cfg.cache_config.num_gpu_blocks_override) for s, a in zip(all_specs, all_avail)]
        specs = {}
        for s in all_specs:
            specs.update(s)
        from onecat_vllm.core.kv_cache_utils import KVCacheConfig
        kvc = KVCacheConfig(min(k.num_blocks for k in kvcs), cfg.cache_config.block_size, specs, max(k.num_state_slots for k in kvcs))
        cc = cfg.cache_config
        if (cc.kv_offloading_size > 0 or cc.num_cpu_blocks_override) and not any(s.kind == "mamba" for s in specs.values()):
            per_block = max(sum(s.page_size_bytes for s in sp.values()) for sp in all_specs)
            kvc.num_cpu_blocks = cc.num_cpu_blocks_override or int(cc.kv_offloading_size * (1 << 30) // max(per_block, 1))
        cc.num_cpu_blocks = kvc.num_cpu_blocks
        max_need = -(-cfg.model_config.max_model_len // cfg.cache_config.block_size) + 1
        if not any(s.kind != "mamba" for s in specs.values()) and cfg.cache_config.num_gpu_blocks_override is None:
            # no attention layer: blocks only count positions, so every sequence may reach max_model_len at once
            kvc.num_blocks = min((cfg.scheduler_config.max_num_seqs + 1) * max_need, 1 << 20)
        if kvc.num_blocks < max_need:
            raise ValueError(f"KV cache of {kvc.num_blocks} blocks cannot hold one sequence of max_model_len="
                             f"{cfg.model_config.max_model_len} ({max_need} blocks): lower max_model_len or raise gpu_memory_utilization")
        cfg.cache_config.num_gpu_blocks = kvc.num_blocks
        self.collective_rpc("initialize_from_config", (kvc,))
        self.collective_rpc("compile_or_warm_up_model")
        return kvc.num_blocks, kvc.num_state_slots

    def execute_model(self, scheduler_output):
        pc = self.cfg.parallel_config
        outs = self.collective_rpc("execute_model", (scheduler_output,))
        out = outs[min((pc.pipeline_parallel_size - 1) * pc.tensor_parallel_size, len(outs) - 1)]  # first TP rank of the last stage
        if pc.pipeline_parallel_size > 1:
            out.status = max(o.status for o in outs)
            out.device_time_ms = sum(o.device_time_ms for o in outs[:: pc.tensor_parallel_size])
        return out

    def launch_model(self, scheduler_output) -> None:
        self.collective_rpc("launch_model", (scheduler_output,))

    def collect_model(self):
        return self.collective_rpc("collect_model")[0]

    def check_health(self) -> None:
        self.collective_rpc("check_health", timeout=10)

    def shutdown(self) -> None:
        pass


class UniProcExecutor(Executor):
    def _init_executor(self) -> None:
        self.worker = Worker(self.cfg, 0, 0)
        self.worker.init_device()
        self.worker.load_model()

    def collective_rpc(self, method, args=(), kwargs=None, timeout=None):
        fn = getattr(self.worker, method) if isinstance(method, str) else (lambda *a, **k: method(self.worker, *a, **k))
        return [fn(*args, **(kwargs or {}))]

    def shutdown(self) -> None:
        if getattr(self, "worker", None) is not None:
            self.worker.shutdown()
            self.worker = None


class ExternalLauncherExecutor(UniProcExecutor):
    """One engine per torchrun rank; scheduling is deterministic so all ranks take identical steps."""

    def _init_executor(self) -> None:
        rank, local = int(os.environ["RANK"]), int(os.environ.get("LOCAL_RANK", 0))
        self.worker = Worker(self.cfg, rank, local, init_method="env://")
        self.worker.init_device()
        self.worker.load_model()
