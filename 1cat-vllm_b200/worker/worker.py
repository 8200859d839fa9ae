"""Per-device worker: device + process-group init, model load, memory profiling, KV allocation, warm-up and
CUDA-graph capture, step execution (reference: vllm/v1/worker/gpu_worker.py:112 class, :244 ``init_device``, :343
``load_model``, :366 ``determine_available_memory``, :552 ``initialize_from_config``, :581
``compile_or_warm_up_model``, :792 ``execute_model``; CPU variant v1/worker/cpu_worker.py:33)."""
from __future__ import annotations

import gc
import os
from typing import Optional

import torch

from onecat_vllm.config import VllmConfig
from onecat_vllm.core.kv_cache_utils import KVCacheConfig, get_kv_cache_config
from onecat_vllm.core.sched_output import ModelRunnerOutput, SchedulerOutput
from onecat_vllm.logger import decorate_logs, init_logger
from onecat_vllm.parallel import state as ps
from onecat_vllm.worker.model_runner import ModelRunner

log = init_logger(__name__)


class Worker:
    def __init__(self, vllm_config: VllmConfig, rank: int = 0, local_rank: int = 0, init_method: Optional[str] = None):
        self.cfg = vllm_config
        self.rank, self.local_rank = rank, local_rank
        self.init_method = init_method
        self.runner: Optional[ModelRunner] = None
        self.device = torch.device("cpu")
        self._baseline_free = 0
        self.sleeping = False

    def init_device(self) -> None:
        from onecat_vllm.utils.plugins import load_general_plugins
        load_general_plugins()  # worker processes register out-of-tree models too
        pc = self.cfg.parallel_config
        if self.cfg.device == "cuda":
            torch.cuda.set_device(self.local_rank)
            from onecat_vllm import envs as _envs
            if _envs.ONECAT_NUMA_BIND:
                from onecat_vllm.utils.numa import bind_to_gpu
                bind_to_gpu(self.local_rank)
            self.device = torch.device("cuda", self.local_rank)
            gc.collect()
            torch.cuda.empty_cache()
            self._baseline_free, self._total = torch.cuda.mem_get_info()
        ps.init_distributed(self.rank, pc.world_size, pc.tensor_parallel_size, pc.pipeline_parallel_size, init_method=self.init_method,
                            enable_ep=pc.enable_expert_parallel, dcp=pc.decode_context_parallel_size, tp_comm=pc.tp_comm)
        if pc.world_size > 1:
            decorate_logs(f"Worker_TP{ps.tp_rank()}")
        if self.cfg.device == "cuda" and pc.tensor_parallel_size > 1 and pc.tp_comm == "fused":
            from onecat_vllm.parallel.fused import FusedTP
            ps.get_state().fused = FusedTP.create(self.cfg, self.device)
            ps.get_state().fused.full_residual = self.cfg.speculative_config.method == "eagle3"
        from onecat_vllm import envs
        if pc.enable_expert_parallel and pc.tensor_parallel_size > 1 and envs.ONECAT_EP_COMM == "a2a" and self.cfg.model_config.num_experts:
            from onecat_vllm.parallel import all2all
            ps.get_state().ep_a2a = all2all.create(self.cfg, self.device)
        self.runner = ModelRunner(self.cfg, self.device)

    def _sleep_pools(self) -> bool:
        return bool(self.cfg.model_config.enable_sleep_mode) and self.device.type == "cuda"

    def load_model(self) -> None:
        from onecat_vllm.utils.cumem import maybe_pool
        with maybe_pool(self._sleep_pools(), "weights"):
            self.runner.load_model()

    def get_kv_cache_specs(self) -> dict:
        return self.runner.get_kv_cache_specs()

    def determine_available_memory(self) -> int:
        """Bytes available for the KV cache: requested share of the device minus what weights and a max-token
        profiling forward need."""
        cc = self.cfg.cache_config
        if cc.kv_cache_memory_bytes is not None:
            return cc.kv_cache_memory_bytes
        if self.device.type != "cuda":
            return int(os.environ.get("ONECAT_CPU_KVCACHE_BYTES", 1 << 30))
        torch.cuda.reset_peak_memory_stats()
        self.runner.dummy_run(self.cfg.scheduler_config.max_num_batched_tokens, 1)
        torch.cuda.synchronize()
        peak = torch.cuda.max_memory_allocated()
        free, total = torch.cuda.mem_get_info()
        non_torch = (total - free) - torch.cuda.memory_reserved()
        budget = int(total * cc.gpu_memory_utilization)
        avail = budget - peak - max(non_torch, 0)
        torch.cuda.empty_cache()
        log.info_once(f"memory: total {total >> 20} MiB, peak torch {peak >> 20} MiB, KV budget {avail >> 20} MiB")
        return max(avail, 0)

    def initialize_from_config(self, kvc: KVCacheConfig) -> None:
        from onecat_vllm.utils.cumem import maybe_pool
        with maybe_pool(self._sleep_pools(), "kv_cache"):
            self.runner.initialize_kv_cache(kvc)

    def compile_or_warm_up_model(self) -> None:
        if self.device.type != "cuda":
            return
        self.runner.dummy_run(min(256, self.cfg.scheduler_config.max_num_batched_tokens), 4)
        from onecat_vllm import envs
        eagle3 = self.cfg.speculative_config.method == "eagle3"
        if eagle3:
            # the head reads tensors recorded inside the target's forward; a replayed graph keeps those in its own pool, which the
            # drafting loop does not look into, so these steps run eagerly
            log.info_once("EAGLE-3 drafting: decode steps run without CUDA graphs")
        if not self.cfg.enforce_eager and envs.ONECAT_USE_CUDA_GRAPH and not eagle3:
            from onecat_vllm.worker.cuda_graphs import DecodeGraphs
            self.runner.graphs = DecodeGraphs(self.runner)
            self.runner.graphs.capture_all()
        torch.cuda.synchronize()

    def execute_model(self, so: SchedulerOutput) -> Optional[ModelRunnerOutput]:
        out = self.runner.execute_model(so)
        return out if ps.get_state().rank == 0 or True else None

    def launch_model(self, so: SchedulerOutput) -> None:
        """Async scheduling: enqueue the step and return; ``collect_model`` hands out the oldest step's result."""
        self.runner.launch_model(so)

    def collect_model(self) -> ModelRunnerOutput:
        return self.runner.collect_model()

    # ---- utility RPCs (reference: gpu_worker.py:160-200 sleep/wake, :885 profile, :958 save_sharded_state)
    def sleep(self, level: int = 1) -> None:
        """With sleep mode on (weights and KV cache in releasable memory): level 1 copies the weights to pinned host memory and
        gives the device memory of weights and KV cache back to the driver, level 2 gives back both without keeping the weights
        (the caller reloads or pushes new ones after ``wake_up``). Addresses stay valid, so captured graphs survive. Without
        sleep mode: level 1 drops the KV cache contents; level 2 also releases it.
        (reference: gpu_worker.py:147 ``sleep`` / :188 ``wake_up``)"""
        if self._sleep_pools():
            from onecat_vllm.utils.cumem import CuMemAllocator
            torch.cuda.synchronize()
            freed = CuMemAllocator.get().sleep(offload_tags=("weights",) if level == 1 else (), discard_tags=None if level == 1 else ("weights", "kv_cache"))
            log.info(f"sleep level {level}: released {freed / 2**30:.2f} GiB of device memory")
            self.sleeping = True
            return
        if self.runner.kv_caches and level >= 2:
            self.runner.kv_caches = []
            if self.device.type == "cuda":
                torch.cuda.empty_cache()
        self.sleeping = True

    def wake_up(self, tags=None) -> None:
        if self._sleep_pools():
            from onecat_vllm.utils.cumem import CuMemAllocator
            CuMemAllocator.get().wake_up(tags)
            if tags is None or "kv_cache" in tags:
                self.runner.zero_kv_cache()   # fresh physical pages: block 0 must read as zeros again
            self.sleeping = False
            return
        if not self.runner.kv_caches:
            self.runner.initialize_kv_cache(self.runner.kv_cache_config)
        self.sleeping = False

    def profile(self, start: bool) -> None:
        from onecat_vllm.tracing.profiler import worker_profiler
        worker_profiler().toggle(start)

    def save_sharded_state(self, path: str) -> None:
        from safetensors.torch import save_file
        os.makedirs(path, exist_ok=True)
        sd = {k: v.detach().cpu().contiguous() for k, v in self.runner.model.state_dict().items()
              if v.dtype not in (torch.float8_e4m3fn,)}
        save_file(sd, os.path.join(path, f"model-rank-{self.rank}.safetensors"))

    def update_weights(self, named: list) -> int:
        """In-place weight update for RLHF-style loops (reference: gpu_worker.py:987-1110)."""
        from onecat_vllm.loader.weights import load_weights, process_weights_after_loading
        n = len(load_weights(self.runner.model, named))
        process_weights_after_loading(self.runner.model)
        return n

    def update_weights_ipc(self, payload: bytes) -> int:
        """Weights shared by a trainer process on this node through CUDA-IPC / shared-memory handles
        (``onecat_vllm.utils.weight_transfer.pack_ipc``); they are copied into the model's own storage."""
        from onecat_vllm.utils.weight_transfer import unpack_ipc
        return self.update_weights(unpack_ipc(payload))

    def init_weight_transfer(self, init_method: str, rank: int, world_size: int, backend=None) -> bool:
        """Join the trainer's broadcast group (reference: gpu_worker.py ``init_weight_transfer_engine``)."""
        from onecat_vllm.utils.weight_transfer import BroadcastWeightTransfer
        self._wt = BroadcastWeightTransfer.init(init_method, rank, world_size, self.device, backend)
        return True

    def init_weight_transfer_offset(self, init_method: str, rank_offset: int, world_size: int, backend=None) -> bool:
        """The same call for every worker of the engine: worker r joins as rank ``rank_offset + r`` (the trainer is rank 0)."""
        return self.init_weight_transfer(init_method, int(rank_offset) + self.rank, world_size, backend)

    def update_weights_from_path(self, path: str) -> int:
        """Load the tensors of a safetensors checkpoint directory in place (HF names; any subset of the model)."""
        from onecat_vllm.loader.weights import iter_safetensors
        return self.update_weights(iter_safetensors(path))

    def update_weights_broadcast(self, meta: dict) -> int:
        """Receive the tensors the trainer (rank 0 of the transfer group) broadcasts and load them in place."""
        if getattr(self, "_wt", None) is None:
            raise ValueError("call init_weight_transfer first")
        return self.update_weights(((n, t.clone()) for n, t in self._wt.receive(meta)))

    # ---- LoRA adapters (reference: gpu_worker.py ``add_lora`` / ``remove_lora`` / ``list_loras``)
    def _lora(self):
        if self.runner.lora_manager is None:
            raise ValueError("LoRA is not enabled (enable_lora=True)")
        return self.runner.lora_manager

    def add_lora(self, req) -> bool:
        from onecat_vllm.lora import LoRARequest
        return self._lora().add_lora(LoRARequest.from_dict(req) if isinstance(req, dict) else req)

    def remove_lora(self, lora_id: int) -> bool:
        return self._lora().remove_lora(lora_id)

    def list_loras(self) -> list:
        return self._lora().list_loras()

    def check_health(self) -> bool:
        return True

    def shutdown(self) -> None:
        """Tear down in dependency order. Captured graphs hold kernels that reference the peer-memory slab and NCCL communicators,
        so they go first (with the device idle); then the slab mappings; the process group last. Destroying the group while a
        graph that captured its collectives is alive can block inside the communicator's own teardown."""
        r = self.runner
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        if r is not None and getattr(r, "graphs", None) is not None:
            r.graphs.release()
            r.graphs = None
        if r is not None and getattr(r, "_kv_server", None) is not None:
            r._kv_server.close()   # peer-to-peer KV connector: stop serving saved blocks
            r._kv_server = None
        self.runner = None
        r = None
        gc.collect()
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        ps.destroy_distributed()
        gc.collect()
        if self.device.type == "cuda":
            torch.cuda.empty_cache()
