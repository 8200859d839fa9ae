"""Clients of the engine core (reference: vllm/v1/engine/core_client.py:82 ``make_client``, :275 ``InprocClient``,
:748 ``SyncMPClient``, :919 ``AsyncMPClient``). ``InprocClient`` steps the core inside the caller; the MP clients
talk to an ``EngineCoreProc`` over ZMQ with msgpack frames and raise ``EngineDeadError`` when it dies."""
from __future__ import annotations

from onecat_vllm.config import VllmConfig
from onecat_vllm.request import EngineCoreOutputs, EngineCoreRequest


class InprocClient:
    def __init__(self, cfg: VllmConfig, log_stats: bool = False):
        from onecat_vllm.engine.core import EngineCore
        self.core = EngineCore(cfg, log_stats=log_stats)

    def add_request(self, req: EngineCoreRequest) -> None:
        self.core.add_request(req)

    def abort_requests(self, ids: list[str]) -> None:
        if ids:
            self.core.abort_requests(ids)

    def get_output(self) -> EngineCoreOutputs:
        outs, _ = self.core.step()
        return outs.get(0) or EngineCoreOutputs()

    def call_utility(self, method: str, *args):
        return getattr(self.core, method)(*args)

    def shutdown(self) -> None:
        self.core.shutdown()


def make_client(cfg: VllmConfig, multiprocess: bool, asyncio_mode: bool, log_stats: bool = False):
    if cfg.parallel_config.data_parallel_size > 1:
        multiprocess = True  # replicas are engine-core processes behind one load-balancing client
    if not multiprocess and not asyncio_mode:
        return InprocClient(cfg, log_stats)
    from onecat_vllm.engine.core_proc import AsyncMPClient, SyncMPClient
    return AsyncMPClient(cfg, log_stats) if asyncio_mode else SyncMPClient(cfg, log_stats)
