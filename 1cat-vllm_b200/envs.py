"""Typed, lazily evaluated environment flags.

The reference exposes several hundred ``VLLM_*`` variables through a module
``__getattr__`` table that can be frozen after start-up (reference:
vllm/envs.py:989,3820,3838). This engine keeps the mechanism and a short table.
"""
from __future__ import annotations

import os
from typing import Any, Callable

_TRUE = ("1", "true", "yes", "on")


def _b(name: str, default: bool) -> Callable[[], bool]:
    return lambda: os.environ.get(name, str(int(default))).lower() in _TRUE


def _i(name: str, default: int) -> Callable[[], int]:
    return lambda: int(os.environ.get(name, default))


def _s(name: str, default):
    return lambda: os.environ.get(name, default)


environment_variables: dict[str, Callable[[], Any]] = {
    # process model
    "ONECAT_ENABLE_MULTIPROCESSING": _b("ONECAT_ENABLE_MULTIPROCESSING", False),
    "ONECAT_WORKER_MULTIPROC_METHOD": _s("ONECAT_WORKER_MULTIPROC_METHOD", "spawn"),
    "ONECAT_EXECUTE_MODEL_TIMEOUT_SECONDS": _i("ONECAT_EXECUTE_MODEL_TIMEOUT_SECONDS", 300),
    "ONECAT_HANDSHAKE_TIMEOUT_SECONDS": _i("ONECAT_HANDSHAKE_TIMEOUT_SECONDS", 120),
    "ONECAT_RPC_RING_CHUNK_BYTES": _i("ONECAT_RPC_RING_CHUNK_BYTES", 1 << 22),
    "ONECAT_RPC_RING_CHUNKS": _i("ONECAT_RPC_RING_CHUNKS", 8),
    "ONECAT_DP_COORDINATOR": _i("ONECAT_DP_COORDINATOR", 0),  # 1: data-parallel replicas report to a coordinator process (shared load table, waves)
    "ONECAT_NUMA_BIND": _i("ONECAT_NUMA_BIND", 0),  # 1: each GPU worker pins itself to the cores of its GPU's NUMA node
    # kernels
    "ONECAT_CPU_ATTENTION": _s("ONECAT_CPU_ATTENTION", "torch"),  # paged attention of the CPU backend: "torch" (the oracle) | "native" (C++ threads)
    "ONECAT_GEMM_BACKEND": _s("ONECAT_GEMM_BACKEND", "tcgen05"),  # "tcgen05" | "library" (debug only)
    "ONECAT_ATTN_PREFILL": _s("ONECAT_ATTN_PREFILL", "tcgen05"),  # head size 128 prefill attention: "tcgen05" | "mma"
    "ONECAT_TP_COMM": _s("ONECAT_TP_COMM", "fused"),  # "fused" (peer-memory kernels) | "nccl" (baseline)
    "ONECAT_TP_ONESHOT": _s("ONECAT_TP_ONESHOT", "lamport"),  # decode-sized reductions: "lamport" (data is its own flag) | "flags"
    # reductions inside the switch (multimem) when every rank has multicast support: auto (the batch sizes where they measured
    # faster than the peer-store kernels) | 1 (every size) | 0 (never)
    "ONECAT_TP_NVLS": _s("ONECAT_TP_NVLS", "auto"),
    "ONECAT_TP_NVLS_MIN_T": _s("ONECAT_TP_NVLS_MIN_T", "1"),  # smallest batch (rows) that takes the switch reduction
    "ONECAT_TP_PUSH": _s("ONECAT_TP_PUSH", "auto"),  # GEMM epilogue pushes partial tiles to peers: auto | always | never
    # expert parallelism: "reduce" = every rank runs its experts over all tokens and the partial sums ride the TP reduction;
    # "a2a" = each rank routes a slice of the tokens and rows are exchanged with the expert owners (peer-memory kernels, or
    # torch.distributed all_to_all with ONECAT_EP_A2A=torch) for batches of at least ONECAT_EP_A2A_MIN_TOKENS tokens
    "ONECAT_EP_COMM": _s("ONECAT_EP_COMM", "reduce"),
    "ONECAT_EP_A2A": _s("ONECAT_EP_A2A", "peer"),
    "ONECAT_EP_A2A_MIN_TOKENS": _i("ONECAT_EP_A2A_MIN_TOKENS", 0),
    "ONECAT_ASYNC_SCHEDULING": _s("ONECAT_ASYNC_SCHEDULING", ""),  # "1" / "0" override the engine argument; empty: follow it
    "ONECAT_DEVICE_WAIT_LIMIT_MS": _i("ONECAT_DEVICE_WAIT_LIMIT_MS", 2000),
    "ONECAT_USE_CUDA_GRAPH": _b("ONECAT_USE_CUDA_GRAPH", True),
    "ONECAT_COMPUTE_NANS_IN_LOGITS": _b("ONECAT_COMPUTE_NANS_IN_LOGITS", False),
    # observability
    "ONECAT_LOGGING_LEVEL": _s("ONECAT_LOGGING_LEVEL", "INFO"),
    "ONECAT_STEP_TRACE": _b("ONECAT_STEP_TRACE", False),
    "ONECAT_NVTX": _b("ONECAT_NVTX", False),
    "ONECAT_OTLP_ENDPOINT": _s("ONECAT_OTLP_ENDPOINT", None),
    # serving
    "ONECAT_API_KEY": _s("ONECAT_API_KEY", None),
    "ONECAT_HOST_IP": _s("ONECAT_HOST_IP", "127.0.0.1"),
    "ONECAT_SERVER_DEV_MODE": _b("ONECAT_SERVER_DEV_MODE", False),  # registers /sleep, /pause, /collective_rpc, /start_profile, ...
    "ONECAT_ALLOW_RUNTIME_LORA_UPDATING": _b("ONECAT_ALLOW_RUNTIME_LORA_UPDATING", False),  # /v1/load_lora_adapter, /v1/unload_lora_adapter
    "ONECAT_USE_NATIVE_FRONTEND": _b("ONECAT_USE_NATIVE_FRONTEND", False),
}

_cache: dict[str, Any] = {}
_frozen = False


def __getattr__(name: str) -> Any:
    if name in _cache:
        return _cache[name]
    fn = environment_variables.get(name)
    if fn is None:
        raise AttributeError(f"module 'envs' has no attribute {name!r}")
    val = fn()
    if _frozen:
        _cache[name] = val
    return val


def enable_envs_cache() -> None:
    """Freeze values after start-up so hot paths never touch ``os.environ``."""
    global _frozen
    _frozen = True
    for k, fn in environment_variables.items():
        _cache[k] = fn()


def disable_envs_cache() -> None:
    global _frozen
    _frozen = False
    _cache.clear()


def is_set(name: str) -> bool:
    return name in os.environ
