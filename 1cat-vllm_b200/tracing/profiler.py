"""Profiler hooks (reference: vllm/profiler/wrapper.py:19 ``WorkerProfiler``, :159 torch profiler, :310 CUDA profiler;
NVTX ranges vllm/sm70_decode_trace.py:44-83). ``worker_profiler().toggle(True/False)`` is driven by the
``/start_profile`` / ``/stop_profile`` routes through the engine core's utility RPC."""
from __future__ import annotations

import contextlib
import os
import time
from typing import Optional

import torch


class WorkerProfiler:
    def __init__(self, out_dir: Optional[str] = None):
        self.out_dir = out_dir or os.environ.get("ONECAT_TORCH_PROFILER_DIR")
        self.prof = None
        self.running = False

    def toggle(self, start: bool) -> None:
        if start and not self.running:
            if self.out_dir:
                acts = [torch.profiler.ProfilerActivity.CPU]
                if torch.cuda.is_available():
                    acts.append(torch.profiler.ProfilerActivity.CUDA)
                self.prof = torch.profiler.profile(activities=acts, on_trace_ready=torch.profiler.tensorboard_trace_handler(self.out_dir))
                self.prof.start()
            elif torch.cuda.is_available():
                torch.cuda.profiler.start()  # cudaProfilerStart: pairs with an external capture tool
            self.running = True
        elif not start and self.running:
            if self.prof is not None:
                self.prof.stop()
                self.prof = None
            elif torch.cuda.is_available():
                torch.cuda.profiler.stop()
            self.running = False


_WP: Optional[WorkerProfiler] = None


def worker_profiler() -> WorkerProfiler:
    global _WP
    if _WP is None:
        _WP = WorkerProfiler()
    return _WP


@contextlib.contextmanager
def nvtx_range(name: str, enabled: bool = True):
    """NVTX range when enabled and a GPU is present; otherwise free."""
    on = enabled and torch.cuda.is_available()
    if on:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if on:
            torch.cuda.nvtx.range_pop()


class StepTimer:
    """CPU phase timers of one engine step (reference: fork traces v1/engine/core.py:588-756)."""

    def __init__(self):
        self.t: dict = {}
        self._last = time.perf_counter()

    def mark(self, phase: str) -> None:
        now = time.perf_counter()
        self.t[phase] = self.t.get(phase, 0.0) + (now - self._last)
        self._last = now

    def reset(self) -> dict:
        out, self.t = self.t, {}
        self._last = time.perf_counter()
        return out
