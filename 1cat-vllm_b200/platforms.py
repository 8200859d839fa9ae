"""What the engine needs to know about the machine it runs on (reference: vllm/platforms/interface.py ``Platform``,
platforms/cuda.py, platforms/cpu.py; vllm/usage/usage_lib.py for the usage record).

Two platforms exist here: B200-class CUDA devices (the product) and the CPU (the PyTorch oracle path, which the tests run on).
``current_platform()`` picks one; the usage record is a local JSON line (there is no reporting server) written only when
``ONECAT_USAGE_STATS_FILE`` names a file."""
from __future__ import annotations

import json
import os
import platform as _pyplatform
import time
from dataclasses import dataclass
from typing import Optional

import torch


@dataclass
class Platform:
    device_type: str                      # "cuda" | "cpu"
    device_name: str
    dispatch_key: str                     # the ops module that serves it: "cuda" (ops/cuda.py) or "ref" (ops/ref.py)

    def is_cuda(self) -> bool:
        return self.device_type == "cuda"

    def is_cpu(self) -> bool:
        return self.device_type == "cpu"

    # ---- capabilities
    def compute_capability(self, index: int = 0) -> Optional[tuple[int, int]]:
        return None

    def supports_native_kernels(self, index: int = 0) -> bool:
        """The sm_100a kernels of this package run (tcgen05 / TMEM / TMA need compute capability 10.x)."""
        return False

    def total_memory(self, index: int = 0) -> int:
        return 0

    def device_count(self) -> int:
        return 1

    def default_dtype(self) -> torch.dtype:
        return torch.float32

    def supported_dtypes(self) -> tuple:
        return (torch.float32, torch.bfloat16)

    def describe(self) -> dict:
        return {"device_type": self.device_type, "device_name": self.device_name, "device_count": self.device_count(),
                "compute_capability": self.compute_capability(), "native_kernels": self.supports_native_kernels(),
                "total_memory": self.total_memory(), "default_dtype": str(self.default_dtype())}


class CpuPlatform(Platform):
    def __init__(self):
        super().__init__("cpu", _pyplatform.processor() or _pyplatform.machine(), "ref")

    def total_memory(self, index: int = 0) -> int:
        try:
            return os.sysconf("SC_PAGE_SIZE") * os.sysconf("SC_PHYS_PAGES")
        except (ValueError, OSError):
            return 0


class CudaPlatform(Platform):
    def __init__(self):
        super().__init__("cuda", torch.cuda.get_device_name(0), "cuda")

    def compute_capability(self, index: int = 0) -> Optional[tuple[int, int]]:
        return tuple(torch.cuda.get_device_capability(index))

    def supports_native_kernels(self, index: int = 0) -> bool:
        return self.compute_capability(index)[0] == 10

    def total_memory(self, index: int = 0) -> int:
        return int(torch.cuda.get_device_properties(index).total_memory)

    def device_count(self) -> int:
        return torch.cuda.device_count()

    def default_dtype(self) -> torch.dtype:
        return torch.bfloat16

    def supported_dtypes(self) -> tuple:
        return (torch.bfloat16,)


_current: Optional[Platform] = None


def current_platform(refresh: bool = False) -> Platform:
    global _current
    if _current is None or refresh:
        _current = CudaPlatform() if torch.cuda.is_available() else CpuPlatform()
    return _current


def resolve_device(device: str) -> str:
    """``auto`` -> the platform's device type; anything else is checked against what exists."""
    if device == "auto":
        return current_platform().device_type
    if device.startswith("cuda") and not torch.cuda.is_available():
        raise ValueError("device='cuda' was asked for but no CUDA device is visible")
    return device


def usage_record(context: str, model_architecture: Optional[str] = None, extra: Optional[dict] = None) -> dict:
    """One record of how the engine was started (architecture, parallel sizes, platform); appended to
    ``ONECAT_USAGE_STATS_FILE`` when that is set, and returned either way."""
    rec = {"time": time.time(), "context": context, "architecture": model_architecture, "platform": current_platform().describe(),
           "python": _pyplatform.python_version(), "torch": torch.__version__}
    rec.update(extra or {})
    path = os.environ.get("ONECAT_USAGE_STATS_FILE")
    if path:
        try:
            with open(path, "a") as f:
                f.write(json.dumps(rec) + "\n")
        except OSError:
            pass
    return rec
