"""Sleep-mode memory: tensors allocated inside ``use_memory_pool(tag)`` live in device memory whose physical pages can be released
(``sleep``) and re-created at the same virtual addresses (``wake_up``), so weights, KV caches and anything that points at them
(captured CUDA graphs included) survive. Tags say what a sleep does with a pool: contents of *offloaded* tags are copied to pinned
host memory and restored on wake-up, *discarded* tags come back uninitialised.

The allocator itself is native (``csrc/cumem/cumem_allocator.cpp`` → ``utils/_cumem.so``, driver virtual-memory API); PyTorch reaches
it through ``torch.cuda.memory.CUDAPluggableAllocator`` + ``torch.cuda.MemPool``.
(reference: vllm/device_allocator/cumem.py:93 ``CuMemAllocator``: use_memory_pool :196, sleep :241, wake_up :307; csrc/cumem_allocator.cpp)"""
from __future__ import annotations

import contextlib
import ctypes
import os
from typing import Iterable, Optional

TAGS = {"default": 0, "weights": 1, "kv_cache": 2, "graphs": 3}


def _so_path() -> str:
    return os.path.join(os.path.dirname(os.path.abspath(__file__)), "_cumem.so")


def _mask(tags: Optional[Iterable[str]]) -> int:
    if tags is None:
        return 0x7FFFFFFF
    m = 0
    for t in tags:
        m |= 1 << TAGS[t]
    return m


class CuMemAllocator:
    _instance: Optional["CuMemAllocator"] = None

    @classmethod
    def get(cls) -> "CuMemAllocator":
        if cls._instance is None:
            cls._instance = cls()
        return cls._instance

    def __init__(self, so_path: Optional[str] = None):
        path = so_path or _so_path()
        if not os.path.exists(path):
            raise RuntimeError(f"{path} is missing: build it with csrc/cumem/build.py")
        self.path = path
        self.lib = ctypes.CDLL(path)
        self.lib.onecat_cumem_malloc.restype = ctypes.c_void_p
        self.lib.onecat_cumem_malloc.argtypes = [ctypes.c_ssize_t, ctypes.c_int, ctypes.c_void_p]
        self.lib.onecat_cumem_free.argtypes = [ctypes.c_void_p, ctypes.c_ssize_t, ctypes.c_int, ctypes.c_void_p]
        self.lib.onecat_cumem_sleep.restype = ctypes.c_longlong
        self.lib.onecat_cumem_sleep.argtypes = [ctypes.c_uint, ctypes.c_uint]
        self.lib.onecat_cumem_wake.restype = ctypes.c_longlong
        self.lib.onecat_cumem_wake.argtypes = [ctypes.c_uint]
        self.lib.onecat_cumem_stat.restype = ctypes.c_longlong
        self.lib.onecat_cumem_stat.argtypes = [ctypes.c_int, ctypes.c_uint]
        self.lib.onecat_cumem_last_error.restype = ctypes.c_char_p
        self._pools: dict = {}
        self._torch_alloc = None

    # ---- raw interface (also what the CPU tests drive, against a stand-in driver)
    def malloc(self, size: int, device: int = 0) -> int:
        p = self.lib.onecat_cumem_malloc(size, device, None)
        if not p:
            raise MemoryError(self.last_error())
        return p

    def free(self, ptr: int) -> None:
        self.lib.onecat_cumem_free(ptr, 0, 0, None)

    def set_tag(self, tag: str) -> None:
        self.lib.onecat_cumem_set_tag(TAGS[tag])

    def last_error(self) -> str:
        return (self.lib.onecat_cumem_last_error() or b"").decode()

    def stats(self, tags: Optional[Iterable[str]] = None) -> dict:
        m = _mask(tags)
        return {"mapped_bytes": self.lib.onecat_cumem_stat(0, m), "asleep_bytes": self.lib.onecat_cumem_stat(1, m),
                "host_backup_bytes": self.lib.onecat_cumem_stat(2, m), "allocations": self.lib.onecat_cumem_stat(3, m)}

    def sleep(self, offload_tags: Iterable[str] = ("weights",), discard_tags: Optional[Iterable[str]] = None) -> int:
        """Release the physical memory of the named pools; returns the bytes given back to the driver. ``discard_tags=None``
        means every other pool."""
        off = _mask(offload_tags)
        disc = (_mask(None) & ~off) if discard_tags is None else _mask(discard_tags)
        n = self.lib.onecat_cumem_sleep(off, disc)
        if n < 0:
            raise RuntimeError("sleep failed: " + self.last_error())
        return n

    def wake_up(self, tags: Optional[Iterable[str]] = None) -> int:
        n = self.lib.onecat_cumem_wake(_mask(tags))
        if n < 0:
            raise RuntimeError("wake_up failed: " + self.last_error())
        return n

    # ---- PyTorch integration
    @contextlib.contextmanager
    def use_memory_pool(self, tag: str = "default"):
        """Allocations PyTorch makes inside the block come from this allocator and carry ``tag``."""
        import torch
        if self._torch_alloc is None:
            self._torch_alloc = torch.cuda.memory.CUDAPluggableAllocator(self.path, "onecat_cumem_malloc", "onecat_cumem_free")
        pool = self._pools.get(tag)
        if pool is None:
            pool = self._pools[tag] = torch.cuda.MemPool(self._torch_alloc.allocator())
        self.set_tag(tag)
        try:
            with torch.cuda.use_mem_pool(pool):
                yield
        finally:
            self.set_tag("default")


@contextlib.contextmanager
def maybe_pool(enabled: bool, tag: str):
    """``use_memory_pool(tag)`` when sleep mode is on and a GPU is in use, otherwise nothing."""
    if not enabled:
        yield
        return
    with CuMemAllocator.get().use_memory_pool(tag):
        yield
