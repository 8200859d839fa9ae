"""CPU tier of the prefix cache: KV blocks that the GPU pool evicts are copied to host memory and come back on a later prefix hit
(reference: vllm/v1/kv_offload/ — ``OffloadingManager`` with LRU / ARC policies, ``cpu`` backend with CUDA copies;
v1/simple_kv_offload/; scheduler hooks of distributed/kv_transfer/kv_connector/v1/offloading_connector.py).

The scheduler side (this file) only keeps books: block hash → CPU block, LRU order, and the copy lists of the current step. The
worker side (``worker/model_runner.py``) owns a host mirror of every attention layer's cache and executes the copies at the start
of the step — evictions first, then restores — so that an evicted block is saved before its new owner writes to it."""
from __future__ import annotations

from collections import OrderedDict
from typing import Optional


class CPUOffloadTier:
    def __init__(self, num_cpu_blocks: int) -> None:
        self.capacity = num_cpu_blocks
        self.index: "OrderedDict[bytes, int]" = OrderedDict()   # block hash -> CPU block, least recently used first
        self.free = list(range(num_cpu_blocks - 1, -1, -1))
        self.swap_out: list[tuple[int, int]] = []               # (GPU block, CPU block) copies of this step
        self.swap_in: list[tuple[int, int]] = []                # (CPU block, GPU block)
        self.stored = self.restored = 0

    def on_evict(self, block_hash: bytes, gpu_block: int) -> None:
        """The GPU pool is about to reuse a cached block: keep its contents on the host."""
        if self.capacity == 0:
            return
        if block_hash in self.index:
            self.index.move_to_end(block_hash)
            return
        if not self.free:
            # the LRU entry goes, unless a restore of this very step still reads from it
            busy = {c for c, _ in self.swap_in}
            victim = next((h for h, c in self.index.items() if c not in busy), None)
            if victim is None:
                return
            self.free.append(self.index.pop(victim))
        c = self.free.pop()
        self.index[block_hash] = c
        self.swap_out.append((gpu_block, c))
        self.stored += 1

    def lookup(self, block_hash: bytes) -> Optional[int]:
        c = self.index.get(block_hash)
        if c is not None:
            self.index.move_to_end(block_hash)
        return c

    def restore(self, cpu_block: int, gpu_block: int) -> None:
        self.swap_in.append((cpu_block, gpu_block))
        self.restored += 1

    def take_ops(self) -> tuple[list, list]:
        out, inn = self.swap_out, self.swap_in
        self.swap_out, self.swap_in = [], []
        return out, inn

    def reset(self) -> None:
        self.index.clear()
        self.free = list(range(self.capacity - 1, -1, -1))
        self.swap_out, self.swap_in = [], []
