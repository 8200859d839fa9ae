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

    def on_stored(self, block_hash: bytes, gpu_block: int) -> None:
        pass  # this tier saves on eviction only

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


class SharedStorageTier:
    """KV connector over a shared directory: every prefix block that becomes full is written through to ``<dir>/<hash>.kv`` and a
    later request — in this engine or in another one pointed at the same directory — restores it instead of recomputing. This is
    the disaggregated prefill / decode arrangement in its simplest form: the prefill instance runs the prompt (``max_tokens=1``),
    the decode instance finds the blocks by their chained hashes (reference: distributed/kv_transfer/kv_connector/v1/base.py:186
    ``KVConnectorBase_V1``; the example ``shared_storage_connector.py``; roles ``kv_producer`` / ``kv_consumer`` / ``kv_both``).
    Same interface as ``CPUOffloadTier``; handles are file paths."""

    def __init__(self, path: str, role: str = "kv_both") -> None:
        import os
        self.path, self.role = path, role
        os.makedirs(path, exist_ok=True)
        self.capacity = 1 << 62
        self.swap_out: list = []
        self.swap_in: list = []
        self.stored = self.restored = 0
        self._written: set = set()

    def _file(self, block_hash: bytes) -> str:
        import os
        return os.path.join(self.path, block_hash.hex() + ".kv")

    def on_evict(self, block_hash: bytes, gpu_block: int) -> None:
        pass  # written through when the block became full

    def on_stored(self, block_hash: bytes, gpu_block: int) -> None:
        import os
        if self.role == "kv_consumer" or block_hash in self._written:
            return
        f = self._file(block_hash)
        self._written.add(block_hash)
        if not os.path.exists(f):
            self.swap_out.append((gpu_block, f))
            self.stored += 1

    def lookup(self, block_hash: bytes):
        import os
        if self.role == "kv_producer":
            return None
        f = self._file(block_hash)
        return f if os.path.exists(f) else None

    def restore(self, handle, gpu_block: int) -> None:
        self.swap_in.append((handle, gpu_block))
        self.restored += 1

    def take_ops(self) -> tuple[list, list]:
        out, inn = self.swap_out, self.swap_in
        self.swap_out, self.swap_in = [], []
        return out, inn

    def reset(self) -> None:
        self.swap_out, self.swap_in = [], []
