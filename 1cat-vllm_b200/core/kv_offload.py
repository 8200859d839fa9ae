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


class ARCOffloadTier(CPUOffloadTier):
    """The same tier with adaptive-replacement eviction: resident blocks live in a recency list T1 (seen once) or a frequency list
    T2 (seen again); hashes of recently evicted blocks are remembered in ghost lists B1 / B2, and a hit on a ghost moves the target
    size ``p`` of T1 towards whichever list would have kept the block (reference: v1/kv_offload/ ARC policy of the CPU offloading
    manager; Megiddo & Modha's algorithm). A scan of one-off prefixes therefore cannot flush the blocks that are re-used."""

    def __init__(self, num_cpu_blocks: int) -> None:
        super().__init__(num_cpu_blocks)
        self.t1: "OrderedDict[bytes, int]" = OrderedDict()
        self.t2: "OrderedDict[bytes, int]" = OrderedDict()
        self.b1: "OrderedDict[bytes, None]" = OrderedDict()
        self.b2: "OrderedDict[bytes, None]" = OrderedDict()
        self.p = 0.0

    def _evict_from(self, lst: OrderedDict, ghosts: OrderedDict) -> bool:
        busy = {c for c, _ in self.swap_in}
        victim = next((h for h, c in lst.items() if c not in busy), None)
        if victim is None:
            return False
        self.free.append(lst.pop(victim))
        self.index.pop(victim, None)
        ghosts[victim] = None
        return True

    def _replace(self, in_b2: bool) -> bool:
        if self.t1 and (len(self.t1) > self.p or (in_b2 and len(self.t1) == int(self.p))):
            return self._evict_from(self.t1, self.b1) or self._evict_from(self.t2, self.b2)
        return self._evict_from(self.t2, self.b2) or self._evict_from(self.t1, self.b1)

    def on_evict(self, block_hash: bytes, gpu_block: int) -> None:
        c = self.capacity
        if c == 0:
            return
        if block_hash in self.index:   # already resident: a second sighting
            self.lookup(block_hash)
            return
        target = self.t1
        if block_hash in self.b1:
            self.p = min(float(c), self.p + max(1.0, len(self.b2) / max(len(self.b1), 1)))
            del self.b1[block_hash]
            target = self.t2
            if not self.free and not self._replace(False):
                return
        elif block_hash in self.b2:
            self.p = max(0.0, self.p - max(1.0, len(self.b1) / max(len(self.b2), 1)))
            del self.b2[block_hash]
            target = self.t2
            if not self.free and not self._replace(True):
                return
        else:
            if len(self.t1) + len(self.b1) >= c:
                if len(self.t1) < c:
                    self.b1.popitem(last=False)
                    if not self.free and not self._replace(False):
                        return
                elif not self._evict_from(self.t1, self.b1):
                    return
                else:
                    self.b1.popitem()   # a block dropped from a full T1 leaves no ghost
            else:
                total = len(self.t1) + len(self.t2) + len(self.b1) + len(self.b2)
                if total >= c:
                    if total >= 2 * c and self.b2:
                        self.b2.popitem(last=False)
                    if not self.free and not self._replace(False):
                        return
        if not self.free:
            return
        blk = self.free.pop()
        target[block_hash] = blk
        self.index[block_hash] = blk
        self.swap_out.append((gpu_block, blk))
        self.stored += 1

    def lookup(self, block_hash: bytes) -> Optional[int]:
        if block_hash in self.t1:
            self.t2[block_hash] = self.t1.pop(block_hash)
        elif block_hash in self.t2:
            self.t2.move_to_end(block_hash)
        return self.index.get(block_hash)

    def reset(self) -> None:
        super().reset()
        self.t1.clear(), self.t2.clear(), self.b1.clear(), self.b2.clear()
        self.p = 0.0


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
