"""Block pool with reference counting and a prefix-cache index
(reference: vllm/v1/core/block_pool.py:130 ``BlockPool``, :184 ``get_cached_block``, :211 ``cache_full_blocks``,
:333 ``get_new_blocks``, :389 ``touch``, :408 ``free_blocks``)."""
from __future__ import annotations

from typing import Iterable, Optional

from onecat_vllm.core.kv_cache_utils import FreeKVCacheBlockQueue, KVCacheBlock


class BlockPool:
    def __init__(self, num_blocks: int, enable_caching: bool = True) -> None:
        assert num_blocks >= 1
        self.num_blocks = num_blocks
        self.enable_caching = enable_caching
        self.blocks = [KVCacheBlock(i) for i in range(num_blocks)]
        self.free_queue = FreeKVCacheBlockQueue(self.blocks)
        self.cached: dict[bytes, dict[int, KVCacheBlock]] = {}
        # block 0 is a placeholder that is never written to nor freed
        self.null_block = self.free_queue.popleft()
        self.null_block.is_null = True
        self.events: list = []
        self.offload = None  # CPUOffloadTier: told about every cached block the pool is about to reuse

    def get_cached_block(self, block_hash: bytes) -> Optional[KVCacheBlock]:
        d = self.cached.get(block_hash)
        if not d:
            return None
        return next(iter(d.values()))

    def cache_full_blocks(self, request, blocks: list[KVCacheBlock], num_cached: int, num_full: int) -> None:
        """Give blocks[num_cached:num_full] their hash and publish them in the index."""
        if not self.enable_caching or num_full <= num_cached:
            return
        assert len(request.block_hashes) >= num_full
        for i in range(num_cached, num_full):
            b = blocks[i]
            if b.block_hash is not None or b.is_null:
                continue
            b.block_hash = request.block_hashes[i]
            self.cached.setdefault(b.block_hash, {})[b.block_id] = b
            self.events.append(("stored", b.block_id, b.block_hash))
            if self.offload is not None:
                self.offload.on_stored(b.block_hash, b.block_id)

    def get_new_blocks(self, n: int) -> list[KVCacheBlock]:
        if n > self.get_num_free_blocks():
            raise ValueError(f"cannot get {n} free blocks from the pool")
        out = self.free_queue.popleft_n(n)
        for b in out:
            if self.enable_caching:
                self._maybe_evict(b)
            assert b.ref_cnt == 0
            b.ref_cnt = 1
        return out

    def _maybe_evict(self, b: KVCacheBlock) -> bool:
        h = b.block_hash
        if h is None:
            return False
        d = self.cached.get(h)
        if d is not None:
            d.pop(b.block_id, None)
            if not d:
                del self.cached[h]
                if self.offload is not None:  # the last GPU copy of this prefix block: keep it on the host
                    self.offload.on_evict(h, b.block_id)
        b.block_hash = None
        self.events.append(("removed", b.block_id, h))
        return True

    def touch(self, blocks: Iterable[KVCacheBlock]) -> None:
        """A prefix hit re-uses blocks: take them out of the free queue if nobody holds them."""
        for b in blocks:
            if b.ref_cnt == 0 and not b.is_null:
                self.free_queue.remove(b)
            b.ref_cnt += 1

    def free_blocks(self, ordered: Iterable[KVCacheBlock]) -> None:
        """``ordered`` is in eviction priority: first in the list is evicted first."""
        for b in ordered:
            if b.is_null:
                continue
            b.ref_cnt -= 1
            assert b.ref_cnt >= 0
            if b.ref_cnt == 0:
                self.free_queue.append(b)

    def reset_prefix_cache(self) -> bool:
        used = self.num_blocks - self.get_num_free_blocks()
        if used != 1:  # only the null block may be held
            return False
        self.cached.clear()
        for b in self.blocks:
            b.block_hash = None
        self.events.append(("cleared", -1, None))
        return True

    def get_num_free_blocks(self) -> int:
        return self.free_queue.num_free_blocks

    def get_usage(self) -> float:
        total = self.num_blocks - 1
        return 0.0 if total <= 0 else 1.0 - self.get_num_free_blocks() / total

    def take_events(self) -> list:
        ev, self.events = self.events, []
        return ev
