"""KV-cache manager: prefix lookup + slot allocation per request
(reference: vllm/v1/core/kv_cache_manager.py:114 ``KVCacheManager``, :198 ``get_computed_blocks``,
:240 ``allocate_slots``; single_type_kv_cache_manager.py:509-557 for the chain walk).

Hybrid (Gated-DeltaNet) models additionally get one recurrent-state slot per sequence
(reference: single_type_kv_cache_manager.py:870 ``MambaManager``); their prefix cache is off because a
recurrent state cannot be rebuilt from a block hit."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

from onecat_vllm.core.block_pool import BlockPool
from onecat_vllm.core.kv_cache_utils import KVCacheBlock


@dataclass
class PrefixCacheStats:
    requests: int = 0
    queries: int = 0
    hits: int = 0
    reset: bool = False


def cdiv(a: int, b: int) -> int:
    return -(-a // b)


class KVCacheManager:
    def __init__(self, num_blocks: int, block_size: int, max_model_len: int, enable_caching: bool = True,
                 num_state_slots: int = 0, use_eagle: bool = False, dcp_world_size: int = 1, log_stats: bool = True,
                 sliding_window: int = 0) -> None:
        self.block_size = block_size * dcp_world_size  # with decode-CP a logical block spans all ranks
        self.max_model_len = max_model_len
        self.enable_caching = enable_caching and num_state_slots == 0
        self.use_eagle = use_eagle
        self.block_pool = BlockPool(num_blocks, self.enable_caching)
        self.req_to_blocks: dict[str, list[KVCacheBlock]] = {}
        self.num_cached_block: dict[str, int] = {}
        self.stats = PrefixCacheStats() if log_stats else None
        self.free_state_slots = list(range(num_state_slots - 1, -1, -1))
        self.req_to_state_slot: dict[str, int] = {}
        self.needs_state = num_state_slots > 0
        self.offload = None
        # Every layer attends to a window of `sliding_window` keys (Mistral-style models): blocks that lie wholly before the window of
        # the next query are given back while the request runs (reference: single_type_kv_cache_manager.py:570 ``SlidingWindowManager``
        # ``remove_skipped_blocks``). Models that mix windowed and global layers share one block table here and keep every block.
        self.sliding_window = sliding_window
        self.window_slack = 128  # keys kept below the window start: the attention kernels load whole key tiles and mask inside them

    def enable_cpu_offload(self, num_cpu_blocks: int, policy: str = "lru") -> None:
        from onecat_vllm.core.kv_offload import ARCOffloadTier, CPUOffloadTier
        if policy not in ("lru", "arc"):
            raise ValueError(f"kv offloading policy {policy!r} is not supported (lru | arc)")
        if policy == "arc":
            CPUOffloadTier = ARCOffloadTier
        if self.enable_caching and num_cpu_blocks > 0:
            self.offload = self.block_pool.offload = CPUOffloadTier(num_cpu_blocks)

    @property
    def usage(self) -> float:
        return self.block_pool.get_usage()

    def get_computed_blocks(self, request) -> tuple[list[KVCacheBlock], int]:
        """Longest cached prefix; at most ``num_tokens - 1`` tokens may hit so that the last token is
        recomputed and yields logits (reference: kv_cache_manager.py:216-222)."""
        if not self.enable_caching or (request.sampling_params is not None and request.sampling_params.prompt_logprobs is not None):
            return [], 0
        max_hit_tokens = request.num_tokens - 1
        max_blocks = max_hit_tokens // self.block_size
        hit: list[KVCacheBlock] = []
        for h in request.block_hashes[:max_blocks]:
            b = self.block_pool.get_cached_block(h)
            if b is None:
                break
            hit.append(b)
        if self.offload is not None and len(hit) < max_blocks:
            hit += self._restore_from_cpu(request.block_hashes[len(hit):max_blocks], hit)
        if self.use_eagle and hit:  # the draft head needs the hidden state of the last matched block
            hit.pop()
        if self.stats is not None:
            self.stats.requests += 1
            self.stats.queries += request.num_tokens
            self.stats.hits += len(hit) * self.block_size
        return hit, len(hit) * self.block_size

    def enable_kv_connector(self, kv_transfer_config: dict) -> None:
        from onecat_vllm.core.kv_offload import SharedStorageTier
        name = kv_transfer_config.get("kv_connector", "SharedStorageConnector")
        if name not in ("SharedStorageConnector", "ExampleConnector", "P2pConnector", "P2pNcclConnector"):
            raise ValueError(f"unknown kv_connector {name!r}: this build has SharedStorageConnector and P2pConnector")
        extra = kv_transfer_config.get("kv_connector_extra_config") or {}
        if self.enable_caching and name.startswith("P2p"):
            from onecat_vllm.core.kv_p2p import P2pTier
            self.offload = self.block_pool.offload = P2pTier(extra.get("host", "127.0.0.1"), int(extra.get("port", 14579)),
                                                             kv_transfer_config.get("kv_role", "kv_consumer"))
        elif self.enable_caching:
            self.offload = self.block_pool.offload = SharedStorageTier(extra.get("shared_storage_path", "/tmp/onecat_kv"),
                                                                       kv_transfer_config.get("kv_role", "kv_both"))

    def _restore_from_cpu(self, hashes: list, gpu_hits: list[KVCacheBlock]) -> list[KVCacheBlock]:
        """Continue a prefix match in the CPU tier: every consecutive hit gets a fresh GPU block, a restore copy for this step and its
        place in the GPU index; the blocks go back to the free queue (cached, unreferenced) so that the caller treats them like
        any other prefix hit. Keeps a reserve of free blocks so that restores never starve new tokens.

        The GPU hits found just before are unreferenced blocks at the head of the free queue (a partial eviction leaves exactly the
        surviving prefix there), so they are held while the fresh blocks are taken: otherwise the restore would pop the hits
        themselves, strip their hashes and hand them out a second time. Hits and restored blocks are released together, tail of
        the prefix first, which puts the whole prefix at the young end of the queue."""
        pool, got = self.block_pool, []
        pool.touch(gpu_hits)
        try:
            for h in hashes:
                c = self.offload.lookup(h)
                if c is None or pool.get_num_free_blocks() < 8:
                    break
                if pool.get_cached_block(h) is not None:  # came back through another request since the walk stopped
                    b = pool.get_cached_block(h)
                    pool.touch([b])
                    got.append(b)
                    continue
                b = pool.get_new_blocks(1)[0]
                b.block_hash = h
                pool.cached.setdefault(h, {})[b.block_id] = b
                self.offload.restore(c, b.block_id)
                got.append(b)
        finally:
            pool.free_blocks(reversed(gpu_hits + got))
        return got

    def allocate_slots(self, request, num_new_tokens: int, num_new_computed_tokens: int = 0,
                       new_computed_blocks: Optional[list[KVCacheBlock]] = None, num_lookahead_tokens: int = 0) -> Optional[list[KVCacheBlock]]:
        """Make room for ``num_new_tokens`` (+ lookahead). Returns the newly added blocks or ``None``
        when the pool cannot serve the request (the scheduler then preempts)."""
        assert num_new_tokens > 0
        new_computed_blocks = new_computed_blocks or []
        blocks = self.req_to_blocks.get(request.request_id, [])
        num_computed = request.num_computed_tokens + num_new_computed_tokens
        if self.sliding_window > 0 and blocks:
            self._free_out_of_window(blocks, num_computed)
        need_tokens = min(num_computed + num_new_tokens + num_lookahead_tokens, self.max_model_len)
        need_blocks = cdiv(need_tokens, self.block_size) - len(blocks) - len(new_computed_blocks)
        evictable_hits = sum(1 for b in new_computed_blocks if b.ref_cnt == 0 and not b.is_null)
        if need_blocks > self.block_pool.get_num_free_blocks() - evictable_hits:
            return None
        if self.needs_state and request.request_id not in self.req_to_state_slot:
            if not self.free_state_slots:
                return None
            self.req_to_state_slot[request.request_id] = self.free_state_slots.pop()
        if new_computed_blocks:
            assert not blocks, "prefix hits only apply to a request without blocks"
            self.block_pool.touch(new_computed_blocks)
            blocks = self.req_to_blocks.setdefault(request.request_id, [])
            blocks.extend(new_computed_blocks)
            self.num_cached_block[request.request_id] = len(new_computed_blocks)
        else:
            blocks = self.req_to_blocks.setdefault(request.request_id, [])
        new_blocks: list[KVCacheBlock] = []
        if need_blocks > 0:
            new_blocks = self.block_pool.get_new_blocks(need_blocks)
            blocks.extend(new_blocks)
        if self.enable_caching:
            # only tokens that are final (not speculative) may be published
            num_final = min(num_computed + num_new_tokens, request.num_tokens)
            self.block_pool.cache_full_blocks(request, blocks, self.num_cached_block.get(request.request_id, 0), num_final // self.block_size)
            self.num_cached_block[request.request_id] = max(self.num_cached_block.get(request.request_id, 0), num_final // self.block_size)
        return new_blocks

    def _free_out_of_window(self, blocks: list[KVCacheBlock], first_query_pos: int) -> None:
        """Keys at positions <= first_query_pos - window are invisible to this and every later query of the request: release the
        blocks they fill (their table entries become the placeholder block, so positions keep their indices)."""
        n = (first_query_pos - self.sliding_window + 1 - self.window_slack) // self.block_size
        gone = []
        for i in range(min(max(n, 0), len(blocks))):
            if not blocks[i].is_null:
                gone.append(blocks[i])
                blocks[i] = self.block_pool.null_block
        if gone:
            self.block_pool.free_blocks(gone)

    def free(self, request) -> None:
        blocks = self.req_to_blocks.pop(request.request_id, [])
        self.num_cached_block.pop(request.request_id, None)
        self.block_pool.free_blocks(reversed(blocks))  # tail blocks are evicted first
        slot = self.req_to_state_slot.pop(request.request_id, None)
        if slot is not None:
            self.free_state_slots.append(slot)

    def get_block_ids(self, request_id: str) -> list[int]:
        return [b.block_id for b in self.req_to_blocks.get(request_id, [])]

    def get_state_slot(self, request_id: str) -> int:
        return self.req_to_state_slot.get(request_id, -1)

    def reset_prefix_cache(self) -> bool:
        ok = self.block_pool.reset_prefix_cache()
        if ok and self.offload is not None:
            self.offload.reset()
        if ok and self.stats is not None:
            self.stats.reset = True
        return ok

    def get_num_common_prefix_blocks(self, running_request_id: str, num_running: int) -> int:
        n = 0
        for b in self.req_to_blocks.get(running_request_id, []):
            if b.ref_cnt == num_running:
                n += 1
            else:
                break
        return n

    def make_prefix_cache_stats(self) -> Optional[PrefixCacheStats]:
        if self.stats is None:
            return None
        s, self.stats = self.stats, PrefixCacheStats()
        return s
