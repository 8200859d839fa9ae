"""Paged KV-cache primitives: blocks, the LRU free queue and chained block hashes.

Behaviour follows the reference (reference: vllm/v1/core/kv_cache_utils.py:116 ``KVCacheBlock``, :164 free
queue, :375-571 hashing; block_pool.py:333-435 free order): freed blocks go to the tail of a doubly linked
list in reverse order and keep their hash until the block is handed out again.
"""
from __future__ import annotations

import hashlib
import pickle
from dataclasses import dataclass
from typing import Callable, Iterable, Optional

NONE_HASH = hashlib.sha256(b"onecat-kv-root").digest()


class KVCacheBlock:
    __slots__ = ("block_id", "ref_cnt", "block_hash", "prev_free", "next_free", "is_null")

    def __init__(self, block_id: int) -> None:
        self.block_id = block_id
        self.ref_cnt = 0
        self.block_hash: Optional[bytes] = None
        self.prev_free: Optional["KVCacheBlock"] = None
        self.next_free: Optional["KVCacheBlock"] = None
        self.is_null = False

    def __repr__(self) -> str:
        return f"KVCacheBlock(id={self.block_id}, ref={self.ref_cnt}, hashed={self.block_hash is not None})"


class FreeKVCacheBlockQueue:
    """Doubly linked list with sentinel head/tail; O(1) removal from the middle (needed when a cached
    free block is re-used by a prefix hit)."""

    def __init__(self, blocks: list[KVCacheBlock]) -> None:
        self.num_free_blocks = len(blocks)
        self.head = KVCacheBlock(-1)
        self.tail = KVCacheBlock(-1)
        prev = self.head
        for b in blocks:
            prev.next_free, b.prev_free = b, prev
            prev = b
        prev.next_free, self.tail.prev_free = self.tail, prev

    def popleft(self) -> KVCacheBlock:
        b = self.head.next_free
        if b is self.tail or b is None:
            raise ValueError("no free blocks")
        self.remove(b)
        return b

    def popleft_n(self, n: int) -> list[KVCacheBlock]:
        if n > self.num_free_blocks:
            raise ValueError("not enough free blocks")
        return [self.popleft() for _ in range(n)]

    def remove(self, b: KVCacheBlock) -> None:
        if b.prev_free is None or b.next_free is None:
            raise RuntimeError(f"block {b.block_id} is not in the free queue")
        b.prev_free.next_free, b.next_free.prev_free = b.next_free, b.prev_free
        b.prev_free = b.next_free = None
        self.num_free_blocks -= 1

    def append(self, b: KVCacheBlock) -> None:
        last = self.tail.prev_free
        last.next_free, b.prev_free = b, last
        b.next_free, self.tail.prev_free = self.tail, b
        self.num_free_blocks += 1

    def append_n(self, blocks: Iterable[KVCacheBlock]) -> None:
        for b in blocks:
            self.append(b)

    def get_all_free_blocks(self) -> list[KVCacheBlock]:
        out, cur = [], self.head.next_free
        while cur is not self.tail:
            out.append(cur)
            cur = cur.next_free
        return out


def _hash_fn(algo: str) -> Callable[[bytes], bytes]:
    if algo in ("sha256", "sha256_cbor"):
        return lambda b: hashlib.sha256(b).digest()
    if algo == "blake2b":
        return lambda b: hashlib.blake2b(b, digest_size=16).digest()
    raise ValueError(f"unknown hash algorithm {algo}")


def hash_block_tokens(hash_fn, parent_hash: Optional[bytes], token_ids: tuple, extra_keys: Optional[tuple] = None) -> bytes:
    """H(parent, tokens of one full block, extra keys) — the chain makes a hash identify the whole prefix."""
    return hash_fn(pickle.dumps((parent_hash or NONE_HASH, tuple(token_ids), extra_keys), protocol=4))


def make_block_hasher(block_size: int, algo: str = "sha256"):
    """Returns ``hasher(request) -> list[new block hashes]`` covering full blocks not hashed yet."""
    fn = _hash_fn(algo)

    def hasher(request) -> list[bytes]:
        start = len(request.block_hashes) * block_size
        toks = request.all_token_ids
        n = len(toks)
        if start + block_size > n:
            return []
        prev = request.block_hashes[-1] if request.block_hashes else None
        extra = (request.cache_salt,) if (request.cache_salt and start == 0) else None
        new = []
        while start + block_size <= n:
            h = hash_block_tokens(fn, prev, tuple(toks[start:start + block_size]), extra)
            new.append(h)
            prev, extra = h, None
            start += block_size
        return new

    return hasher


@dataclass
class KVCacheSpec:
    """Per-layer cache requirement (reference: v1/kv_cache_interface.py:95-838)."""

    kind: str  # "full" | "mla" | "mamba"
    block_size: int
    num_kv_heads: int
    head_size: int
    dtype_bytes: int
    state_bytes: int = 0  # mamba: bytes of recurrent + conv state per sequence

    @property
    def page_size_bytes(self) -> int:
        if self.kind == "mamba":
            return self.state_bytes
        coef = 1 if self.kind == "mla" else 2
        return coef * self.block_size * self.num_kv_heads * self.head_size * self.dtype_bytes


@dataclass
class KVCacheConfig:
    num_blocks: int
    block_size: int
    layer_specs: dict  # layer name -> KVCacheSpec
    num_state_slots: int = 0  # mamba/GDN slots (one per running sequence + spec copies)
    num_cpu_blocks: int = 0   # host mirror for the CPU tier of the prefix cache


def get_kv_cache_config(layer_specs: dict, available_bytes: int, block_size: int, max_num_seqs: int,
                        override_blocks: Optional[int] = None) -> KVCacheConfig:
    """Size the block pool from the memory left after weights/activations
    (reference: v1/core/kv_cache_utils.py:935,1839,1945). Mamba state is reserved first, one slot per
    sequence; the rest is split into pages shared by all attention layers."""
    attn = [s for s in layer_specs.values() if s.kind != "mamba"]
    mamba = [s for s in layer_specs.values() if s.kind == "mamba"]
    slots = max_num_seqs + 1 if mamba else 0
    reserved = sum(s.state_bytes for s in mamba) * slots
    per_block = sum(s.page_size_bytes for s in attn)
    if override_blocks is not None:
        n = override_blocks
    else:
        # a model without attention layers keeps no KV: its blocks are bookkeeping only (positions of a request), so the pool just has
        # to be large enough never to limit the batch
        n = max((available_bytes - reserved) // per_block, 0) if per_block else max(1024, (max_num_seqs + 1) * 256)
    if attn and n < 2:
        raise ValueError("not enough memory for the KV cache: increase gpu_memory_utilization or lower max_model_len")
    return KVCacheConfig(int(n), block_size, dict(layer_specs), slots)
