"""Budget keeper of the encoder cache: which multimodal encoder outputs are (to be) held on the workers
(reference: vllm/v1/core/encoder_cache_manager.py ``EncoderCacheManager``: ``check_and_update_cache``, ``can_allocate``, ``allocate``,
``free_encoder_input``, ``get_freed_mm_hashes``).

Entries are keyed by the content hash of the item, so two requests with the same image share one entry; an entry nobody references
any more stays cached until its space is needed ("freeable", evicted oldest first). Sizes are in embedding positions."""
from __future__ import annotations

from collections import OrderedDict


class EncoderCacheManager:
    def __init__(self, cache_size: int):
        self.cache_size = cache_size
        self.num_free_slots = cache_size          # slots not occupied by any entry
        self.num_freeable_slots = cache_size      # free slots + slots of entries nobody references
        self.cached: dict[str, set] = {}          # mm_hash -> ids of the requests that use it
        self.sizes: dict[str, int] = {}
        self.freeable: "OrderedDict[str, int]" = OrderedDict()
        self.freed: list[str] = []

    def check_and_update_cache(self, request, input_id: int) -> bool:
        """True when the item's encoder output is already cached; the request then holds a reference to it."""
        h = request.mm_features[input_id].mm_hash
        if h not in self.cached:
            return False
        if not self.cached[h]:  # cached but unreferenced: take it back from the freeable list
            n = self.freeable.pop(h)
            self.num_freeable_slots -= n
        self.cached[h].add(request.request_id)
        return True

    def can_allocate(self, request, input_id: int, encoder_compute_budget: int, num_tokens_to_schedule: int = 0) -> bool:
        n = request.mm_features[input_id].length
        if n > encoder_compute_budget:
            return False
        need = n + num_tokens_to_schedule
        if need <= self.num_free_slots:
            return True
        if need > self.num_freeable_slots:
            return False
        while need > self.num_free_slots:  # evict unreferenced entries, oldest first
            h, k = self.freeable.popitem(last=False)
            del self.cached[h]
            del self.sizes[h]
            self.freed.append(h)
            self.num_free_slots += k
        return True

    def allocate(self, request, input_id: int) -> None:
        f = request.mm_features[input_id]
        self.cached.setdefault(f.mm_hash, set()).add(request.request_id)
        self.sizes[f.mm_hash] = f.length
        self.num_free_slots -= f.length
        self.num_freeable_slots -= f.length

    def get_cached_input_ids(self, request) -> set:
        return {i for i, f in enumerate(request.mm_features) if request.request_id in self.cached.get(f.mm_hash, ())}

    def free_encoder_input(self, request, input_id: int) -> None:
        h = request.mm_features[input_id].mm_hash
        refs = self.cached.get(h)
        if not refs or request.request_id not in refs:
            return
        refs.discard(request.request_id)
        if not refs:
            self.freeable[h] = self.sizes[h]
            self.num_freeable_slots += self.sizes[h]

    def free(self, request) -> None:
        for i in range(len(getattr(request, "mm_features", None) or [])):
            self.free_encoder_input(request, i)

    def reset(self) -> int:
        """Evict every entry that no request references (the workers drop the outputs with the next step's freed list). Entries
        still in use stay. Returns how many were evicted (reference: encoder_cache_manager.py ``reset``; the ``/reset_mm_cache`` route)."""
        n = 0
        for h, size in list(self.freeable.items()):
            del self.freeable[h]
            self.cached.pop(h, None)
            self.sizes.pop(h, None)
            self.num_free_slots += size
            self.freed.append(h)
            n += 1
        return n

    def get_freed_mm_hashes(self) -> list[str]:
        out, self.freed = self.freed, []
        return out
