"""Multimodal inputs: items → placeholder ranges in the prompt + encoder inputs, identified by content hashes
(reference: vllm/multimodal/registry.py:98 ``MultiModalRegistry``; multimodal/processing/processor.py:972 ``BaseMultiModalProcessor``
with its prompt updates; multimodal/hasher.py; multimodal/inputs.py ``MultiModalFeatureSpec`` / ``PlaceholderRange``).

A prompt may carry ``multi_modal_data = {"image": item | [items]}``. An item is either

* ready embeddings ``[n, hidden]`` (``{"image_embeds": tensor}`` or a bare 2-D tensor): they replace the ``n`` placeholder positions as
  they are (reference: the ``image_embeds`` input of the Qwen2-VL family), or
* encoder input ``{"pixel_values": [patches, patch_dim], "image_grid_thw": (t, h, w)}``: the model's vision tower turns it into
  ``t * h * w / merge^2`` embeddings when the scheduler schedules that encoder input.

The processor finds each placeholder token in the prompt (one per item, the model's ``image_token_id``), expands it to the item's
number of embedding positions and records the range; the content hash of an item keys the encoder cache, so that the same image in
two requests is encoded once, and salts the prefix cache, so that two different images behind the same placeholder ids never share
KV blocks."""
from __future__ import annotations

import hashlib
from dataclasses import dataclass, field
from typing import Any, Callable, Optional

import torch


@dataclass
class MultiModalFeature:
    modality: str          # "image" | "video" | "audio"
    mm_hash: str           # content hash: encoder-cache key
    offset: int            # first placeholder position in the (expanded) prompt
    length: int            # number of embedding positions
    kind: str              # "embeds" (data is [length, hidden]) | "pixels" (data is the encoder's input dict)
    data: Any = None

    def to_wire(self) -> dict:
        return {"modality": self.modality, "mm_hash": self.mm_hash, "offset": self.offset, "length": self.length, "kind": self.kind, "data": self.data}

    @classmethod
    def from_wire(cls, d: dict) -> "MultiModalFeature":
        return cls(d["modality"], d["mm_hash"], int(d["offset"]), int(d["length"]), d["kind"], d.get("data"))


def hash_item(modality: str, item: Any) -> str:
    """Content hash of one item: dtype, shape and bytes of every tensor it holds (reference: multimodal/hasher.py)."""
    h = hashlib.sha256(modality.encode())

    def feed(x):
        if isinstance(x, torch.Tensor):
            t = x.detach().cpu().contiguous()
            h.update(str(t.dtype).encode() + str(tuple(t.shape)).encode())
            h.update(t.view(torch.uint8).numpy().tobytes() if t.numel() else b"")
        elif isinstance(x, dict):
            for k in sorted(x):
                h.update(str(k).encode())
                feed(x[k])
        elif isinstance(x, (list, tuple)):
            for y in x:
                feed(y)
        else:
            h.update(repr(x).encode())
    feed(item)
    return h.hexdigest()


@dataclass
class ProcessedPrompt:
    token_ids: list[int]
    features: list[MultiModalFeature] = field(default_factory=list)


class MultiModalProcessor:
    """Default processor: one placeholder token per item in the prompt, expanded to the item's length."""

    def __init__(self, placeholder_ids: dict[str, int], hidden_size: int, merge_size: int = 2):
        self.placeholder_ids, self.hidden, self.merge = placeholder_ids, hidden_size, merge_size

    def item_length(self, modality: str, item: Any) -> tuple[str, int, Any]:
        if isinstance(item, torch.Tensor) or (isinstance(item, dict) and f"{modality}_embeds" in item):
            e = item if isinstance(item, torch.Tensor) else torch.as_tensor(item[f"{modality}_embeds"])
            if e.dim() != 2 or e.shape[1] != self.hidden:
                raise ValueError(f"{modality} embeddings must be [n, {self.hidden}], got {tuple(e.shape)}")
            return "embeds", int(e.shape[0]), e
        if isinstance(item, dict) and "pixel_values" in item:
            thw = item.get(f"{modality}_grid_thw", item.get("grid_thw"))
            if thw is None:
                raise ValueError("pixel inputs need their (t, h, w) patch grid")
            t, hh, ww = (int(x) for x in torch.as_tensor(thw).reshape(-1)[:3])
            pv = torch.as_tensor(item["pixel_values"])
            if pv.dim() != 2 or pv.shape[0] != t * hh * ww or hh % self.merge or ww % self.merge:
                raise ValueError(f"pixel_values must be [t*h*w, patch_dim] with h and w multiples of {self.merge}")
            return "pixels", t * hh * ww // (self.merge * self.merge), {"pixel_values": pv, "grid_thw": (t, hh, ww)}
        raise ValueError(f"unsupported {modality} item: pass embeddings [n, hidden] or {{'pixel_values': ..., '{modality}_grid_thw': ...}}")

    def apply(self, token_ids: list[int], mm_data: dict) -> ProcessedPrompt:
        items: dict[str, list] = {}
        for modality, v in (mm_data or {}).items():
            if modality not in self.placeholder_ids:
                raise ValueError(f"this model takes no {modality!r} inputs (known: {sorted(self.placeholder_ids)})")
            items[modality] = list(v) if isinstance(v, (list, tuple)) else [v]
        by_id = {tid: m for m, tid in self.placeholder_ids.items() if m in items}
        cursor = {m: 0 for m in items}
        out: list[int] = []
        feats: list[MultiModalFeature] = []
        for t in token_ids:
            m = by_id.get(t)
            if m is None:
                out.append(t)
                continue
            if cursor[m] >= len(items[m]):
                raise ValueError(f"the prompt has more {m} placeholders than items")
            item = items[m][cursor[m]]
            cursor[m] += 1
            kind, n, data = self.item_length(m, item)
            feats.append(MultiModalFeature(m, hash_item(m, data), len(out), n, kind, data))
            out.extend([t] * n)
        for m, c in cursor.items():
            if c != len(items[m]):
                raise ValueError(f"{len(items[m])} {m} items but {c} placeholders in the prompt")
        return ProcessedPrompt(out, feats)


def mrope_positions(num_tokens: int, features: list, merge: int = 2, t_step: float = 1.0):
    """(temporal, height, width) rotary positions of a prompt, ``int32 [3, num_tokens]``, and the offset that generated tokens add to
    their index. Text tokens carry the same running value in all three rows; an item with a patch grid ``(t, h, w)`` places its
    ``t * h/merge * w/merge`` positions on a grid starting at the running value, and the text after it continues from the largest
    coordinate used plus one. Items given as bare embeddings have no grid and count like text.
    (reference: model_executor/layers/rotary_embedding/mrope.py ``get_input_positions``; HF ``Qwen2VLModel.get_rope_index``)"""
    import numpy as np
    pos = np.zeros((3, num_tokens), dtype=np.int32)
    cursor, nxt = 0, 0
    for f in sorted(features or (), key=lambda x: x.offset):
        n_text = f.offset - cursor
        if n_text > 0:
            pos[:, cursor:f.offset] = nxt + np.arange(n_text, dtype=np.int32)
            nxt += n_text
        grid = f.data.get("grid_thw") if isinstance(f.data, dict) else None
        if grid is not None:
            t, gh, gw = int(grid[0]), int(grid[1]) // merge, int(grid[2]) // merge
            if t * gh * gw != f.length:
                raise ValueError(f"item at {f.offset}: grid {tuple(grid)} does not give {f.length} positions")
            ti = (np.arange(t, dtype=np.float64) * t_step).astype(np.int32)
            pos[0, f.offset:f.offset + f.length] = nxt + np.repeat(ti, gh * gw)
            pos[1, f.offset:f.offset + f.length] = nxt + np.tile(np.repeat(np.arange(gh, dtype=np.int32), gw), t)
            pos[2, f.offset:f.offset + f.length] = nxt + np.tile(np.arange(gw, dtype=np.int32), t * gh)
            nxt += max(int(ti[-1]) + 1, gh, gw)
        else:
            pos[:, f.offset:f.offset + f.length] = nxt + np.arange(f.length, dtype=np.int32)
            nxt += f.length
        cursor = f.offset + f.length
    if cursor < num_tokens:
        pos[:, cursor:] = nxt + np.arange(num_tokens - cursor, dtype=np.int32)
        nxt += num_tokens - cursor
    return pos, int(nxt - num_tokens)


class MultiModalRegistry:
    """Architecture → processor factory (reference: ``MULTIMODAL_REGISTRY.register_processor``)."""

    def __init__(self):
        self._factories: dict[str, Callable] = {}

    def register_processor(self, arch: str, factory: Callable) -> None:
        self._factories[arch] = factory

    def supports(self, model_config) -> bool:
        return bool(getattr(model_config, "mm_token_ids", None))

    def create_processor(self, model_config) -> Optional[MultiModalProcessor]:
        if not self.supports(model_config):
            return None
        f = self._factories.get(model_config.architecture)
        if f is not None:
            return f(model_config)
        return MultiModalProcessor(dict(model_config.mm_token_ids), model_config.hidden_size, getattr(model_config, "vision_merge_size", 2))


MULTIMODAL_REGISTRY = MultiModalRegistry()
