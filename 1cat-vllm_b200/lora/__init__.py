"""Multi-LoRA serving: adapters loaded from PEFT checkpoints, kept in an LRU of ``max_loras`` slots on the worker, and applied per
token inside the linear layers (reference: vllm/lora/request.py, lora/model_manager.py:64 ``LoRAModelManager``,
lora/worker_manager.py:25, lora/layers/*, lora/punica_wrapper/punica_gpu.py:33 shrink / expand over a token → adapter map).

A step's batch may mix requests of different adapters and of none. The runner publishes a ``LoRABatch`` (token → slot) for the step;
every ``LinearBase.forward`` that has adapter weights adds, per active slot, ``scale * (x_s A^T) B^T`` to the rows of that slot's
tokens. The two small GEMMs per slot go through the library GEMM (rank ≤ 64): they are not on the critical path of the
named benchmarks. Stacked layers (qkv, gate|up) keep one (A, B) pair per sub-projection and add into that projection's
output columns. Under tensor parallelism each rank holds the matching slice of B (column-parallel layers) or of A (row-parallel
layers)."""
from __future__ import annotations

import json
import os
from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Optional

import torch


@dataclass(frozen=True)
class LoRARequest:
    lora_name: str
    lora_int_id: int
    lora_path: str = ""

    def to_dict(self) -> dict:
        return {"lora_name": self.lora_name, "lora_int_id": self.lora_int_id, "lora_path": self.lora_path}

    @classmethod
    def from_dict(cls, d: Optional[dict]) -> Optional["LoRARequest"]:
        return None if not d else cls(d["lora_name"], int(d["lora_int_id"]), d.get("lora_path", ""))


@dataclass
class LoRABatch:
    """Token → adapter slot for one model step (``-1`` = no adapter)."""

    token_slot: torch.Tensor                       # [T] int64
    rows_of: dict = field(default_factory=dict)    # slot -> index tensor of its token rows


_ACTIVE: Optional[LoRABatch] = None


def set_active(batch: Optional[LoRABatch]) -> None:
    global _ACTIVE
    _ACTIVE = batch


def active() -> Optional[LoRABatch]:
    return _ACTIVE


# checkpoint sub-module → (our stacked module, index of the sub-projection)
_STACKED = {"q_proj": ("qkv_proj", 0), "k_proj": ("qkv_proj", 1), "v_proj": ("qkv_proj", 2), "gate_proj": ("gate_up_proj", 0),
            "up_proj": ("gate_up_proj", 1)}


@dataclass
class _Pair:
    a: torch.Tensor   # [r, in]
    b: torch.Tensor   # [out_i, r], already multiplied by alpha / r
    col0: int         # first output column of the sub-projection inside the layer's output


def apply_lora(layer, x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    """Add the active adapters' deltas to ``y`` (the layer's base output for inputs ``x``)."""
    batch = _ACTIVE
    slots = getattr(layer, "lora_slots", None)
    if batch is None or not slots:
        return y
    for slot, rows in batch.rows_of.items():
        pairs = slots.get(slot)
        if not pairs:
            continue
        xs = x.index_select(0, rows)
        for p in pairs:
            d = (xs @ p.a.t()) @ p.b.t()
            y[:, p.col0:p.col0 + p.b.shape[0]].index_add_(0, rows, d.to(y.dtype))
    return y


class LoRAManager:
    """Worker-side adapter store: slot assignment, loading, LRU eviction."""

    def __init__(self, model: torch.nn.Module, max_loras: int, max_rank: int, device, dtype):
        self.model, self.max_loras, self.max_rank, self.device, self.dtype = model, max_loras, max_rank, device, dtype
        self.slot_of: "OrderedDict[int, int]" = OrderedDict()   # lora id -> slot, in LRU order
        self.names: dict[int, str] = {}
        self.mods = dict(model.named_modules())

    def list_loras(self) -> list[int]:
        return list(self.slot_of)

    def slot(self, req: LoRARequest) -> int:
        """Slot of an adapter, loading it (and evicting the least recently used one) if needed."""
        if req.lora_int_id in self.slot_of:
            self.slot_of.move_to_end(req.lora_int_id)
            return self.slot_of[req.lora_int_id]
        if len(self.slot_of) >= self.max_loras:
            old, s = next(iter(self.slot_of.items()))
            self.remove_lora(old)
        used = set(self.slot_of.values())
        s = next(i for i in range(self.max_loras) if i not in used)
        self._load(req, s)
        self.slot_of[req.lora_int_id] = s
        self.names[req.lora_int_id] = req.lora_name
        return s

    def add_lora(self, req: LoRARequest) -> bool:
        self.slot(req)
        return True

    def remove_lora(self, lora_id: int) -> bool:
        s = self.slot_of.pop(lora_id, None)
        self.names.pop(lora_id, None)
        if s is None:
            return False
        for m in self.mods.values():
            sl = getattr(m, "lora_slots", None)
            if sl:
                sl.pop(s, None)
        return True

    # ---- loading a PEFT adapter directory: adapter_config.json + adapter_model.safetensors (or .bin)
    def _load(self, req: LoRARequest, slot: int) -> None:
        path = req.lora_path
        with open(os.path.join(path, "adapter_config.json")) as f:
            cfg = json.load(f)
        r, alpha = int(cfg["r"]), float(cfg.get("lora_alpha", cfg["r"]))
        if r > self.max_rank:
            raise ValueError(f"adapter rank {r} exceeds max_lora_rank={self.max_rank}")
        st = os.path.join(path, "adapter_model.safetensors")
        if os.path.exists(st):
            from safetensors.torch import load_file
            tensors = load_file(st)
        else:
            tensors = torch.load(os.path.join(path, "adapter_model.bin"), map_location="cpu", weights_only=True)
        scale = alpha / r
        found: dict = {}
        for name, w in tensors.items():
            # base_model.model.model.layers.3.self_attn.q_proj.lora_A.weight
            n = name
            for pre in ("base_model.model.", "base_model."):
                if n.startswith(pre):
                    n = n[len(pre):]
                    break
            if ".lora_A" in n:
                mod, which = n.split(".lora_A")[0], "a"
            elif ".lora_B" in n:
                mod, which = n.split(".lora_B")[0], "b"
            else:
                continue
            found.setdefault(mod, {})[which] = w
        n_applied = 0
        for mod, ab in found.items():
            if "a" not in ab or "b" not in ab:
                continue
            parent, leaf = mod.rsplit(".", 1)
            target, sub = (parent + "." + _STACKED[leaf][0], _STACKED[leaf][1]) if leaf in _STACKED else (mod, 0)
            layer = self.mods.get(target)
            if layer is None or not hasattr(layer, "local_output_sizes"):
                continue  # a module this model does not have (or one on another pipeline stage)
            if getattr(layer, "fuse_silu_mul", False):
                raise ValueError("this model was built without enable_lora: its gate|up projection applies SiLU·mul in the GEMM epilogue")
            col0 = sum(layer.local_output_sizes[:sub])
            a, b = ab["a"], ab["b"]
            # tensor parallelism: a column-parallel layer keeps this rank's rows of B (its slice of the sub-projection's outputs); a
            # row-parallel layer keeps this rank's columns of A, and its delta is a partial sum that joins the layer's reduction
            if layer.tp > 1 and layer.parallel == "column" and layer.segment_tp[sub] > 1:
                loc = layer.local_output_sizes[sub]
                b = b.narrow(0, layer._segment_rank(sub) * loc, loc)
            elif layer.tp > 1 and layer.parallel == "row":
                a = a.narrow(1, layer.tp_rank * layer.in_features, layer.in_features)
            a = a.to(self.device, self.dtype).contiguous()
            b = (b.float() * scale).to(self.device, self.dtype).contiguous()
            if a.shape[1] != layer.in_features or b.shape[0] != layer.local_output_sizes[sub]:
                raise ValueError(f"adapter tensor shapes for {mod} do not match the layer ({tuple(a.shape)}, {tuple(b.shape)})")
            if not hasattr(layer, "lora_slots") or layer.lora_slots is None:
                layer.lora_slots = {}
            layer.lora_slots.setdefault(slot, []).append(_Pair(a, b, col0))
            n_applied += 1
        if n_applied == 0:
            raise ValueError(f"adapter at {path} has no tensors for this model")

    # ---- per step
    def make_batch(self, token_reqs: list, device) -> Optional[LoRABatch]:
        """``token_reqs``: per token the ``LoRARequest`` of its request or ``None``."""
        if not any(r is not None for r in token_reqs):
            return None
        slot_cache: dict = {}
        ids = []
        for r in token_reqs:
            if r is None:
                ids.append(-1)
            else:
                if r.lora_int_id not in slot_cache:
                    slot_cache[r.lora_int_id] = self.slot(r)
                ids.append(slot_cache[r.lora_int_id])
        t = torch.tensor(ids, dtype=torch.long, device=device)
        rows = {s: (t == s).nonzero(as_tuple=True)[0] for s in set(slot_cache.values())}
        return LoRABatch(t, rows)
