"""Same-node weight hand-over for RLHF-style loops: the trainer shares its tensors through inter-process handles (CUDA IPC for
device tensors, shared memory for host tensors) and every worker loads them in place, without a checkpoint on disk
(reference: distributed/weight_transfer/ipc_engine.py, packed_tensor.py, base.py:49; worker side gpu_worker.py:987-1110).

Trainer::

    payload = pack_ipc(model.state_dict().items())          # names follow the HF checkpoint layout
    llm.collective_rpc("update_weights_ipc", args=(payload,))

``packed=True`` first copies all tensors of one dtype into one flat buffer, so a single handle crosses the process boundary per
dtype instead of one per tensor."""
from __future__ import annotations

import pickle
from typing import Iterable

import torch


def _handle(t: torch.Tensor):
    from torch.multiprocessing.reductions import reduce_tensor
    if not t.is_cuda:
        t.share_memory_()
    return reduce_tensor(t)


def pack_ipc(named: Iterable[tuple[str, torch.Tensor]], packed: bool = False) -> bytes:
    named = [(n, t.detach()) for n, t in named]
    if not packed:
        return pickle.dumps({"packed": False, "items": [(n, _handle(t.contiguous())) for n, t in named]})
    groups: dict = {}
    for n, t in named:
        groups.setdefault((t.dtype, t.device), []).append((n, t))
    out = []
    for (dt, dev), items in groups.items():
        flat = torch.empty(sum(t.numel() for _, t in items), dtype=dt, device=dev)
        meta, o = [], 0
        for n, t in items:
            flat[o:o + t.numel()].copy_(t.reshape(-1))
            meta.append((n, tuple(t.shape), o))
            o += t.numel()
        out.append((_handle(flat), meta))
    return pickle.dumps({"packed": True, "groups": out})


def unpack_ipc(payload: bytes) -> list[tuple[str, torch.Tensor]]:
    """Rebuild the shared tensors in this process. The tensors alias the sender's memory: copy out of them before the sender
    reuses it."""
    d = pickle.loads(payload)
    if not d["packed"]:
        return [(n, fn(*args)) for n, (fn, args) in d["items"]]
    out = []
    for (fn, args), meta in d["groups"]:
        flat = fn(*args)
        for n, shape, o in meta:
            numel = 1
            for s in shape:
                numel *= s
            out.append((n, flat[o:o + numel].view(shape)))
    return out
