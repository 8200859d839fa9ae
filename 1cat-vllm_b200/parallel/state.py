"""Process-group bookkeeping for one-process-per-GPU execution.

The reference builds world/TP/PP/DP/EP ``GroupCoordinator`` objects on top of ``torch.distributed``
(reference: vllm/distributed/parallel_state.py:408,1617,1753-1994). Here a rank's coordinates are plain
integers; ``torch.distributed`` (NCCL on GPUs, gloo on CPU) carries the bootstrap and the baseline
collectives, and the hot tensor-parallel path goes through the peer-memory kernels in
``onecat_vllm.parallel.fused``.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist


@dataclass
class ParallelState:
    rank: int = 0
    world_size: int = 1
    tp_rank: int = 0
    tp_size: int = 1
    pp_rank: int = 0
    pp_size: int = 1
    ep_rank: int = 0
    ep_size: int = 1
    dcp_rank: int = 0
    dcp_size: int = 1
    tp_group: Optional[object] = None
    pp_group: Optional[object] = None
    cpu_group: Optional[object] = None
    tp_comm: str = "fused"
    fused: Optional[object] = None  # onecat_vllm.parallel.fused.FusedTP once the symmetric heap exists
    ep_a2a: Optional[object] = None  # onecat_vllm.parallel.all2all manager when experts exchange tokens instead of partial sums

    @property
    def is_first_pp(self) -> bool:
        return self.pp_rank == 0

    @property
    def is_last_pp(self) -> bool:
        return self.pp_rank == self.pp_size - 1


_STATE = ParallelState()


def get_state() -> ParallelState:
    return _STATE


def tp_size() -> int:
    return _STATE.tp_size


def tp_rank() -> int:
    return _STATE.tp_rank


def rank_layout(rank: int, tp: int, pp: int) -> tuple[int, int]:
    """rank → (tp_rank, pp_rank); TP ranks are contiguous (reference: parallel_state.py:1836-1910)."""
    return rank % tp, rank // tp


def pp_layer_range(num_layers: int, pp_rank: Optional[int] = None, pp_size: Optional[int] = None) -> tuple[int, int]:
    """Contiguous slice of decoder layers owned by a pipeline stage; earlier stages take the remainder
    (reference: model_executor/models/utils.py ``get_pp_indices``)."""
    pp_rank = _STATE.pp_rank if pp_rank is None else pp_rank
    pp_size = _STATE.pp_size if pp_size is None else pp_size
    base, rem = divmod(num_layers, pp_size)
    start = pp_rank * base + min(pp_rank, rem)
    return start, start + base + (1 if pp_rank < rem else 0)


def pp_neighbor(delta: int) -> int:
    """Global rank of the stage ``delta`` steps away that holds the same tensor-parallel shard."""
    return (_STATE.pp_rank + delta) * _STATE.tp_size + _STATE.tp_rank


def init_distributed(rank: int, world_size: int, tp: int, pp: int = 1, backend: Optional[str] = None,
                     init_method: Optional[str] = None, enable_ep: bool = False, dcp: int = 1, tp_comm: str = "fused",
                     timeout_s: float = 600.0) -> ParallelState:
    global _STATE
    assert world_size == tp * pp, "world_size must equal tp * pp"
    tpr, ppr = rank_layout(rank, tp, pp)
    st = ParallelState(rank, world_size, tpr, tp, ppr, pp, tpr if enable_ep else 0, tp if enable_ep else 1,
                       tpr % dcp, dcp, tp_comm=tp_comm)
    if world_size > 1:
        if not dist.is_initialized():
            import datetime
            backend = backend or ("nccl" if torch.cuda.is_available() else "gloo")
            kw = dict(backend=backend, rank=rank, world_size=world_size, timeout=datetime.timedelta(seconds=timeout_s))
            if init_method:
                kw["init_method"] = init_method
            if backend == "nccl":
                kw["device_id"] = torch.device("cuda", torch.cuda.current_device())
            dist.init_process_group(**kw)
        for p in range(pp):
            ranks = list(range(p * tp, (p + 1) * tp))
            g = dist.new_group(ranks) if (tp > 1 and pp > 1) else (dist.group.WORLD if tp > 1 else None)
            if p == ppr:
                st.tp_group = g
        if pp > 1:
            for t in range(tp):
                g = dist.new_group([t + p * tp for p in range(pp)])
                if t == tpr:
                    st.pp_group = g
    _STATE = st
    return st


def destroy_distributed() -> None:
    global _STATE
    for mgr in (_STATE.ep_a2a, _STATE.fused):
        if mgr is not None:
            try:
                mgr.close()
            except Exception:
                pass
    if dist.is_initialized():
        try:
            if torch.cuda.is_available() and dist.get_backend() == "nccl":
                torch.cuda.synchronize()
            dist.destroy_process_group()
        except Exception:
            pass
    _STATE = ParallelState()


# ---- baseline collectives (library path; the fused kernels replace these on the hot path)
def all_reduce(x: torch.Tensor) -> torch.Tensor:
    if _STATE.tp_size > 1:
        dist.all_reduce(x, group=_STATE.tp_group)
    return x


def all_gather_last_dim(x: torch.Tensor) -> torch.Tensor:
    if _STATE.tp_size == 1:
        return x
    outs = [torch.empty_like(x) for _ in range(_STATE.tp_size)]
    dist.all_gather(outs, x.contiguous(), group=_STATE.tp_group)
    return torch.cat(outs, dim=-1)


def broadcast_object(obj, src: int = 0):
    if _STATE.world_size == 1:
        return obj
    lst = [obj]
    dist.broadcast_object_list(lst, src=src)
    return lst[0]
