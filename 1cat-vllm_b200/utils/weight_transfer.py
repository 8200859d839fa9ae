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


# ---- collective engine: the trainer is rank 0 of a dedicated process group, every inference worker another rank ---------------
class BroadcastWeightTransfer:
    """Weight hand-over across processes or nodes by broadcast over a process group of its own (NCCL between GPUs, gloo on CPU),
    in the reference's protocol: ``init`` joins the group, the trainer announces each update as a list of (name, dtype, shape), and
    the tensors follow packed into flat buffers of at most ``bucket_bytes`` per dtype, so one collective moves many small tensors
    (reference: distributed/weight_transfer/nccl_engine.py ``NCCLWeightTransferEngine``, packed_tensor.py; worker hooks
    gpu_worker.py:958-1110 ``init_weight_transfer_engine`` / ``update_weights``).

    Trainer (rank 0)::

        eng = BroadcastWeightTransfer.init("tcp://127.0.0.1:29600", rank=0, world_size=1 + num_workers, device=dev)
        eng.send(model.state_dict().items())

    Worker ``i`` (rank ``i + 1``): ``worker.init_weight_transfer(init_method, rank, world_size)`` once, then
    ``worker.update_weights_broadcast(meta)`` with the ``meta`` the trainer's ``describe`` returned (sent to the workers by any
    side channel, e.g. the engine's ``collective_rpc``, before the trainer calls ``send``)."""

    def __init__(self, group, device: torch.device, bucket_bytes: int = 256 << 20):
        self.group, self.device, self.bucket_bytes = group, device, bucket_bytes

    @classmethod
    def init(cls, init_method: str, rank: int, world_size: int, device, backend: str | None = None, timeout_s: float = 120.0,
             bucket_bytes: int = 256 << 20) -> "BroadcastWeightTransfer":
        import datetime

        import torch.distributed as dist
        from torch.distributed import rendezvous
        device = torch.device(device)
        backend = backend or ("nccl" if device.type == "cuda" else "gloo")
        # a store and a backend object of its own, outside torch.distributed's registry: the engine's default and tensor-parallel
        # groups (if any) stay untouched, and a trainer without any process group can still join
        store, r, w = next(rendezvous(init_method, rank, world_size, timeout=datetime.timedelta(seconds=timeout_s)))
        store.set_timeout(datetime.timedelta(seconds=timeout_s))
        prefix = dist.PrefixStore("onecat_weight_transfer", store)
        if backend == "nccl":
            torch.cuda.set_device(device)
            opts = dist.ProcessGroupNCCL.Options()
            opts._timeout = datetime.timedelta(seconds=timeout_s)
            pg = dist.ProcessGroupNCCL(prefix, r, w, opts)
        else:
            pg = dist.ProcessGroupGloo(prefix, r, w, datetime.timedelta(seconds=timeout_s))
        return cls(pg, device, bucket_bytes)

    def describe(self, named: Iterable[tuple[str, torch.Tensor]]) -> dict:
        """What the receivers need before the collective: the sender's bucket size (both sides must cut the same buckets) and the
        names, dtypes (as strings) and shapes in transfer order."""
        return {"bucket_bytes": self.bucket_bytes, "tensors": [(n, str(t.dtype).replace("torch.", ""), tuple(t.shape)) for n, t in named]}

    @staticmethod
    def _buckets(meta: dict):
        cur, size, dt0 = [], 0, None
        bucket_bytes = int(meta["bucket_bytes"])
        for n, dt, shape in meta["tensors"]:
            shape = tuple(shape)
            numel = 1
            for s in shape:
                numel *= s
            nbytes = numel * torch.empty((), dtype=getattr(torch, dt)).element_size()
            if cur and (dt != dt0 or size + nbytes > bucket_bytes):
                yield dt0, cur
                cur, size = [], 0
            dt0 = dt
            cur.append((n, shape, numel))
            size += nbytes
        if cur:
            yield dt0, cur

    def send(self, named: Iterable[tuple[str, torch.Tensor]]) -> dict:
        import torch.distributed as dist
        named = [(n, t.detach()) for n, t in named]
        meta = self.describe(named)
        by_name = dict(named)
        for dt, items in self._buckets(meta):
            flat = torch.empty(sum(k for _, _, k in items), dtype=getattr(torch, dt), device=self.device)
            o = 0
            for n, _shape, k in items:
                flat[o:o + k].copy_(by_name[n].reshape(-1))
                o += k
            self._bcast(flat)
        return meta

    def receive(self, meta: dict):
        """Yields (name, tensor) in transfer order; each tensor is a view of a bucket that is reused for the next one, so consume
        (copy) it before advancing."""
        import torch.distributed as dist
        for dt, items in self._buckets(meta):
            flat = torch.empty(sum(k for _, _, k in items), dtype=getattr(torch, dt), device=self.device)
            self._bcast(flat)
            o = 0
            for n, shape, k in items:
                yield n, flat[o:o + k].view(shape)
                o += k

    def _bcast(self, flat: torch.Tensor) -> None:
        import torch.distributed as dist
        opts = dist.BroadcastOptions()
        opts.rootRank = 0
        self.group.broadcast([flat], opts).wait()
        if flat.is_cuda:
            torch.cuda.current_stream(flat.device).synchronize()

    def close(self) -> None:
        self.group = None
