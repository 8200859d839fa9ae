"""Peer-memory tensor parallelism: symmetric slab, buffers and the fused reduce + residual + RMSNorm launch.

Each rank cudaMallocs one slab and maps every peer's slab through CUDA IPC handles exchanged over the bootstrap process
group (reference: the IPC buffer set-up of vllm/distributed/device_communicators/custom_all_reduce.py:100-261,726-759).
Slab layout, identical on every rank:

    part[parity][src]   bf16 [Tmax, H]   partial sums of source rank ``src``, written into this slab by that rank's GEMM epilogue
                                         (every rank for decode-sized batches, only the rows this rank owns for large ones)
    gather[0], gather[1] bf16 [Tmax, H]  two-shot mode: normalised rows pushed here by their owner ranks
    flags               int32 [2][2][tp][1024]   (parity, stage, source rank, CTA)

All addresses are fixed for the life of the process, so the kernels can be captured in CUDA graphs."""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from onecat_vllm import envs
from onecat_vllm.logger import init_logger

log = init_logger(__name__)
_MAXB = 1024
ONE_SHOT, TWO_SHOT = 0, 1


class FusedTP:
    def __init__(self, tp: int, rank: int, device: torch.device, tmax: int, hidden: int, group=None):
        from onecat_vllm.ops import _C
        self._C = _C
        self.tp, self.rank, self.device, self.tmax, self.H = tp, rank, device, tmax, hidden
        buf = tmax * hidden * 2
        buf = -(-buf // 256) * 256
        self.off_part = [[(par * tp + src) * buf for src in range(tp)] for par in range(2)]
        self.off_gather = [2 * tp * buf, (2 * tp + 1) * buf]
        self.off_flags = (2 * tp + 2) * buf
        self.flag_bytes = 2 * 2 * tp * _MAXB * 4
        self.bytes = self.off_flags + self.flag_bytes
        self.base = _C.comm_alloc(self.bytes)
        handle = _C.comm_export(self.base)
        handles = [None] * tp
        dist.all_gather_object(handles, handle, group=group)
        self.peers = []
        for r, h in enumerate(handles):
            self.peers.append(self.base if r == rank else _C.comm_import(h))
        self.seq = torch.zeros(_MAXB, dtype=torch.int32, device=device)
        self.parity = 0
        self.wait_ns = int(envs.ONECAT_DEVICE_WAIT_LIMIT_MS) * 1_000_000
        self.num_sms = torch.cuda.get_device_properties(device).multi_processor_count
        self.launches = 0
        dist.barrier(group=group)
        log.info_once(f"fused TP: slab of {self.bytes >> 20} MiB mapped on {tp} ranks")

    @classmethod
    def create(cls, cfg, device) -> "FusedTP":
        from onecat_vllm.parallel.state import get_state
        st = get_state()
        return cls(st.tp_size, st.tp_rank, device, cfg.scheduler_config.max_num_batched_tokens, cfg.model_config.hidden_size, st.tp_group)

    # ---- buffers
    def _tensor(self, rank: int, off: int, T: int, H: int) -> torch.Tensor:
        return self._C.comm_tensor(self.peers[rank], off, [T, H], 0, self.device.index or 0)

    def partial_buffer(self, T: int, H: int, dtype) -> Optional[torch.Tensor]:
        """This rank's own slot for the current reduction (what a GEMM without the push epilogue writes to)."""
        if H != self.H or T > self.tmax or dtype != torch.bfloat16:
            return None
        return self._tensor(self.rank, self.off_part[self.parity][self.rank], T, H)

    def use_push(self, T: int) -> bool:
        """Whether the GEMM epilogue should push its tiles to the peers (overlapping the transfer with the GEMM) or leave them
        local for the reduction kernel to pull. The epilogue's 64-byte row segments are a poor fit for NVLink at prefill sizes,
        so by default only decode-sized batches push. ``ONECAT_TP_PUSH`` = always | never | auto."""
        mode = envs.ONECAT_TP_PUSH
        return mode == "always" or (mode == "auto" and T <= 128)

    def push_spec(self, T: int):
        """Destinations for a row-parallel GEMM epilogue: slot ``[parity][my rank]`` in every rank's slab. Decode-sized batches go to
        all ranks (each reduces everything itself); large ones send each row only to the rank that owns it."""
        off = self.off_part[self.parity][self.rank]
        dst = [p + off for p in self.peers]
        if self.mode_for(T) == ONE_SHOT:
            return dst, 0
        return dst, -(-T // self.tp)

    def _in_slab(self, t: torch.Tensor) -> bool:
        return self.base + self.off_part[self.parity][self.rank] == t.data_ptr()

    def mode_for(self, T: int) -> int:
        return ONE_SHOT if T * (self.tp - 1) <= 512 or self.tp == 2 else TWO_SHOT

    # ---- the fused op
    def reduce_add_norm(self, partial: torch.Tensor, residual: Optional[torch.Tensor], w: Optional[torch.Tensor], eps: float = 1e-6,
                        gemma: bool = False, mode: Optional[int] = None, pushed: bool = False):
        T, H = partial.shape
        assert H == self.H and T <= self.tmax, "shape outside the symmetric slab"
        par = self.parity
        mode = self.mode_for(T) if mode is None else mode
        if pushed and mode == self.mode_for(T):
            # every source's partial already sits in this rank's slab: the reduction reads local memory only
            part = [self.base + self.off_part[par][src] for src in range(self.tp)]
        else:
            if not self._in_slab(partial):
                self._tensor(self.rank, self.off_part[par][self.rank], T, H).copy_(partial)
            part = [p + self.off_part[par][src] for src, p in enumerate(self.peers)]  # pull each source's own slot
        flags = [p + self.off_flags for p in self.peers]
        res_out = torch.empty(T, H, dtype=torch.bfloat16, device=self.device) if residual is not None else None
        if mode == ONE_SHOT:
            x = torch.empty(T, H, dtype=torch.bfloat16, device=self.device)
            xo = [0] * self.tp
            xo[self.rank] = x.data_ptr()
            grid = min(T, 2 * self.num_sms, _MAXB)
        else:
            x = self._tensor(self.rank, self.off_gather[par], T, H)
            xo = [p + self.off_gather[par] for p in self.peers]
            per = -(-T // self.tp)
            grid = max(1, min(per, 2 * self.num_sms, _MAXB))
        if w is not None and w.dtype != torch.bfloat16:
            w = w.to(torch.bfloat16)
        self._C.tp_reduce_norm(part, flags, self.seq, xo, residual, res_out, w, T, H, self.rank, mode, gemma, par, eps, self.wait_ns, grid)
        self.parity ^= 1
        self.launches += 1
        from onecat_vllm.ops import cuda as K
        K._LAUNCHES += 1
        return x, (res_out if residual is not None else None)

    def all_reduce(self, partial: torch.Tensor) -> torch.Tensor:
        x, _ = self.reduce_add_norm(partial, None, None, mode=ONE_SHOT)
        return x

    def close(self) -> None:
        if getattr(self, "base", None) is None:
            return
        torch.cuda.synchronize()
        for r, p in enumerate(self.peers):
            if r != self.rank:
                self._C.comm_unimport(p)
        self._C.comm_free(self.base)
        self.base = None
