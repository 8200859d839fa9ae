"""Peer-memory tensor parallelism: symmetric slab, buffers and the fused reduce + residual + RMSNorm launch.

Each rank cudaMallocs one slab and maps every peer's slab through CUDA IPC handles exchanged over the bootstrap process
group (reference: the IPC buffer set-up of vllm/distributed/device_communicators/custom_all_reduce.py:100-261,726-759).
Slab layout, identical on every rank:

    part[parity][src]   bf16 [Tmax, H]   partial sums of source rank ``src``, written into this slab by that rank's GEMM epilogue
                                         (every rank for decode-sized batches, only the rows this rank owns for large ones)
    gather[0], gather[1] bf16 [Tmax, H]  two-shot mode: normalised rows pushed here by their owner ranks
    flags               int32 [2][2][tp][1024]   (parity, stage, source rank, CTA)
    arrive[3][src]      bf16 [Tl, H]     decode-sized batches: rotating arrival buffers of the flag-free one-shot reduction, filled
                                         with the "not here yet" value (bf16 -0.0); the words that say which buffer is in use live in
                                         ordinary device memory of each rank (every rank advances its own in step)

All addresses are fixed for the life of the process, so the kernels can be captured in CUDA graphs."""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from onecat_vllm import envs
from onecat_vllm.logger import init_logger

log = init_logger(__name__)
_MAXB = 1024
ONE_SHOT, TWO_SHOT, LAMPORT, NVLS = 0, 1, 2, 3
_LAM_BUFS = 3


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
        # flag-free path: rows per source and buffer (the one-shot regime of tp > 2 never exceeds 512 / (tp - 1) rows)
        self.lam_rows = min(tmax, 256)
        self.lam_src = self.lam_rows * hidden            # elements between sources
        self.lam_buf = tp * self.lam_src                 # elements between buffers
        self.off_lam = -(-(self.off_flags + self.flag_bytes) // 256) * 256
        self.bytes = self.off_lam + _LAM_BUFS * self.lam_buf * 2
        self.base = _C.comm_alloc(self.bytes)
        _C.comm_tensor(self.base, self.off_lam, [_LAM_BUFS * self.lam_buf], 0, device.index or 0).view(torch.int16).fill_(-32768)
        torch.cuda.synchronize(device)
        handle = _C.comm_export(self.base)
        handles = [None] * tp
        dist.all_gather_object(handles, handle, group=group)
        self.peers = []
        for r, h in enumerate(handles):
            self.peers.append(self.base if r == rank else _C.comm_import(h))
        self.seq = torch.zeros(_MAXB, dtype=torch.int32, device=device)
        self.lam_ctr = torch.zeros(2, dtype=torch.int32, device=device)  # [buffer in use, CTAs finished]
        self.use_lamport = envs.ONECAT_TP_ONESHOT != "flags"
        self.nvls_min_t = int(envs.ONECAT_TP_NVLS_MIN_T)
        self.full_residual = False
        self.parity = 0
        self.nvls_mode = {"1": "always", "0": "never"}.get(envs.ONECAT_TP_NVLS, "auto")
        # the switch only pays from four ranks up (see mode_for): below that the automatic policy never takes it, so nothing is set up
        want_nv = self.nvls_mode == "always" or (self.nvls_mode == "auto" and tp >= 4)
        self.nv = self._nvls_setup(tp, rank, device, buf, group) if want_nv else None
        self.wait_ns = int(envs.ONECAT_DEVICE_WAIT_LIMIT_MS) * 1_000_000
        self.num_sms = torch.cuda.get_device_properties(device).multi_processor_count
        self.launches = 0
        dist.barrier(group=group)
        log.info_once(f"fused TP: slab of {self.bytes >> 20} MiB mapped on {tp} ranks")

    def _nvls_setup(self, tp: int, rank: int, device, buf: int, group):
        """A second symmetric buffer, allocated and exchanged by ``torch.distributed._symmetric_memory`` and bound to an NVLink
        multicast object, for the reduction that adds inside the switch: ``part[parity]`` (this rank's partial sums), four rotating
        ``out`` and ``res`` buffers (normalised rows and new residual rows, broadcast by their owners; a result stays valid for the
        next three reductions) and the flag area. ``None`` when any rank has no multicast
        support (the peer-store kernels then serve every size)."""
        ok, nv = 0, None
        try:
            import torch.distributed._symmetric_memory as symm
            pg = group if group is not None else dist.group.WORLD
            flags = 2 * 2 * tp * _MAXB * 4
            t = symm.empty(10 * buf + flags, dtype=torch.uint8, device=device)
            t.zero_()
            torch.cuda.synchronize(device)
            hdl = symm.rendezvous(t, group=pg.group_name)
            mc = int(getattr(hdl, "multicast_ptr", 0) or 0)
            if mc and len(hdl.buffer_ptrs) == tp:
                nv = dict(t=t, hdl=hdl, mc=mc, ptrs=[int(x) for x in hdl.buffer_ptrs], part=[0, buf], out=[(2 + i) * buf for i in range(4)],
                          res=[(6 + i) * buf for i in range(4)], flags=10 * buf, slot=0)
                ok = 1
        except Exception as e:  # no symmetric-memory support in this build / on this machine
            log.info_once(f"fused TP: no switch reductions ({type(e).__name__}: {e})")
        flag = torch.tensor([ok], device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
        if int(flag.item()) != 1:
            return None
        log.info_once("fused TP: reductions inside the switch (multimem) enabled")
        return nv

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
        if self.mode_for(T) == NVLS:
            return self._nv_tensor(self.nv["part"][self.parity], T, H)
        return self._tensor(self.rank, self.off_part[self.parity][self.rank], T, H)

    def _nv_tensor(self, off: int, T: int, H: int) -> torch.Tensor:
        return self.nv["t"][off: off + T * H * 2].view(torch.bfloat16).view(T, H)

    def use_push(self, T: int) -> bool:
        """Whether the GEMM epilogue should push its tiles to the peers (overlapping the transfer with the GEMM) or leave them
        local for the reduction kernel to send or pull. Measured at TP2 / TP4: for decode-sized batches the flag-free reduction that
        sends the rows itself is faster (26.6 against 30.1 us at TP4, one token: the few CTAs of a small GEMM issue all peers'
        stores from their epilogue warps), for prefill-sized batches the push wins (478 against 543 us at 8192 tokens), so by default
        only batches of 512 tokens and more push. ``ONECAT_TP_PUSH`` = always | never | auto."""
        mode = envs.ONECAT_TP_PUSH
        if self.mode_for(T) == NVLS:
            return False   # the switch pulls the partial sums from where the GEMM left them
        return mode == "always" or (mode == "auto" and T >= 512)

    def push_spec(self, T: int):
        """Destinations for a row-parallel GEMM epilogue: slot ``[my rank]`` in every rank's slab. Decode-sized batches go to all
        ranks (each reduces everything itself; flag-free arrival buffers when enabled); large ones send each row only to the rank
        that owns it."""
        mode = self.mode_for(T)
        if mode == LAMPORT:
            off = self.off_lam + self.rank * self.lam_src * 2
            return [p + off for p in self.peers], 0, self.lam_ctr.data_ptr(), self.lam_buf
        off = self.off_part[self.parity][self.rank]
        dst = [p + off for p in self.peers]
        if mode == ONE_SHOT:
            return dst, 0
        return dst, -(-T // self.tp)

    def _in_slab(self, t: torch.Tensor) -> bool:
        return self.base + self.off_part[self.parity][self.rank] == t.data_ptr()

    def mode_for(self, T: int) -> int:
        if self.full_residual:   # somebody reads the residual stream between layers: every rank must hold all of its rows
            return LAMPORT if (self.use_lamport and T <= self.lam_rows) else ONE_SHOT
        one = T * (self.tp - 1) <= 1024 or self.tp == 2   # up to 1024 peer rows per rank: ~10 MB over NVLink, still cheaper than two phases
        if self.nv is not None and T >= self.nvls_min_t:
            # Measured at 8 ranks (hidden 5120, us per reduction): 64 rows 23.9 through the switch against 20.7 flag-free; 256 rows
            # 25.0 against 43.8 two-shot; 1024 rows 56.4 against 57.1; 8192 rows 325 against 268. At 2 ranks the switch never wins.
            if self.nvls_mode == "always" or (self.nvls_mode == "auto" and self.tp >= 4 and not one and T <= 512):
                return NVLS
        if one and self.use_lamport and T <= self.lam_rows:
            return LAMPORT
        return ONE_SHOT if one else TWO_SHOT

    # ---- the fused op
    def reduce_add_norm(self, partial: torch.Tensor, residual: Optional[torch.Tensor], w: Optional[torch.Tensor], eps: float = 1e-6,
                        gemma: bool = False, mode: Optional[int] = None, pushed: bool = False):
        T, H = partial.shape
        assert H == self.H and T <= self.tmax, "shape outside the symmetric slab"
        par = self.parity
        if mode is None or (mode == ONE_SHOT and self.mode_for(T) in (LAMPORT, NVLS)):
            mode = self.mode_for(T)
        if w is not None and w.dtype != torch.bfloat16:
            w = w.to(torch.bfloat16)
        from onecat_vllm.ops import cuda as K
        if mode == NVLS:
            nv = self.nv
            src = self._nv_tensor(nv["part"][par], T, H)
            if partial.data_ptr() != src.data_ptr():
                src.copy_(partial)
            slot = nv["slot"]
            nv["slot"] = (slot + 1) % 4
            x = self._nv_tensor(nv["out"][slot], T, H)
            res_out = self._nv_tensor(nv["res"][slot], T, H) if residual is not None else None
            part = [nv["mc"] + nv["part"][par]] + [0] * (self.tp - 1)
            xo = [nv["mc"] + nv["out"][slot], (nv["mc"] + nv["res"][slot]) if residual is not None else 0] + [0] * (self.tp - 2)
            flags = [p + nv["flags"] for p in nv["ptrs"]]
            grid = max(1, min(-(-T // self.tp), 2 * self.num_sms, _MAXB))
            self._C.tp_reduce_norm(part, flags, self.seq, xo, residual, None, w, T, H, self.rank, NVLS, gemma, par, eps, self.wait_ns, grid,
                                   [], 0, 0, 0, False)
            self.parity ^= 1
            self.launches += 1
            K._LAUNCHES += 1
            return x, res_out
        res_out = torch.empty(T, H, dtype=torch.bfloat16, device=self.device) if residual is not None else None
        if mode == LAMPORT:
            x = torch.empty(T, H, dtype=torch.bfloat16, device=self.device)
            xo = [0] * self.tp
            xo[self.rank] = x.data_ptr()
            part = [0] * self.tp
            if not pushed:
                if partial.stride(0) != H or partial.stride(1) != 1:
                    partial = partial.contiguous()
                part[self.rank] = partial.data_ptr()
            lam = [p + self.off_lam for p in self.peers]
            grid = min(T, 2 * self.num_sms, _MAXB)
            self._C.tp_reduce_norm(part, [0] * self.tp, self.seq, xo, residual, res_out, w, T, H, self.rank, mode, gemma, 0, eps, self.wait_ns, grid,
                                   lam, self.lam_buf, self.lam_src, self.lam_ctr.data_ptr(), bool(pushed))
            self.launches += 1
            K._LAUNCHES += 1
            return x, (res_out if residual is not None else None)
        if pushed and mode == self.mode_for(T):
            # every source's partial already sits in this rank's slab: the reduction reads local memory only
            part = [self.base + self.off_part[par][src] for src in range(self.tp)]
        else:
            if not self._in_slab(partial):
                self._tensor(self.rank, self.off_part[par][self.rank], T, H).copy_(partial)
            part = [p + self.off_part[par][src] for src, p in enumerate(self.peers)]  # pull each source's own slot
        flags = [p + self.off_flags for p in self.peers]
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
        self._C.tp_reduce_norm(part, flags, self.seq, xo, residual, res_out, w, T, H, self.rank, mode, gemma, par, eps, self.wait_ns, grid,
                               [], 0, 0, 0, False)
        self.parity ^= 1
        self.launches += 1
        K._LAUNCHES += 1
        return x, (res_out if residual is not None else None)

    def all_reduce(self, partial: torch.Tensor) -> torch.Tensor:
        x, _ = self.reduce_add_norm(partial, None, None, mode=ONE_SHOT, pushed=getattr(partial, "_tp_pushed", False))
        return x

    def close(self) -> None:
        if getattr(self, "base", None) is None:
            return
        torch.cuda.synchronize()
        self.nv = None
        for r, p in enumerate(self.peers):
            if r != self.rank:
                self._C.comm_unimport(p)
        self._C.comm_free(self.base)
        self.base = None
