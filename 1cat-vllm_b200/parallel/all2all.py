"""Expert-parallel token exchange ("all-to-all managers"): each rank routes the tokens it owns, rows travel to the ranks that hold
their experts, the expert outputs travel back and are summed per token with the routing weights.

Two managers share one interface, ``moe(layer, x_local, topk_w, topk_ids, t_off, T_total, gather) -> y_local``:

``PeerAll2All``   the product path on GPUs. One cudaMalloc slab per rank, mapped into every peer through CUDA IPC; rows are
                  stored straight into the owner's expert-major recv buffer by the dispatch kernel, the grouped tcgen05 GEMMs run
                  over that buffer as it lies, outputs are stored straight back into the sender's return buffer, and the combine
                  kernel can store the finished rows into every rank's gather buffer (all inside ``_C.fused_moe_a2a``;
                  bounded flag waits, no library collective).
``TorchAll2All``  ``torch.distributed.all_to_all_single`` with per-rank split sizes: the library baseline, the CPU (gloo) path and
                  the oracle of the peer path's tests.

(reference: vllm/distributed/device_communicators/all2all.py:84-137 ``AgRsAll2AllManager`` / DeepEP managers;
vllm/model_executor/layers/fused_moe/modular_kernel.py:1036-1684 prepare / finalize)"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from onecat_vllm import envs
from onecat_vllm.logger import init_logger
from onecat_vllm.ops import ref

log = init_logger(__name__)


def token_slice(T: int, n: int, rank: int) -> tuple[int, int]:
    """Rows ``[lo, hi)`` of a replicated ``[T, H]`` batch that ``rank`` routes (contiguous, earlier ranks take the remainder)."""
    base, rem = divmod(T, n)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


class TorchAll2All:
    """Library exchange: sort pairs by (owner rank, expert), all_to_all the per-expert counts, then the rows, run the local
    experts over what arrived, all_to_all the outputs back and combine."""

    def __init__(self, n: int, rank: int, group=None):
        self.n, self.rank, self.group = n, rank, group

    def moe(self, layer, x, topk_w, topk_ids, t_off: int = 0, T_total: Optional[int] = None, gather: bool = False):
        n, El, k = self.n, layer.E_local, topk_ids.shape[1]
        T, H = x.shape
        ids = topk_ids.reshape(-1).long()
        order = torch.argsort(ids, stable=True)                     # expert-major == owner-major (experts are contiguous per owner)
        sorted_ids = ids[order]
        send_counts = torch.bincount(sorted_ids, minlength=n * El).view(n, El)
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=self.group)
        in_split, out_split = recv_counts.sum(1).tolist(), send_counts.sum(1).tolist()
        rows = x[order // k].contiguous()
        recv = torch.empty(sum(in_split), H, dtype=x.dtype, device=x.device)
        dist.all_to_all_single(recv, rows, in_split, out_split, group=self.group)
        # recv holds, per source rank, that rank's rows in local-expert order
        e_of = torch.cat([torch.repeat_interleave(torch.arange(El, device=x.device), recv_counts[s]) for s in range(n)]) if recv.shape[0] else \
            torch.zeros(0, dtype=torch.long, device=x.device)
        out = self._experts(layer, recv, e_of)
        back = torch.empty(rows.shape[0], H, dtype=x.dtype, device=x.device)
        dist.all_to_all_single(back, out, out_split, in_split, group=self.group)
        ret = torch.empty_like(back)
        ret[order] = back                                            # back to pair order
        y = (ret.view(T, k, H).float() * topk_w.view(T, k, 1).float()).sum(1).to(x.dtype) if T else x.new_zeros(0, H)
        if not gather:
            return y
        return self._gather(y, T_total if T_total is not None else T)

    def _experts(self, layer, rows, e_of):
        w13, w2 = layer.dequantized()
        out = torch.empty_like(rows)
        for e in range(layer.E_local):
            sel = (e_of == e).nonzero().flatten()
            if sel.numel():
                h = ref.silu_and_mul(torch.nn.functional.linear(rows[sel].float(), w13[e].float()))
                out[sel] = torch.nn.functional.linear(h, w2[e].float()).to(rows.dtype)
        return out

    def _gather(self, y, T_total):
        sizes = [hi - lo for lo, hi in (token_slice(T_total, self.n, r) for r in range(self.n))]
        rows = max(max(sizes), 1)                                    # the library gathers equal shapes: pad to the longest slice
        mine = y.new_zeros(rows, y.shape[1])
        mine[: y.shape[0]] = y
        parts = [torch.empty_like(mine) for _ in range(self.n)]
        dist.all_gather(parts, mine, group=self.group)
        return torch.cat([p[:sz] for p, sz in zip(parts, sizes)], 0)

    def close(self):
        pass


class PeerAll2All:
    """Peer-memory exchange. ``max_tokens`` bounds the tokens of one step over all ranks; the recv buffer is sized for the worst
    case (every pair of every rank routed to one rank), so no routing pattern can overflow it."""

    def __init__(self, n: int, rank: int, device: torch.device, max_tokens: int, hidden: int, num_experts: int, top_k: int, group=None):
        from onecat_vllm.ops import _C
        self._C, self.n, self.rank, self.device, self.H, self.E, self.k = _C, n, rank, device, hidden, num_experts, top_k
        assert num_experts % n == 0 and num_experts <= 1024 and n <= 8
        self.max_tokens = max_tokens
        self.t_local_max = -(-max_tokens // n)
        self.cap = max_tokens * min(top_k, num_experts // n)
        self.ret_rows = self.t_local_max * top_k

        def up(v):
            return -(-v // 256) * 256
        self.off_counts = 0
        self.off_flags = up(n * num_experts * 4)
        self.off_recv_x = self.off_flags + up(4 * 8 * 4)
        self.off_recv_meta = self.off_recv_x + up(self.cap * hidden * 2)
        self.off_ret = self.off_recv_meta + up(self.cap * 4)
        self.off_gather = self.off_ret + up(self.ret_rows * hidden * 2)
        self.bytes = self.off_gather + up(max_tokens * hidden * 2)
        self.base = _C.comm_alloc(self.bytes)
        _C.comm_tensor(self.base, 0, [self.off_recv_x], 2, device.index or 0).zero_()   # counts and flags start at zero
        torch.cuda.synchronize(device)
        handles = [None] * n
        dist.all_gather_object(handles, _C.comm_export(self.base), group=group)
        self.peers = [self.base if r == rank else _C.comm_import(h) for r, h in enumerate(handles)]
        self.state = torch.zeros(8 + 2 * num_experts, dtype=torch.int32, device=device)
        self.wait_ns = int(envs.ONECAT_DEVICE_WAIT_LIMIT_MS) * 1_000_000
        dist.barrier(group=group)
        log.info_once(f"expert-parallel exchange: slab of {self.bytes >> 20} MiB mapped on {n} ranks")

    def moe(self, layer, x, topk_w, topk_ids, t_off: int = 0, T_total: Optional[int] = None, gather: bool = False):
        from onecat_vllm.ops import cuda as K
        ks = layer.kernel_state
        assert ks is not None, "the peer exchange runs the grouped tcgen05 GEMMs: experts must be prepared for them"
        T = x.shape[0]
        T_total = T_total if T_total is not None else self.max_tokens
        assert T_total <= self.max_tokens and T <= self.t_local_max and x.shape[1] == self.H
        if T and (x.stride(-1) != 1 or (x.stride(0) * 2) % 16):
            x = x.contiguous()
        ws = K.workspace(x.device)
        K._LAUNCHES += 9
        y = self._C.fused_moe_a2a(x, ks["w13"], ks["w2"], topk_w.contiguous().float(), topk_ids.contiguous().to(torch.int32), layer.E_local,
                                  ws.counters, ks.get("wkind", 0), ks.get("w13_sz"), ks.get("w2_sz"), ks.get("I2", 0), ks.get("gk", 1),
                                  self.peers, [self.off_counts, self.off_flags, self.off_recv_x, self.off_recv_meta, self.off_ret, self.off_gather],
                                  self.state, self.rank, self.cap, self.ret_rows, T_total, t_off, gather, self.wait_ns)
        if not gather:
            return y
        return self._C.comm_tensor(self.base, self.off_gather, [T_total, self.H], 0, self.device.index or 0)

    def close(self):
        if getattr(self, "base", None) is None:
            return
        torch.cuda.synchronize()
        for r, p in enumerate(self.peers):
            if r != self.rank:
                self._C.comm_unimport(p)
        self._C.comm_free(self.base)
        self.base = None


def create(cfg, device, group=None):
    """The manager for this process: the peer path on GPUs unless ``ONECAT_EP_A2A=torch``."""
    from onecat_vllm.parallel.state import get_state
    st = get_state()
    mc = cfg.model_config
    if device.type == "cuda" and envs.ONECAT_EP_A2A != "torch":
        return PeerAll2All(st.ep_size, st.ep_rank, device, cfg.scheduler_config.max_num_batched_tokens, mc.hidden_size, mc.num_experts,
                           mc.num_experts_per_tok, group if group is not None else st.tp_group)
    log.info_once(f"expert-parallel exchange: torch.distributed all_to_all on {st.ep_size} ranks")
    return TorchAll2All(st.ep_size, st.ep_rank, group if group is not None else st.tp_group)
