"""Expert-parallel load balancing: measure how many tokens each expert receives, re-place (and replicate) experts so that the ranks
carry equal load, and move the expert weights accordingly
(reference: vllm/distributed/eplb/eplb_state.py ``EplbState`` — sliding load window, rearrangement every N steps;
eplb/policy/default.py ``rebalance_experts`` — replicate the hottest experts, then pack onto ranks;
eplb/rebalance_execute.py ``rearrange_expert_weights_inplace`` — P2P shuffles).

Vocabulary: a model has ``E`` *logical* experts per layer; the deployment has ``P >= E`` *physical* slots per layer, ``P / ranks`` on
each rank; ``phy2log[l, p]`` says which logical expert slot ``p`` holds, and a logical expert with several slots (replicas) has its
tokens spread over them."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch


def replicate_experts(load: torch.Tensor, num_phy: int) -> tuple[torch.Tensor, torch.Tensor]:
    """``load [E]`` → ``(phy2log [num_phy], replicas [E])``: every expert gets one slot, each further slot goes to the expert whose load
    per replica is currently highest."""
    E = load.numel()
    assert num_phy >= E
    phy2log = list(range(E))
    cnt = torch.ones(E, dtype=torch.int64)
    lf = load.double().clamp_min(0)
    for _ in range(num_phy - E):
        e = int(torch.argmax(lf / cnt.double()))
        phy2log.append(e)
        cnt[e] += 1
    return torch.tensor(phy2log, dtype=torch.int64), cnt


def pack_balanced(weights: torch.Tensor, num_bins: int) -> torch.Tensor:
    """Longest-processing-time packing of ``len(weights)`` items into ``num_bins`` bins of equal *count*: returns the bin of each item."""
    n = weights.numel()
    assert n % num_bins == 0
    cap = n // num_bins
    order = torch.argsort(weights.double(), descending=True).tolist()
    fill, tot = [0] * num_bins, [0.0] * num_bins
    out = torch.empty(n, dtype=torch.int64)
    for i in order:
        b = min((k for k in range(num_bins) if fill[k] < cap), key=lambda k: tot[k])
        out[i] = b
        fill[b] += 1
        tot[b] += float(weights[i])
    return out


def rebalance_experts(load: torch.Tensor, num_phy: int, num_ranks: int) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """``load [L, E]`` → ``(phy2log [L, P], log2phy [L, E, max_rep] (-1 padded), logcnt [L, E])``. Slots ``r*P/R .. (r+1)*P/R - 1`` live
    on rank ``r``."""
    L, E = load.shape
    assert num_phy % num_ranks == 0
    per = num_phy // num_ranks
    phy2log = torch.empty(L, num_phy, dtype=torch.int64)
    logcnt = torch.empty(L, E, dtype=torch.int64)
    for l in range(L):
        p2l, cnt = replicate_experts(load[l], num_phy)
        w = load[l].double()[p2l] / cnt.double()[p2l]          # load each physical slot will see
        bins = pack_balanced(w, num_ranks)
        placed = torch.empty(num_phy, dtype=torch.int64)
        nxt = [r * per for r in range(num_ranks)]
        for i in range(num_phy):
            placed[nxt[int(bins[i])]] = p2l[i]
            nxt[int(bins[i])] += 1
        phy2log[l], logcnt[l] = placed, cnt
    mr = int(logcnt.max())
    log2phy = torch.full((L, E, mr), -1, dtype=torch.int64)
    for l in range(L):
        k = [0] * E
        for p in range(num_phy):
            e = int(phy2log[l, p])
            log2phy[l, e, k[e]] = p
            k[e] += 1
    return phy2log, log2phy, logcnt


def map_to_physical(topk_ids: torch.Tensor, log2phy_l: torch.Tensor, logcnt_l: torch.Tensor) -> torch.Tensor:
    """Logical expert ids ``[T, k]`` of one layer → physical slot ids: token ``t`` uses replica ``t mod replicas`` of each of its
    experts, which spreads a hot expert's tokens evenly over its slots without any communication."""
    T = topk_ids.shape[0]
    ids = topk_ids.long()
    rep = torch.arange(T, device=ids.device).unsqueeze(1) % logcnt_l.to(ids.device)[ids]
    return log2phy_l.to(ids.device)[ids, rep]


@dataclass
class EplbConfig:
    window_size: int = 1000          # steps of load history
    step_interval: int = 3000        # rearrange every this many steps
    num_redundant_experts: int = 0   # P - E


class EplbState:
    """Per-model bookkeeping: a sliding window of per-layer expert token counts and the current placement."""

    def __init__(self, num_layers: int, num_experts: int, num_ranks: int, cfg: Optional[EplbConfig] = None):
        self.cfg = cfg or EplbConfig()
        self.L, self.E, self.R = num_layers, num_experts, num_ranks
        self.P = num_experts + self.cfg.num_redundant_experts
        assert self.P % num_ranks == 0, "physical experts must divide evenly over the ranks"
        self.window = torch.zeros(self.cfg.window_size, num_layers, num_experts, dtype=torch.int64)
        self.cursor = 0
        self.steps = 0
        self.phy2log, self.log2phy, self.logcnt = rebalance_experts(torch.ones(num_layers, num_experts), self.P, num_ranks)

    def record(self, layer: int, topk_ids: torch.Tensor) -> None:
        """Count this step's routed tokens of one layer (logical ids)."""
        self.window[self.cursor, layer] += torch.bincount(topk_ids.reshape(-1).long().cpu(), minlength=self.E)[: self.E]

    def step(self) -> bool:
        """Advance the window; True when a rearrangement is due."""
        self.steps += 1
        self.cursor = (self.cursor + 1) % self.cfg.window_size
        self.window[self.cursor].zero_()
        return self.steps % self.cfg.step_interval == 0

    def load(self) -> torch.Tensor:
        return self.window.sum(0)

    def balancedness(self, load: Optional[torch.Tensor] = None) -> float:
        """mean / max of the per-rank load under the current placement (1.0 = perfectly even)."""
        load = self.load().double() if load is None else load.double()
        per = self.P // self.R
        slot = load.gather(1, self.phy2log) / self.logcnt.double().gather(1, self.phy2log)
        rank = slot.view(self.L, self.R, per).sum(-1)
        return float((rank.mean(1) / rank.max(1).values.clamp_min(1e-9)).mean())

    def plan(self) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        return rebalance_experts(self.load().clamp_min(1), self.P, self.R)


def rearrange_expert_weights(old_phy2log: torch.Tensor, new_phy2log: torch.Tensor, weights: list[list[torch.Tensor]], rank: int, num_ranks: int,
                             group=None) -> None:
    """Move expert weights in place so that this rank's local slots hold ``new_phy2log``. ``weights[l]`` is the list of this rank's
    stacked expert tensors of layer ``l`` (each ``[P/R, ...]``). A slot whose new expert is already on this rank is copied locally;
    otherwise it is received from the lowest rank that held the expert, which sends it (point-to-point, batched per layer)."""
    import torch.distributed as dist
    L, P = old_phy2log.shape
    per = P // num_ranks
    for l in range(L):
        old, new = old_phy2log[l].tolist(), new_phy2log[l].tolist()
        src_of = {}
        for p, e in enumerate(old):
            src_of.setdefault(e, p)                      # lowest slot (hence lowest rank) that holds each expert
        snap = [w.clone() for w in weights[l]]           # sources are read from the old contents
        ops, recv_into = [], []
        for p in range(P):
            e = new[p]
            dst_rank, sp = p // per, src_of[e]
            local_here = next((q for q in range(rank * per, (rank + 1) * per) if old[q] == e), None)
            if dst_rank == rank:
                if local_here is not None:
                    for w, s in zip(weights[l], snap):
                        w[p - rank * per].copy_(s[local_here - rank * per])
                else:
                    for wi, w in enumerate(weights[l]):
                        buf = torch.empty_like(w[p - rank * per])
                        ops.append(dist.P2POp(dist.irecv, buf, sp // per, group=group, tag=0))
                        recv_into.append((w, p - rank * per, buf))
            elif sp // per == rank:
                # some other rank needs expert e and this rank is its designated source — unless that rank has a copy of its own
                if not any(old[q] == e for q in range(dst_rank * per, (dst_rank + 1) * per)):
                    for s in snap:
                        ops.append(dist.P2POp(dist.isend, s[sp - rank * per].contiguous(), dst_rank, group=group, tag=0))
        if ops:
            for r in dist.batch_isend_irecv(ops):
                r.wait()
        for w, i, buf in recv_into:
            w[i].copy_(buf)
