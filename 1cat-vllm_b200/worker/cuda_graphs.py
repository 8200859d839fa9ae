"""CUDA graphs for uniform decode batches (reference: vllm/v1/cudagraph_dispatcher.py:141,272-359;
compilation/cuda_graph.py:147,268; capture sizes config/vllm.py:2084-2200).

A graph is keyed by (padded request count, tokens per request, KV-split count). Batches are padded up to the next
captured size; the split count follows the live context length in power-of-two buckets, so short contexts never
launch a grid sized for the longest one (the reference's context-bucketed graphs). All inputs live in the runner's
persistent device buffers, so replay needs no pointer patching."""
from __future__ import annotations

import bisect
from typing import Optional

import torch

from onecat_vllm.logger import init_logger
from onecat_vllm.worker.attn_metadata import AttentionMetadata

log = init_logger(__name__)


class DecodeGraphs:
    def __init__(self, runner):
        self.r = runner
        sc = runner.cfg.scheduler_config
        self.sizes = [s for s in sc.graph_capture_sizes() if s <= max(sc.max_num_seqs, 1)]
        if not self.sizes or self.sizes[-1] < sc.max_num_seqs:
            self.sizes.append(sc.max_num_seqs)
        self.graphs: dict = {}
        self.pool = None
        self.stream = torch.cuda.Stream()
        mc = runner.mc
        from onecat_vllm.ops import cuda as K
        layers = [l for l in runner.model.model.layers if l.kind == "full_attention"]
        mla = [l for l in runner.model.model.layers if l.kind == "mla"]
        self.attn_layers = layers
        self.max_q = 1 + runner.num_spec
        tmax = self.sizes[-1] * self.max_q
        # geometry that sizes the split-KV grid and workspace: (query heads, KV heads, head size); MLA runs all heads of a request
        # against one latent "head" of 512
        self.geom = None
        if layers:
            a = layers[0].self_attn
            self.geom = (a.Hq, a.Hkv, a.D)
            K.workspace(runner.device).attn_static(32 * tmax * a.Hq * a.D, 32 * tmax * a.Hq * 2)
        elif mla:
            a = mla[0].self_attn
            self.geom = ("mla", a.H, 512)
            K.workspace(runner.device).attn_static(32 * tmax * a.H * 512, 32 * tmax * a.H * 2)
        # every mixer's decode path runs without host synchronisation on fixed addresses (attention, latent attention, Gated-DeltaNet
        # with its state slots; fused mixture-of-experts builds its work list on the device). What stays eager: experts that run the
        # per-expert loop (biased / clamped activations), pipeline stages, and anything without an attention geometry.
        kinds_ok = all(l.kind in ("full_attention", "linear_attention", "mla") and getattr(l, "graph_safe", True) for l in runner.model.model.layers)
        moe_ok = all(getattr(getattr(l.mlp, "experts", None), "kernel_state", True) is not None for l in runner.model.model.layers if hasattr(l, "mlp"))
        self.eligible = kinds_ok and moe_ok and self.geom is not None
        self.hits = self.misses = 0

    def plan(self, R: int, q: int, max_seq: int) -> Optional[tuple]:
        """Returns (padded R, q, splits) or None when the batch must run eagerly."""
        if not self.eligible or R > self.sizes[-1] or q > self.max_q:
            return None
        rp = self.sizes[bisect.bisect_left(self.sizes, R)]
        from onecat_vllm.ops.cuda import _sms, choose_decode_splits, choose_kv_splits
        if self.geom[0] == "mla":
            want = choose_kv_splits(rp * (-(-q * self.geom[1] // 16)), max_seq, _sms(self.r.device))
        else:
            want = choose_decode_splits(rp * self.geom[1], max_seq, _sms(self.r.device))
        s = 1  # bucketed to powers of two (rounding up keeps the grid sized for the live context)
        while s < want:
            s *= 2
        return rp, q, min(s, 32)

    def _metadata(self, rp: int, q: int, splits: int) -> AttentionMetadata:
        r = self.r
        T = rp * q
        md = AttentionMetadata(rp, T, r._view("qsl", rp + 1), r._view("seq", rp), r.d_bt[:rp], r._view("slot", T), r._view("pos", T),
                               q, 0, r._view("sslot", rp), r._view("hinit", rp), [q] * rp, [0] * rp, is_uniform_decode=True,
                               uniform_query_len=q)
        if r._seg["pos3"]:
            md.mrope_positions = r._view("pos3", 3 * r._tcap).view(3, r._tcap)[:, :T]
        if self.geom[0] == "mla":
            md.attn_plan = (("mla", self.geom[1], 512), (q, 0, splits))
        else:
            Hq, Hkv, D = self.geom
            G = Hq // Hkv
            short = (32 if D == 128 else 16) // G
            # uniform batch: every request has q tokens; they take the decode kernel when q*G rows fit its tile
            md.attn_plan = ((Hq, Hkv, D), (q if q <= short else short, 0 if q <= short else rp * (-(-q // (64 // G))), splits))
        md.static_ws = True
        return md

    def capture(self, key: tuple) -> None:
        rp, q, splits = key
        r = self.r
        md = self._metadata(rp, q, splits)
        ids = r._view("ids", rp * q)
        torch.cuda.synchronize()
        with torch.cuda.stream(self.stream):
            for _ in range(2):  # warm up allocator and lazy kernel attributes outside capture
                r.model(ids, md, r.kv_caches)
        self.stream.synchronize()
        from onecat_vllm.ops import cuda as K
        g = torch.cuda.CUDAGraph()
        n0 = K.launches()
        with torch.cuda.graph(g, pool=self.pool, stream=self.stream):
            out = r.model(ids, md, r.kv_caches)
        if self.pool is None:
            self.pool = g.pool()
        self.graphs[key] = (g, out, K.launches() - n0)  # kernels of ours inside one replay

    def capture_all(self) -> None:
        """Pre-capture the no-split graphs; split variants are captured on first use."""
        if not self.eligible:
            log.info_once("CUDA graphs disabled for this model (a layer's decode path needs the host)")
            return
        r = self.r
        r.np_pack[:] = 0
        r.np_bt[:] = 0
        r._bt_owner = [None] * len(r._bt_owner)
        o = r._off
        r.np_pack[o["slot"][0]: o["slot"][0] + o["slot"][1]] = -1
        r.d_pack.copy_(r.h_pack)
        r.d_bt.copy_(r.h_bt)
        for s in reversed(self.sizes):
            self.capture((s, 1, 1))
        log.info_once(f"captured {len(self.graphs)} decode graphs (sizes up to {self.sizes[-1]})")

    def run(self, key: tuple, T: int) -> torch.Tensor:
        if key not in self.graphs:
            self.misses += 1
            self.capture(key)
        else:
            self.hits += 1
        g, out, n = self.graphs[key]
        g.replay()
        self.r.graph_launches = getattr(self.r, "graph_launches", 0) + n
        return out[:T]

    def release(self) -> None:
        """Drop every captured graph (and with it the kernels, communicator references and pool memory it holds)."""
        for g, _out, _n in self.graphs.values():
            g.reset()
        self.graphs.clear()
        self.pool = None
