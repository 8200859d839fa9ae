"""Draft-token proposers for speculative decoding (reference: vllm/v1/spec_decode/llm_base_proposer.py:167,977,1427
MTP/EAGLE multi-step drafting; ngram_proposer.py prompt lookup; metadata.py:10).

``propose`` runs after the target step and returns, per request of the batch, the draft tokens to verify in the next
step (empty for requests still in prefill). The MTP proposer first re-runs the draft layer over this step's positions
with the token ids shifted by one and the target's hidden states (so its own KV cache stays in sync), then drafts
``k-1`` more tokens one position at a time."""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch

from onecat_vllm.worker.attn_metadata import AttentionMetadata


class NgramProposer:
    """Prompt lookup: find the longest recent n-gram (``min_n..max_n``) earlier in the context and propose what
    followed it."""

    def __init__(self, k: int, min_n: int, max_n: int):
        self.k, self.min_n, self.max_n = k, min_n, max_n
        try:  # the C++ scan (csrc/native/ngram.cpp); the Python loop below is its restatement and the fallback
            from onecat_vllm.utils import _native
            self._native = _native.ngram_propose
        except ImportError:
            self._native = None

    def propose_one(self, tokens: list) -> list:
        if self._native is not None:
            return self._native(np.asarray(tokens, dtype=np.int32), self.min_n, self.max_n, self.k)
        return self.propose_one_py(tokens)

    def propose_one_py(self, tokens: list) -> list:
        n_tok = len(tokens)
        for n in range(min(self.max_n, n_tok - 1), self.min_n - 1, -1):
            pat = tokens[n_tok - n:]
            for start in range(n_tok - n - 1, -1, -1):
                if tokens[start:start + n] == pat:
                    follow = tokens[start + n:start + n + self.k]
                    if follow:
                        return list(follow)
        return []

    def propose(self, runner, so, req_ids, rows, sampled, hidden, md, drafts_of):
        out = []
        for rid, s in zip(req_ids, sampled):
            st = runner.requests[rid]
            out.append(self.propose_one(st.token_ids) if s else [])
        return out


class SuffixProposer(NgramProposer):
    """Suffix-cache drafting: the request's own context first (prompt lookup), then a bounded index of the sequences that earlier
    requests of this engine finished, so repeated answers are drafted from their previous occurrence (reference:
    v1/spec_decode/suffix_decoding.py). The index is the C++ ``SuffixIndex``."""

    def __init__(self, k: int, min_n: int, max_n: int, max_tokens: int = 1 << 22):
        super().__init__(k, min_n, max_n)
        from onecat_vllm.utils import _native
        self.index = _native.SuffixIndex(min_n, max_n, max_tokens)
        self._live: dict = {}

    def propose(self, runner, so, req_ids, rows, sampled, hidden, md, drafts_of):
        # sequences of requests that left the batch since the last call go into the index
        for rid in [r for r in self._live if r not in runner.requests]:
            self.index.add(np.asarray(self._live.pop(rid), dtype=np.int32))
        out = []
        for rid, s in zip(req_ids, sampled):
            st = runner.requests[rid]
            self._live[rid] = st.token_ids
            if not s:
                out.append([])
                continue
            toks = np.asarray(st.token_ids, dtype=np.int32)
            d = self._native(toks, self.min_n, self.max_n, self.k)
            out.append(d if d else self.index.propose(toks[-self.max_n:], self.k))
        return out


class MTPProposer:
    def __init__(self, runner):
        self.k = runner.num_spec

    @torch.inference_mode()
    def propose(self, runner, so, req_ids, rows, sampled, hidden, md, drafts_of):
        mtp, dev, bs = runner.mtp, runner.device, runner.block_size
        R, T = md.num_reqs, md.num_tokens
        qsl = md.query_start_loc.tolist() if md.query_lens_cpu is None else np.concatenate([[0], np.cumsum(md.query_lens_cpu)]).tolist()
        # ---- pass 1: shifted ids over this step's positions
        ids = runner._view("ids", T).clone()
        shifted = torch.zeros_like(ids)
        shifted[:-1] = ids[1:]
        last_valid = []  # flat index of the last position whose next token is known
        nxt = []
        for r, rid in enumerate(req_ids):
            st = runner.requests[rid]
            a, b = qsl[r], qsl[r + 1]
            if not sampled[r]:
                # prefill chunk: the next token of the last position is the next prompt token
                pos_end = st.num_computed_tokens + (b - a)
                shifted[b - 1] = st.token_ids[pos_end] if pos_end < len(st.token_ids) else 0
                last_valid.append(-1)
                nxt.append(0)
                continue
            n_acc = len(sampled[r])  # accepted drafts + 1 (recovered or bonus)
            idx = a + (b - a) - (len(drafts_of[r]) + 1) + (n_acc - 1)
            shifted[idx] = sampled[r][-1]
            last_valid.append(idx)
            nxt.append(sampled[r][-1])
        if runner.spec.method == "eagle3":   # the head reads the target's residual stream at three depths, not its final hidden state
            hidden = torch.cat(runner.model.model.last_aux, dim=-1)
        h1 = mtp(shifted, hidden, md, runner.mtp_cache)
        active = [r for r in range(R) if last_valid[r] >= 0]
        out: list = [[] for _ in range(R)]
        if not active:
            return out
        sel = torch.tensor([last_valid[r] for r in active], device=dev)
        hcur = h1[sel]
        tok = mtp.compute_logits(hcur).argmax(-1)
        drafts = [tok]
        # ---- passes 2..k: one token per request at the following positions (lookahead slots were reserved)
        pos0 = np.array([runner.requests[req_ids[r]].num_computed_tokens + (qsl[r + 1] - qsl[r]) - (len(drafts_of[r]) + 1) + len(sampled[r])
                         for r in active], dtype=np.int32)
        A = len(active)
        bt = torch.zeros(A, runner.max_blocks_per_req, dtype=torch.int32, device=dev)
        for i, r in enumerate(active):
            b_ids = runner.requests[req_ids[r]].block_ids
            bt[i, : len(b_ids)] = torch.tensor(b_ids, dtype=torch.int32)
        for step in range(1, self.k):
            pos = pos0 + (step - 1)
            ok = pos < runner.max_model_len - 1
            slots = np.full(A, -1, dtype=np.int32)
            for i, r in enumerate(active):
                b_ids = runner.requests[req_ids[r]].block_ids
                if ok[i] and pos[i] // bs < len(b_ids):
                    slots[i] = b_ids[pos[i] // bs] * bs + pos[i] % bs
            md1 = AttentionMetadata(A, A, torch.arange(A + 1, dtype=torch.int32, device=dev), torch.tensor(pos + 1, dtype=torch.int32, device=dev), bt,
                                    torch.tensor(slots, dtype=torch.int32, device=dev), torch.tensor(pos, dtype=torch.int32, device=dev), 1,
                                    int(pos.max()) + 1, query_lens_cpu=[1] * A, seq_lens_cpu=(pos + 1).tolist())
            hcur = mtp(drafts[-1].to(torch.int32), hcur, md1, runner.mtp_cache)
            drafts.append(mtp.compute_logits(hcur).argmax(-1))
        d = torch.stack(drafts, dim=1).tolist()
        for i, r in enumerate(active):
            out[r] = d[i]
        return out


class DraftModelProposer:
    """A separate, smaller language model of the same vocabulary drafts the tokens. It keeps its own paged K/V under the target's block
    ids: one pass over the step's input tokens brings its cache level with the target's, then k single-token passes start from the token
    the target just sampled (reference: v1/spec_decode/draft_model.py; spec_decode/llm_base_proposer.py:167)."""

    def __init__(self, runner):
        self.k = runner.num_spec

    @torch.inference_mode()
    def propose(self, runner, so, req_ids, rows, sampled, hidden, md, drafts_of):
        draft, dev, bs = runner.draft, runner.device, runner.block_size
        R, T = md.num_reqs, md.num_tokens
        qsl = md.query_start_loc.tolist() if md.query_lens_cpu is None else np.concatenate([[0], np.cumsum(md.query_lens_cpu)]).tolist()
        draft.model(runner._view("ids", T), md, runner.draft_caches)     # fills the draft's K/V at this step's positions
        active = [r for r in range(R) if sampled[r]]
        out: list = [[] for _ in range(R)]
        if not active:
            return out
        # position of the token the target just sampled: the step's first position + inputs that were kept
        pos0 = np.array([runner.requests[req_ids[r]].num_computed_tokens + (qsl[r + 1] - qsl[r]) - (len(drafts_of[r]) + 1) + len(sampled[r])
                         for r in active], dtype=np.int32)
        A = len(active)
        bt = torch.zeros(A, runner.max_blocks_per_req, dtype=torch.int32, device=dev)
        for i, r in enumerate(active):
            b_ids = runner.requests[req_ids[r]].block_ids
            bt[i, : len(b_ids)] = torch.tensor(b_ids, dtype=torch.int32)
        tok = torch.tensor([sampled[r][-1] for r in active], dtype=torch.int32, device=dev)
        drafts = []
        for step in range(self.k):
            pos = pos0 + step
            ok = pos < runner.max_model_len - 1
            slots = np.full(A, -1, dtype=np.int32)
            for i, r in enumerate(active):
                b_ids = runner.requests[req_ids[r]].block_ids
                if ok[i] and pos[i] // bs < len(b_ids):
                    slots[i] = b_ids[pos[i] // bs] * bs + pos[i] % bs
            md1 = AttentionMetadata(A, A, torch.arange(A + 1, dtype=torch.int32, device=dev), torch.tensor(pos + 1, dtype=torch.int32, device=dev), bt,
                                    torch.tensor(slots, dtype=torch.int32, device=dev), torch.tensor(pos, dtype=torch.int32, device=dev), 1,
                                    int(pos.max()) + 1, query_lens_cpu=[1] * A, seq_lens_cpu=(pos + 1).tolist())
            h = draft.model(tok, md1, runner.draft_caches)
            tok = draft.compute_logits(h).argmax(-1).to(torch.int32)
            drafts.append(tok)
        d = torch.stack(drafts, dim=1).tolist()
        for i, r in enumerate(active):
            out[r] = d[i]
        return out


class MedusaHeads(torch.nn.Module):
    """Medusa: head ``i`` maps the target's last hidden state to the token ``i + 2`` positions ahead through residual SiLU blocks
    and its own vocabulary projection; no attention and no KV cache (reference: models/medusa.py ``ResidualBlock`` / ``Medusa``;
    spec_decode/medusa.py)."""

    def __init__(self, hidden: int, vocab: int, num_heads: int, num_layers: int, dtype):
        super().__init__()
        self.blocks = torch.nn.ModuleList([torch.nn.ModuleList([torch.nn.Linear(hidden, hidden, dtype=dtype) for _ in range(num_layers)])
                                           for _ in range(num_heads)])
        self.lm_heads = torch.nn.ModuleList([torch.nn.Linear(hidden, vocab, bias=False, dtype=dtype) for _ in range(num_heads)])

    def forward(self, h: torch.Tensor) -> list:
        out = []
        for layers, head in zip(self.blocks, self.lm_heads):
            x = h
            for lin in layers:
                x = x + torch.nn.functional.silu(lin(x))
            out.append(head(x))
        return out

    def load(self, path: str) -> int:
        """Tensor names: ``blocks.{i}.layers.{j}.{weight,bias}`` and ``lm_heads.{i}.weight``; the original release's
        ``{i}.{j}.linear.*`` / ``{i}.{L}.weight`` layout is accepted too."""
        import os
        import re
        from onecat_vllm.loader.weights import iter_safetensors
        if any(f.endswith(".safetensors") for f in os.listdir(path)):
            items = list(iter_safetensors(path))
        else:
            f = next(f for f in ("medusa_lm_head.pt", "pytorch_model.bin") if os.path.exists(os.path.join(path, f)))
            items = list(torch.load(os.path.join(path, f), map_location="cpu", weights_only=True).items())
        sd = dict(self.state_dict())
        n = 0
        L = len(self.blocks[0]) if len(self.blocks) else 0
        for name, w in items:
            name = re.sub(r"^blocks\.(\d+)\.layers\.(\d+)\.", r"blocks.\1.\2.", name)
            m = re.match(r"^(?:medusa_head\.)?(\d+)\.(\d+)\.(?:linear\.)?(weight|bias)$", name)
            if m:
                i, j, leaf = int(m.group(1)), int(m.group(2)), m.group(3)
                name = f"lm_heads.{i}.weight" if j == L else f"blocks.{i}.{j}.{leaf}"
            if name in sd and sd[name].shape == w.shape:
                sd[name].copy_(w)
                n += 1
        return n


class MedusaProposer:
    def __init__(self, runner):
        sc, mc = runner.spec, runner.mc
        self.k = sc.num_speculative_tokens
        self.heads = MedusaHeads(mc.hidden_size, mc.vocab_size, self.k, sc.medusa_num_layers, mc.dtype).to(runner.device).eval()
        g = torch.Generator().manual_seed(mc.seed + 2)
        with torch.no_grad():
            for p in self.heads.parameters():
                p.copy_(torch.empty(p.shape).normal_(0, 0.02, generator=g))
        if sc.model:
            self.heads.load(sc.model)

    @torch.inference_mode()
    def propose(self, runner, so, req_ids, rows, sampled, hidden, md, drafts_of):
        R = md.num_reqs
        qsl = np.concatenate([[0], np.cumsum(md.query_lens_cpu)]).tolist() if md.query_lens_cpu is not None else md.query_start_loc.tolist()
        out: list = [[] for _ in range(R)]
        active, idx = [], []
        for r in range(R):
            if sampled[r]:
                # the hidden state of the last accepted position: the one that produced the newest token
                active.append(r)
                idx.append(qsl[r + 1] - (len(drafts_of[r]) + 1) + (len(sampled[r]) - 1))
        if not active:
            return out
        logits = self.heads(hidden[torch.tensor(idx, device=hidden.device)])
        toks = torch.stack([lg.argmax(-1) for lg in logits], dim=1).tolist()
        for i, r in enumerate(active):
            out[r] = toks[i]
        return out


def make_proposer(runner):
    sc = runner.spec
    if sc.method == "ngram":
        return NgramProposer(sc.num_speculative_tokens, sc.prompt_lookup_min, sc.prompt_lookup_max)
    if sc.method in ("mtp", "eagle", "eagle3"):
        return MTPProposer(runner)
    if sc.method == "draft_model":
        return DraftModelProposer(runner)
    if sc.method == "suffix":
        return SuffixProposer(sc.num_speculative_tokens, sc.prompt_lookup_min, sc.prompt_lookup_max)
    if sc.method == "medusa":
        return MedusaProposer(runner)
    raise ValueError(f"unknown speculative method {sc.method!r}")
