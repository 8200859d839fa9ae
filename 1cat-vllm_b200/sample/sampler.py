"""Token sampler (reference: vllm/v1/sample/sampler.py:87-366; ops/topk_topp_sampler.py:22-438).

Order: raw logprobs (if requested) → logits processors (allowed ids, bad words, min_tokens, logit bias, grammar
mask) → penalties → temperature → min-p / top-k / top-p → exponential-noise argmax; greedy rows take the argmax
of the processed logits. Sampled ids come back as int64 ``[B]``."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from onecat_vllm import ops
from onecat_vllm.core.sched_output import LogprobsLists
from onecat_vllm.ops import ref
from onecat_vllm.sample.metadata import SamplingMetadata

_EPS = 1e-5


@dataclass
class SamplerOutput:
    sampled_token_ids: torch.Tensor  # [B] int64
    logprobs: Optional[tuple] = None  # (topk_ids [B,k+1], topk_logprobs [B,k+1], ranks [B])


class Sampler:
    @staticmethod
    def is_plain_greedy(md: SamplingMetadata) -> bool:
        """Every row takes the arg-max of the untouched logits (so the token can be found without materialising them)."""
        return (md.all_greedy and md.no_penalties and not md.min_tokens and not any(md.logit_bias) and
                not any(a is not None for a in md.allowed_token_ids) and not md.bad_words_token_ids and md.grammar_bitmask is None
                and not md.thinking and not md.custom_processors)

    def __call__(self, logits: torch.Tensor, md: SamplingMetadata) -> SamplerOutput:
        raw_lp = None
        if md.max_num_logprobs is not None:
            raw_lp = torch.log_softmax(logits.float(), dim=-1)
        simple = self.is_plain_greedy(md)
        if simple:
            sampled = ops.argmax(logits)  # greedy fast path: no fp32 copy of the logits
        else:
            lg = logits.float()
            lg = self.apply_logits_processors(lg, md)
            lg = self.apply_penalties(lg, md)
            for proc in md.custom_processors:   # user processors see the fp32 logits after the built-in ones
                lg = proc.apply(lg, md.row_info)
            sampled = self.sample(lg, md)
        lp = None
        if raw_lp is not None:
            lp = self.gather_logprobs(raw_lp, md.max_num_logprobs, sampled)
        return SamplerOutput(sampled.long(), lp)

    # ------------------------------------------------------------------
    @staticmethod
    def apply_logits_processors(lg: torch.Tensor, md: SamplingMetadata) -> torch.Tensor:
        B, V = lg.shape
        for i, allowed in enumerate(md.allowed_token_ids):
            if allowed is not None:
                mask = torch.ones(V, dtype=torch.bool, device=lg.device)
                mask[torch.tensor(allowed, device=lg.device)] = False
                lg[i].masked_fill_(mask, -float("inf"))
        for i, words in md.bad_words_token_ids.items():
            out = md.output_token_ids[i]
            for w in words:
                if len(w) == 1 or (len(out) >= len(w) - 1 and out[len(out) - len(w) + 1:] == w[:-1]):
                    lg[i, w[-1]] = -float("inf")
        for i, (mn, stop_ids) in md.min_tokens.items():
            if len(md.output_token_ids[i]) < mn and stop_ids:
                lg[i, torch.tensor(sorted(stop_ids), device=lg.device)] = -float("inf")
        for i, bias in enumerate(md.logit_bias):
            if bias:
                idx = torch.tensor(list(bias.keys()), device=lg.device)
                lg[i, idx] += torch.tensor(list(bias.values()), device=lg.device, dtype=lg.dtype)
        if md.grammar_bitmask is not None:
            lg.masked_fill_(~md.grammar_bitmask, -float("inf"))
        for i, (budget, start, end) in md.thinking.items():
            # inside a thinking block (after the last think-start, no think-end yet) that has used its budget: only think-end may follow
            out = md.output_token_ids[i]
            last_start = max((j for j, t in enumerate(out) if t == start), default=-1)
            if last_start >= 0 and end not in out[last_start:] and len(out) - last_start - 1 >= budget:
                keep = lg[i, end].clone()
                lg[i].fill_(-float("inf"))
                lg[i, end] = keep if torch.isfinite(keep) else 0.0
        return lg

    @staticmethod
    def apply_penalties(lg: torch.Tensor, md: SamplingMetadata) -> torch.Tensor:
        if md.no_penalties:
            return lg
        B, V = lg.shape
        pm = torch.zeros(B, V, dtype=torch.bool, device=lg.device)
        oc = torch.zeros(B, V, dtype=torch.int32, device=lg.device)
        for i in range(B):
            if md.prompt_token_ids and md.prompt_token_ids[i]:
                pm[i, torch.tensor(md.prompt_token_ids[i], device=lg.device)] = True
            if md.output_token_ids[i]:
                ids = torch.tensor(md.output_token_ids[i], device=lg.device)
                oc[i].scatter_add_(0, ids, torch.ones_like(ids, dtype=torch.int32))
        return ref.apply_penalties(lg, pm, oc, md.presence_penalties, md.frequency_penalties, md.repetition_penalties)

    @staticmethod
    def sample(lg: torch.Tensor, md: SamplingMetadata) -> torch.Tensor:
        if lg.is_cuda and not md.all_greedy:
            # one kernel: filters by threshold search (no sort) and the exponential-race draw
            from onecat_vllm.ops import cuda as K
            return K.sample(lg if lg.stride(-1) == 1 else lg.contiguous(), md.temperature, md.top_k, md.top_p, md.min_p, md.generators)
        greedy = lg.argmax(-1) if not md.all_random else None
        if md.all_greedy:
            return greedy
        t = md.temperature
        lt = lg / torch.where(t < _EPS, torch.ones_like(t), t).unsqueeze(-1)
        if md.top_k is not None or md.top_p is not None or md.min_p is not None:
            lt = ref.top_k_top_p_min_p(lt, md.top_k, md.top_p, md.min_p)
        probs = torch.softmax(lt, dim=-1)
        rnd = ref.random_sample(probs, md.generators)
        if greedy is None:
            return rnd
        return torch.where(t < _EPS, greedy, rnd)

    @staticmethod
    def gather_logprobs(lp: torch.Tensor, k: int, sampled: torch.Tensor):
        tok_lp = lp.gather(-1, sampled.long().unsqueeze(-1))
        ranks = (lp > tok_lp).sum(-1) + 1
        if k > 0:
            tv, ti = lp.topk(k, dim=-1)
            ids = torch.cat([sampled.long().unsqueeze(-1), ti], dim=-1)
            vals = torch.cat([tok_lp, tv], dim=-1)
        else:
            ids, vals = sampled.long().unsqueeze(-1), tok_lp
        return ids, vals, ranks


def to_logprobs_lists(lp: Optional[tuple], row_counts: list[int]) -> Optional[list[Optional[LogprobsLists]]]:
    """Split batched logprob tensors into per-request lists (``row_counts[i]`` sampled positions each)."""
    if lp is None:
        return None
    ids, vals, ranks = (t.tolist() for t in lp)
    out, o = [], 0
    for n in row_counts:
        out.append(LogprobsLists(ids[o:o + n], vals[o:o + n], ranks[o:o + n]) if n else None)
        o += n
    return out
