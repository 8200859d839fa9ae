"""Speculative-decoding verifier (reference: vllm/v1/sample/rejection_sampler.py:196 class, :896 ``rejection_sample``,
:942-957 synthetic mode, :1150-1204 uniforms in float64; CPU kernels csrc/cpu/spec_decode_utils.cpp:211-409).

Inputs are the target logits of the ``k+1`` positions each request verified. Greedy rows accept while the draft
equals the target argmax; random rows accept draft ``x`` iff ``p_target(x)/p_draft(x) >= u`` and on the first
rejection emit a recovered token; when every draft is accepted the bonus token (sampled from the last position)
is appended. In synthetic mode acceptance is ``u < rate[pos]`` from a seeded stream, which makes the verifier path
measurable with random weights."""
from __future__ import annotations

from typing import Optional

import torch

from onecat_vllm.ops import ref
from onecat_vllm.sample.metadata import SamplingMetadata

PLACEHOLDER = -1


class RejectionSampler:
    def __init__(self, synthetic_rates: Optional[list[float]] = None, seed: int = 0):
        self.synthetic_rates = synthetic_rates
        self._gen: dict = {}
        self.seed = seed

    def _generator(self, device) -> torch.Generator:
        key = str(device)
        if key not in self._gen:
            g = torch.Generator(device=device)
            g.manual_seed(self.seed)
            self._gen[key] = g
        return self._gen[key]

    def __call__(self, draft_ids: torch.Tensor, num_draft: torch.Tensor, target_logits: torch.Tensor, bonus_ids: torch.Tensor,
                 md: SamplingMetadata, draft_probs: Optional[torch.Tensor] = None) -> torch.Tensor:
        """draft_ids ``[B,k]`` (padded), num_draft ``[B]``, target_logits ``[B,k+1,V]`` (row i = logits after consuming
        draft i-1), bonus_ids ``[B]``. Returns ``[B,k+1]`` int64 padded with -1."""
        B, k = draft_ids.shape
        dev = target_logits.device
        gen = self._generator(dev)
        uniforms = torch.rand(B, k, dtype=torch.float64, device=dev, generator=gen)
        if target_logits.is_cuda:
            from onecat_vllm.ops import cuda as K
            return K.rejection_sample(draft_ids, num_draft, target_logits, bonus_ids, md, draft_probs, uniforms,
                                      self.synthetic_rates, gen)
        greedy = torch.ones(B, dtype=torch.bool) if md.all_greedy else (md.temperature < 1e-5)
        if md.all_greedy and self.synthetic_rates is None:
            probs = target_logits[:, :k].float()
            noise = None
        else:
            t = md.temperature if md.temperature is not None else torch.ones(B, device=dev)
            t = torch.where(t < 1e-5, torch.ones_like(t), t).view(B, 1, 1)
            probs = torch.softmax(target_logits[:, :k].float() / t, dim=-1)
            noise = torch.empty_like(probs).exponential_(generator=gen)
            if md.all_greedy:  # synthetic mode with greedy requests: the "recovered" token is the argmax
                noise = None
        return ref.rejection_sample(draft_ids, num_draft, probs, bonus_ids, draft_probs, uniforms,
                                    greedy if self.synthetic_rates is None else None, self.synthetic_rates, noise, PLACEHOLDER)

    @staticmethod
    def parse_output(out: torch.Tensor) -> list[list[int]]:
        """Strip padding: per request the accepted tokens (+ recovered or bonus)."""
        return [[t for t in row if t != PLACEHOLDER] for row in out.tolist()]
