"""Offline inference API (reference: vllm/entrypoints/llm.py:66 class, :422 ``generate``, :487 ``chat``, :806-889
sleep / wake_up / collective_rpc / get_metrics; run loop entrypoints/offline_utils.py:326,573)."""
from __future__ import annotations

import itertools
import os
from typing import Optional, Sequence, Union

from onecat_vllm.config import EngineArgs
from onecat_vllm.engine.llm_engine import LLMEngine
from onecat_vllm.inputs import PromptType
from onecat_vllm.outputs import RequestOutput
from onecat_vllm.outputs import PoolingRequestOutput
from onecat_vllm.sampling_params import BeamSearchParams, PoolingParams, RequestOutputKind, SamplingParams


class LLM:
    """``LLM(model=<checkpoint dir>)`` loads an HF-format checkpoint; ``LLM(hf_config={...})`` builds the architecture
    with random weights (synthetic benchmarks and tests)."""

    def __init__(self, model: str = "dummy", **kwargs):
        self.engine_args = EngineArgs(model=model, **kwargs)
        self.llm_engine = LLMEngine.from_engine_args(self.engine_args)
        self._counter = itertools.count()
        if os.environ.get("ONECAT_USAGE_STATS_FILE"):
            from onecat_vllm.platforms import usage_record
            cfg = self.llm_engine.cfg
            usage_record("LLM_CLASS", cfg.model_config.architecture, {"tensor_parallel_size": cfg.parallel_config.tensor_parallel_size,
                                                                      "quantization": cfg.model_config.quant.method})

    def get_tokenizer(self):
        return self.llm_engine.tokenizer

    def generate(self, prompts: Union[PromptType, Sequence[PromptType]], sampling_params: Optional[Union[SamplingParams, Sequence[SamplingParams]]] = None,
                 use_tqdm: bool = False, priority: Optional[list[int]] = None, lora_request=None) -> list[RequestOutput]:
        """``lora_request``: one ``LoRARequest`` for all prompts or a list with one entry (or ``None``) per prompt."""
        if isinstance(prompts, (str, dict)) or (isinstance(prompts, list) and prompts and isinstance(prompts[0], int)):
            prompts = [prompts]
        if sampling_params is None:
            sampling_params = SamplingParams()
        sps = list(sampling_params) if isinstance(sampling_params, (list, tuple)) else [sampling_params] * len(prompts)
        if len(sps) != len(prompts):
            raise ValueError("the number of sampling params must match the number of prompts")
        ids = []
        for i, (p, sp) in enumerate(zip(prompts, sps)):
            sp = sp.clone()
            sp.output_kind = RequestOutputKind.FINAL_ONLY
            rid = str(next(self._counter))
            ids.append(rid)
            lr = lora_request[i] if isinstance(lora_request, (list, tuple)) else lora_request
            self.llm_engine.add_request(rid, p, sp, priority=priority[i] if priority else 0, lora_request=lr)
        return self._run_engine(ids, use_tqdm)

    def chat(self, messages, sampling_params: Optional[SamplingParams] = None, add_generation_prompt: bool = True, **kw) -> list[RequestOutput]:
        tok = self.get_tokenizer()
        if tok is None:
            raise ValueError("chat() needs a tokenizer")
        convs = messages if messages and isinstance(messages[0], list) else [messages]
        from onecat_vllm.engine.renderers import render_chat
        arch = self.llm_engine.cfg.model_config.architecture
        prompts = [render_chat(tok, c, architecture=arch, add_generation_prompt=add_generation_prompt, **kw) for c in convs]
        return self.generate(prompts, sampling_params)

    def beam_search(self, prompts: Sequence[PromptType], params: BeamSearchParams) -> list[dict]:
        """Beam search by repeated one-token steps with ``2 * beam_width`` log-probabilities per beam; the prefix cache makes every
        step after the first a one-token decode per beam (reference: entrypoints/llm.py ``beam_search``, beam_search.py). Returns per
        prompt ``{"sequences": [{"tokens", "cum_logprob", "text"} ...]}`` sorted best first (score = cum_logprob / len ** length_penalty)."""
        from onecat_vllm.inputs import parse_prompt
        tok = self.get_tokenizer()
        eos = self.llm_engine.cfg.model_config.eos_token_id
        if eos is None and tok is not None:
            eos = getattr(tok, "eos_token_id", None)
        W = params.beam_width
        sp = SamplingParams(temperature=0.0, max_tokens=1, logprobs=2 * W, detokenize=False)
        results = []
        for prompt in prompts:
            text, ids, _ = parse_prompt(prompt)
            if ids is None:
                ids = list(tok.encode(text))
            n0 = len(ids)
            beams = [(list(ids), 0.0)]
            done: list = []
            score = lambda toks, lp: lp / (max(len(toks) - n0, 1) ** params.length_penalty)
            for _ in range(params.max_tokens):
                if not beams:
                    break
                outs = self.generate([{"prompt_token_ids": b[0]} for b in beams], sp)
                cand = []
                for (toks, lp), o in zip(beams, outs):
                    for tid, l in o.outputs[0].logprobs[0].items():
                        if tid == eos and not params.ignore_eos:
                            done.append((toks + [tid], lp + l.logprob))
                        else:
                            cand.append((toks + [tid], lp + l.logprob))
                cand.sort(key=lambda c: -c[1])
                beams = cand[:W]
            done += beams
            done.sort(key=lambda c: -score(*c))
            results.append({"sequences": [{"tokens": t, "cum_logprob": lp, "text": tok.decode(t[n0:]) if tok is not None else None}
                                          for t, lp in done[:W]]})
        return results

    # ---- pooling tasks (reference: entrypoints/llm.py ``encode`` / ``embed`` / ``score``)
    def encode(self, prompts: Union[PromptType, Sequence[PromptType]], pooling_params: Optional[PoolingParams] = None,
               use_tqdm: bool = False) -> list[PoolingRequestOutput]:
        if isinstance(prompts, (str, dict)) or (isinstance(prompts, list) and prompts and isinstance(prompts[0], int)):
            prompts = [prompts]
        pp = pooling_params or PoolingParams(task="encode", normalize=False)
        ids = []
        for p in prompts:
            rid = str(next(self._counter))
            ids.append(rid)
            self.llm_engine.add_request(rid, p, pp)
        return self._run_engine(ids, use_tqdm)

    def embed(self, prompts, pooling_params: Optional[PoolingParams] = None, use_tqdm: bool = False) -> list[PoolingRequestOutput]:
        return self.encode(prompts, pooling_params or PoolingParams(task="embed", normalize=True), use_tqdm)

    def classify(self, prompts, pooling_params: Optional[PoolingParams] = None, use_tqdm: bool = False) -> list[PoolingRequestOutput]:
        """Class probabilities from a sequence-classification checkpoint (reference: entrypoints/llm.py ``LLM.classify``)."""
        return self.encode(prompts, pooling_params or PoolingParams(task="classify", normalize=False), use_tqdm)

    def score(self, text_1: Union[str, Sequence[str]], text_2: Union[str, Sequence[str]], use_tqdm: bool = False) -> list[float]:
        """Similarity of text pairs (1:N or N:N): a cross-encoder checkpoint (sequence classification with one label) scores the
        concatenated pair; any other model gives the cosine similarity of the two texts' embeddings
        (reference: entrypoints/llm.py ``LLM.score``, entrypoints/pooling/score/)."""
        a = [text_1] if isinstance(text_1, str) else list(text_1)
        b = [text_2] if isinstance(text_2, str) else list(text_2)
        if len(a) == 1:
            a = a * len(b)
        if len(a) != len(b):
            raise ValueError("score() takes 1:N or N:N inputs")
        mc = self.llm_engine.cfg.model_config
        if mc.num_labels == 1:
            tok = self.get_tokenizer()
            sep = getattr(tok, "sep_token_id", None)
            sep = mc.eos_token_id if sep is None else sep
            pairs = [{"prompt_token_ids": list(tok.encode(x)) + ([sep] if sep is not None else []) + list(tok.encode(y, add_special_tokens=False))}
                     for x, y in zip(a, b)]
            return [o.outputs.data[0] for o in self.classify(pairs, use_tqdm=use_tqdm)]
        embs = self.embed(a + b, use_tqdm=use_tqdm)
        ea, eb = embs[: len(a)], embs[len(a):]
        return [sum(x * y for x, y in zip(p.outputs.data, q.outputs.data)) for p, q in zip(ea, eb)]

    def _run_engine(self, ids: list[str], use_tqdm: bool = False) -> list[RequestOutput]:
        done: dict[str, RequestOutput] = {}
        bar = None
        if use_tqdm:
            from tqdm import tqdm
            bar = tqdm(total=len(ids), desc="Processed prompts")
        eng = self.llm_engine
        while eng.has_unfinished_requests():
            for out in eng.step():
                if out.finished:
                    done[out.request_id] = out
                    if bar:
                        bar.update(1)
        if bar:
            bar.close()
        return [done[i] for i in ids if i in done]

    # ---- control surface
    def sleep(self, level: int = 1) -> None:
        self.llm_engine.sleep(level)

    def wake_up(self, tags=None) -> None:
        self.llm_engine.wake_up(tags)

    def reset_prefix_cache(self) -> bool:
        return self.llm_engine.reset_prefix_cache()

    def collective_rpc(self, method, args=(), kwargs=None):
        return self.llm_engine.collective_rpc(method, args, kwargs)

    def get_metrics(self) -> dict:
        return self.llm_engine.get_metrics()

    def shutdown(self) -> None:
        self.llm_engine.shutdown()
