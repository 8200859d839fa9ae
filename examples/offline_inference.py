"""Offline generation: text and token-id prompts, greedy and sampled.

    python examples/offline_inference.py --device cpu
    python examples/offline_inference.py --model /path/to/checkpoint
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from onecat_vllm import LLM, SamplingParams  # noqa: E402

from _tiny import engine_kwargs, parse  # noqa: E402

if __name__ == "__main__":
    args = parse(__doc__)
    llm = LLM(**engine_kwargs(args))
    prompts = ["The capital of France is", {"prompt_token_ids": [72, 101, 108, 108, 111]}]
    for sp in (SamplingParams(temperature=0.0, max_tokens=16), SamplingParams(temperature=0.8, top_p=0.9, top_k=40, seed=1, max_tokens=16, n=2)):
        for out in llm.generate(prompts, sp):
            for c in out.outputs:
                print(f"[T={sp.temperature}] {out.prompt!r} -> {c.text!r}  ({len(c.token_ids)} tokens, finish={c.finish_reason})")
    llm.shutdown()
