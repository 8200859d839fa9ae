"""Constrained decoding: the answer is one of a fixed set of strings.

    python examples/structured_output.py --device cpu
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from onecat_vllm import LLM, SamplingParams  # noqa: E402
from onecat_vllm.sampling_params import StructuredOutputsParams  # noqa: E402

from _tiny import engine_kwargs, parse  # noqa: E402

if __name__ == "__main__":
    args = parse(__doc__)
    llm = LLM(**engine_kwargs(args))
    sp = SamplingParams(temperature=0.7, seed=0, max_tokens=8, structured_outputs=StructuredOutputsParams(choice=["yes", "no", "maybe"]))
    for out in llm.generate(["Is water wet? Answer:", "Will it rain tomorrow? Answer:"], sp):
        print(repr(out.prompt), "->", repr(out.outputs[0].text))
    llm.shutdown()
