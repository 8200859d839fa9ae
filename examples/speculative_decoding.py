"""Speculative decoding: n-gram lookup needs nothing but the prompt; a draft head or a draft model takes a checkpoint directory.

    python examples/speculative_decoding.py --device cpu
    python examples/speculative_decoding.py --model /path/to/target --method draft_model --draft /path/to/draft
    python examples/speculative_decoding.py --model /path/to/target --method eagle3 --draft /path/to/eagle3-head
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from onecat_vllm import LLM, SamplingParams  # noqa: E402

import _tiny  # noqa: E402

if __name__ == "__main__":
    import argparse
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--model", default=None)
    ap.add_argument("--device", default="auto")
    ap.add_argument("--method", default="ngram", choices=["ngram", "suffix", "mtp", "eagle", "eagle3", "medusa", "draft_model"])
    ap.add_argument("--draft", default=None, help="checkpoint directory of the draft head / draft model")
    ap.add_argument("--num-speculative-tokens", type=int, default=3)
    a = ap.parse_args()
    a.tensor_parallel_size = 1
    spec = dict(method=a.method, num_speculative_tokens=a.num_speculative_tokens)
    if a.draft:
        spec["model"] = a.draft
    llm = LLM(speculative_config=spec, disable_log_stats=False, **_tiny.engine_kwargs(a))
    text = "one two three one two three one two three one two"
    out = llm.generate([text], SamplingParams(temperature=0.0, max_tokens=48, ignore_eos=True))[0]
    m = llm.llm_engine.get_metrics()
    print(repr(out.outputs[0].text))
    print("draft tokens:", m.get("vllm:spec_decode_num_draft_tokens_total"), "accepted:", m.get("vllm:spec_decode_num_accepted_tokens_total"))
    llm.shutdown()
