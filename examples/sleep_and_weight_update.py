"""Sleep mode and in-place weight update, the two hooks an RLHF loop needs between rollouts.

    python examples/sleep_and_weight_update.py --device cpu
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from onecat_vllm import LLM, SamplingParams  # noqa: E402

from _tiny import engine_kwargs, parse  # noqa: E402

if __name__ == "__main__":
    args = parse(__doc__)
    llm = LLM(enable_sleep_mode=True, **engine_kwargs(args))
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    prompt = [{"prompt_token_ids": [72, 101, 108, 108, 111]}]
    before = llm.generate(prompt, sp)[0].outputs[0].token_ids
    llm.sleep(level=1)          # level 1: the KV cache is dropped, the weights are kept (on a GPU: offloaded to host memory)
    llm.wake_up()
    assert llm.generate(prompt, sp)[0].outputs[0].token_ids == before
    # push new weights for one tensor (HF checkpoint names; any subset of the model may be sent)
    name = "model.norm.weight"
    new = torch.linspace(-1.0, 2.0, llm.llm_engine.cfg.model_config.hidden_size)
    n = llm.collective_rpc("update_weights", ([(name, new)],))
    llm.reset_prefix_cache()    # cached KV was computed with the old weights
    after = llm.generate(prompt, sp)[0].outputs[0].token_ids
    print("tensors updated per worker:", n, "| before:", before, "| after:", after)
    llm.shutdown()
