"""Grammar-constrained decoding end to end on CPU (reference test model: tests/v1/structured_output/test_utils.py,
tests/v1/entrypoints/llm/test_struct_output_generate.py)."""
import json

import numpy as np
import pytest

from onecat_vllm import LLM, SamplingParams
from onecat_vllm.engine.tokenizer import ByteTokenizer
from onecat_vllm.sampling_params import StructuredOutputsParams
from onecat_vllm.structured import StructuredOutputManager, unpack_bitmask

TINY = dict(architectures=["Qwen3ForCausalLM"], hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
            num_key_value_heads=2, head_dim=16, vocab_size=320, max_position_embeddings=512, rms_norm_eps=1e-6, rope_theta=10000.0)


@pytest.mark.parametrize("backend", ["builtin", "xgrammar"])
def test_choice_bitmask_walk(backend):
    if backend == "xgrammar":
        pytest.importorskip("xgrammar")
    m = StructuredOutputManager(ByteTokenizer(), 300, backend=backend)
    assert m.grammar_init("a", StructuredOutputsParams(choice=["yes", "no", "nope"]))
    assert not m.grammar_init("b", None)
    got = b""
    for _ in range(6):
        mask, rows = m.grammar_bitmask(["plain", "a"])
        assert rows == {"a": 0} and mask.shape == (1, 10)
        allowed = np.nonzero(unpack_bitmask(mask, 300)[0])[0].tolist()
        t = allowed[0]
        assert m.accept_tokens("a", [t])
        if t == ByteTokenizer.eos_token_id:
            break
        got += bytes([t])
    assert got.decode() in ("yes", "no", "nope")
    m.free("a")
    assert m.grammar_bitmask(["a"]) == (None, {})


@pytest.mark.parametrize("spec", [None, {"method": "ngram", "num_speculative_tokens": 2}])
def test_generate_follows_choice_and_json(spec):
    pytest.importorskip("xgrammar")
    llm = LLM(hf_config=TINY, tokenizer="byte", device="cpu", max_model_len=256, speculative_config=spec)
    schema = {"type": "object", "properties": {"n": {"type": "integer"}, "ok": {"type": "boolean"}}, "required": ["n", "ok"],
              "additionalProperties": False}
    sps = [SamplingParams(temperature=0.0, max_tokens=16, structured_outputs=StructuredOutputsParams(choice=["alpha", "beta"])),
           SamplingParams(temperature=0.8, seed=1, max_tokens=96, structured_outputs=StructuredOutputsParams(json=schema)),
           SamplingParams(temperature=0.0, max_tokens=8)]
    outs = llm.generate(["pick:", "json:", "free:"], sps)
    assert outs[0].outputs[0].text in ("alpha", "beta")
    assert outs[0].outputs[0].finish_reason == "stop"
    if outs[1].outputs[0].finish_reason == "stop":
        obj = json.loads(outs[1].outputs[0].text)
        assert isinstance(obj["n"], int) and isinstance(obj["ok"], bool)
    else:  # ran out of tokens: still a prefix of valid JSON
        assert outs[1].outputs[0].text.lstrip().startswith("{")
    assert len(outs[2].outputs[0].token_ids) == 8
