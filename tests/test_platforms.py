"""Platform description and the local usage record."""
import json

import pytest
import torch

from onecat_vllm import platforms


def test_cpu_platform_and_usage_record(tmp_path, monkeypatch):
    p = platforms.current_platform(refresh=True)
    if not torch.cuda.is_available():
        assert p.is_cpu() and p.dispatch_key == "ref" and not p.supports_native_kernels() and p.default_dtype() == torch.float32
        assert platforms.resolve_device("auto") == "cpu"
        with pytest.raises(ValueError):
            platforms.resolve_device("cuda")
    d = p.describe()
    assert d["device_type"] == p.device_type and d["total_memory"] > 0
    out = tmp_path / "usage.jsonl"
    monkeypatch.setenv("ONECAT_USAGE_STATS_FILE", str(out))
    rec = platforms.usage_record("LLM_CLASS", "LlamaForCausalLM", {"tensor_parallel_size": 2})
    line = json.loads(out.read_text().strip())
    assert line["architecture"] == "LlamaForCausalLM" and line["tensor_parallel_size"] == 2 and line["platform"] == rec["platform"]


def test_out_of_tree_layer_class_replaces_a_decoder_block():
    from onecat_vllm import LLM, SamplingParams
    from onecat_vllm.layers.mlp import MLP
    from onecat_vllm.utils import plugins
    calls = []

    class CountingMLP(MLP):
        def forward(self, x):
            calls.append(x.shape[0])
            return super().forward(x)
    cfg = dict(architectures=["LlamaForCausalLM"], hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
               num_key_value_heads=2, head_dim=16, vocab_size=300, max_position_embeddings=256)
    sp = SamplingParams(temperature=0, max_tokens=4, ignore_eos=True)
    base = LLM(hf_config=cfg, device="cpu", dtype="float32", max_model_len=64)
    want = base.generate([[1, 2, 3]], sp)[0].outputs[0].token_ids
    base.shutdown()
    plugins.register_layer("MLP", CountingMLP)
    try:
        llm = LLM(hf_config=cfg, device="cpu", dtype="float32", max_model_len=64)
        got = llm.generate([[1, 2, 3]], sp)[0].outputs[0].token_ids
        llm.shutdown()
    finally:
        plugins.unregister_layer("MLP")
    assert got == want and len(calls) >= 2 * 4        # two layers, four steps
