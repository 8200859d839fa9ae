"""Multi-LoRA serving on CPU: a PEFT-format adapter applied per request must equal a model whose weights have the adapter
merged in; requests with and without adapters share a batch (reference test model: tests/lora/test_llama_tp.py, test_lora_manager.py)."""
import json
import os

import pytest
import torch

from onecat_vllm import LLM, SamplingParams
from onecat_vllm.lora import LoRARequest

CFG = dict(architectures=["LlamaForCausalLM"], hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
           num_key_value_heads=2, head_dim=16, vocab_size=300, max_position_embeddings=256)
TARGETS = {"self_attn.q_proj": (64, 64), "self_attn.k_proj": (64, 32), "self_attn.v_proj": (64, 32), "self_attn.o_proj": (64, 64),
           "mlp.gate_proj": (64, 128), "mlp.up_proj": (64, 128), "mlp.down_proj": (128, 64)}


def _write_adapter(path, seed, r=4, alpha=8.0, std=0.2):
    from safetensors.torch import save_file
    g = torch.Generator().manual_seed(seed)
    t = {}
    for l in range(CFG["num_hidden_layers"]):
        for name, (i, o) in TARGETS.items():
            t[f"base_model.model.model.layers.{l}.{name}.lora_A.weight"] = torch.randn(r, i, generator=g) * std
            t[f"base_model.model.model.layers.{l}.{name}.lora_B.weight"] = torch.randn(o, r, generator=g) * std
    os.makedirs(path, exist_ok=True)
    save_file(t, os.path.join(path, "adapter_model.safetensors"))
    json.dump({"r": r, "lora_alpha": alpha, "target_modules": [n.split(".")[-1] for n in TARGETS]}, open(os.path.join(path, "adapter_config.json"), "w"))
    return t, alpha / r


def _base_ckpt(path, merged=None, scale=1.0):
    from onecat_vllm.config import ModelConfig
    from onecat_vllm.loader.weights import dummy_init, save_pretrained, to_hf_state_dict
    from onecat_vllm.models import build_model
    m = build_model(ModelConfig.from_hf_dict(CFG, dtype=torch.float32), "cpu")
    dummy_init(m, 0, std=0.08)
    if merged is None:
        save_pretrained(m, CFG, path)
        return
    sd = to_hf_state_dict(m)
    for k in list(sd):
        key = "base_model.model." + k[: -len(".weight")]
        if key + ".lora_A.weight" in merged:
            sd[k] = sd[k].float() + scale * merged[key + ".lora_B.weight"] @ merged[key + ".lora_A.weight"]
    from safetensors.torch import save_file
    os.makedirs(path, exist_ok=True)
    save_file({k: v.contiguous() for k, v in sd.items()}, os.path.join(path, "model.safetensors"))
    json.dump(CFG, open(os.path.join(path, "config.json"), "w"))


@pytest.mark.timeout(300)
def test_lora_requests_match_merged_weights(tmp_path):
    base = str(tmp_path / "base")
    _base_ckpt(base)
    ad1, s1 = _write_adapter(str(tmp_path / "a1"), 1)
    ad2, s2 = _write_adapter(str(tmp_path / "a2"), 2, r=8, alpha=4.0)
    prompts = [[(5 * i + j) % 290 + 1 for j in range(6 + 3 * i)] for i in range(4)]
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    kw = dict(device="cpu", dtype="float32", max_model_len=128)
    want = {}
    for tag, ad, sc in (("a1", ad1, s1), ("a2", ad2, s2)):
        merged = str(tmp_path / f"merged_{tag}")
        _base_ckpt(merged, ad, sc)
        m = LLM(model=merged, **kw)
        want[tag] = [o.outputs[0].token_ids for o in m.generate([{"prompt_token_ids": p} for p in prompts], sp)]
        m.shutdown()
    llm = LLM(model=base, enable_lora=True, max_loras=2, **kw)
    plain = [o.outputs[0].token_ids for o in llm.generate([{"prompt_token_ids": p} for p in prompts], sp)]
    r1, r2 = LoRARequest("a1", 1, str(tmp_path / "a1")), LoRARequest("a2", 2, str(tmp_path / "a2"))
    # one batch mixing both adapters and no adapter
    mix = llm.generate([{"prompt_token_ids": p} for p in prompts], sp, lora_request=[r1, r2, None, r1])
    got = [o.outputs[0].token_ids for o in mix]
    assert got[0] == want["a1"][0] and got[1] == want["a2"][1] and got[2] == plain[2] and got[3] == want["a1"][3]
    assert want["a1"][0] != plain[0], "the adapter must change the output for the test to mean anything"
    assert sorted(llm.llm_engine.list_loras()) == [1, 2]
    assert llm.llm_engine.remove_lora(1) and llm.llm_engine.list_loras() == [2]
    # evicted adapters are reloaded on demand
    again = llm.generate([{"prompt_token_ids": prompts[0]}], sp, lora_request=r1)[0].outputs[0].token_ids
    assert again == want["a1"][0]
    llm.shutdown()
    with pytest.raises(ValueError):
        LLM(model=base, **kw).generate([{"prompt_token_ids": prompts[0]}], sp, lora_request=r1)


@pytest.mark.timeout(300)
def test_lora_under_tensor_parallelism_matches_single_rank(tmp_path):
    """Two gloo ranks: B of column-parallel layers and A of row-parallel layers are sharded per rank; the outputs must equal the
    single-rank run with the same adapters."""
    base = str(tmp_path / "base")
    _base_ckpt(base)
    _write_adapter(str(tmp_path / "a1"), 1)
    prompts = [[(5 * i + j) % 290 + 1 for j in range(6 + 3 * i)] for i in range(3)]
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    r1 = LoRARequest("a1", 1, str(tmp_path / "a1"))
    kw = dict(device="cpu", dtype="float32", max_model_len=128, enable_lora=True, max_loras=2)
    one = LLM(model=base, **kw)
    want = [o.outputs[0].token_ids for o in one.generate([{"prompt_token_ids": p} for p in prompts], sp, lora_request=[r1, None, r1])]
    one.shutdown()
    two = LLM(model=base, tensor_parallel_size=2, distributed_executor_backend="mp", **kw)
    got = [o.outputs[0].token_ids for o in two.generate([{"prompt_token_ids": p} for p in prompts], sp, lora_request=[r1, None, r1])]
    two.shutdown()
    assert got == want
