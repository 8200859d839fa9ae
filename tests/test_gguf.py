"""GGUF loading: the container reader and the block dequantisers against the ``gguf`` package, and a tiny model written as GGUF
(llama layout, q/k rows permuted as the converters do) that must generate the same tokens as its safetensors original."""
import numpy as np
import pytest
import torch

gguf = pytest.importorskip("gguf")

from onecat_vllm import LLM, SamplingParams  # noqa: E402
from onecat_vllm.loader import gguf as G  # noqa: E402


@pytest.mark.parametrize("name", ["Q8_0", "Q4_0", "Q4_1", "Q5_0", "Q5_1", "Q4_K", "Q5_K", "Q6_K", "Q2_K", "Q3_K", "F16", "BF16"])
def test_block_formats_match_the_gguf_package(name):
    from gguf import quants
    qt = gguf.GGMLQuantizationType[name]
    rng = np.random.default_rng(0)
    w = (rng.standard_normal((8, 512)) * 0.1).astype(np.float32)
    try:
        packed = quants.quantize(w, qt)
    except (NotImplementedError, quants.QuantError):
        # the package has no quantiser for this type: random blocks exercise the decoder just as well (finite scales only)
        _, bl, bb = G.GGML_TYPES[int(qt)]
        packed = rng.integers(0, 256, size=(8, 512 // bl * bb), dtype=np.uint8)
        halves = {"Q2_K": (80, 84), "Q3_K": (108, 110), "Q4_K": (0, 4), "Q5_K": (0, 4), "Q6_K": (208, 210)}[name]
        blocks = packed.reshape(-1, bb)
        blocks[:, halves[0]:halves[1]] = np.frombuffer(np.float16(0.01).tobytes() * ((halves[1] - halves[0]) // 2), dtype=np.uint8)
    want = quants.dequantize(packed, qt).astype(np.float32)
    got = G.dequantize(np.ascontiguousarray(packed).view(np.uint8).reshape(-1), int(qt)).float().numpy().reshape(want.shape)
    np.testing.assert_allclose(got, want, rtol=1e-6, atol=1e-7)


CFG = dict(architectures=["LlamaForCausalLM"], hidden_size=64, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
           num_key_value_heads=2, head_dim=16, vocab_size=320, max_position_embeddings=512, rms_norm_eps=1e-5, rope_theta=10000.0,
           eos_token_id=2, bos_token_id=1)


def _permute(w: np.ndarray, heads: int) -> np.ndarray:
    """What the HF -> GGUF converter does to llama q/k projections."""
    return w.reshape(heads, 2, w.shape[0] // heads // 2, *w.shape[1:]).swapaxes(1, 2).reshape(w.shape)


def _write_gguf(path, sd, qtype):
    from gguf import quants
    w = gguf.GGUFWriter(path, "llama")
    w.add_block_count(CFG["num_hidden_layers"])
    w.add_embedding_length(CFG["hidden_size"])
    w.add_feed_forward_length(CFG["intermediate_size"])
    w.add_head_count(CFG["num_attention_heads"])
    w.add_head_count_kv(CFG["num_key_value_heads"])
    w.add_layer_norm_rms_eps(CFG["rms_norm_eps"])
    w.add_rope_freq_base(CFG["rope_theta"])
    w.add_context_length(CFG["max_position_embeddings"])
    w.add_key_length(CFG["head_dim"])
    w.add_bos_token_id(1)
    w.add_eos_token_id(2)
    names = {"model.embed_tokens.weight": "token_embd.weight", "model.norm.weight": "output_norm.weight", "lm_head.weight": "output.weight"}
    parts = {"input_layernorm": "attn_norm", "post_attention_layernorm": "ffn_norm", "self_attn.q_proj": "attn_q", "self_attn.k_proj": "attn_k",
             "self_attn.v_proj": "attn_v", "self_attn.o_proj": "attn_output", "mlp.gate_proj": "ffn_gate", "mlp.up_proj": "ffn_up",
             "mlp.down_proj": "ffn_down"}
    stored = {}
    for k, v in sd.items():
        a = v.float().numpy()
        if k in names:
            gn = names[k]
        else:
            _, _, layer, rest = k.split(".", 3)
            part, suffix = rest.rsplit(".", 1)
            gn = f"blk.{layer}.{parts[part]}.{suffix}"
        if gn.endswith("attn_q.weight"):
            a = _permute(a, CFG["num_attention_heads"])
        if gn.endswith("attn_k.weight"):
            a = _permute(a, CFG["num_key_value_heads"])
        if a.ndim == 2 and qtype is not None and "token_embd" not in gn:
            packed = quants.quantize(a, qtype)
            w.add_tensor(gn, packed, raw_shape=packed.shape, raw_dtype=qtype)
            deq = quants.dequantize(packed, qtype).astype(np.float32)
            if gn.endswith("attn_q.weight"):
                deq = G._unpermute_llama(torch.from_numpy(deq), CFG["num_attention_heads"]).numpy()
            if gn.endswith("attn_k.weight"):
                deq = G._unpermute_llama(torch.from_numpy(deq), CFG["num_key_value_heads"]).numpy()
            stored[k] = torch.from_numpy(deq)
        else:
            w.add_tensor(gn, np.ascontiguousarray(a))
            stored[k] = v.float()
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()
    return stored


def _tiny_state_dict():
    from onecat_vllm.config import ModelConfig
    from onecat_vllm.loader.weights import dummy_init, to_hf_state_dict
    from onecat_vllm.models import build_model
    m = build_model(ModelConfig.from_hf_dict(CFG, dtype=torch.float32), "cpu")
    dummy_init(m, 0, std=0.08)
    return {k: v[: CFG["vocab_size"]] if ("embed_tokens" in k or k.startswith("lm_head")) else v for k, v in to_hf_state_dict(m).items()}


@pytest.mark.parametrize("qname", [None, "Q8_0"])
def test_gguf_model_generates_the_same_tokens_as_its_original(tmp_path, qname):
    from safetensors.torch import save_file
    import json
    sd = _tiny_state_dict()
    qtype = gguf.GGMLQuantizationType[qname] if qname else None
    gpath = str(tmp_path / "tiny.gguf")
    stored = _write_gguf(gpath, sd, qtype)

    f = G.GGUFFile(gpath)
    assert f.metadata["general.architecture"] == "llama" and int(f.metadata["llama.block_count"]) == 2
    hf = G.config_from_metadata(f.metadata, f.tensors)
    assert hf["num_key_value_heads"] == 2 and hf["head_dim"] == 16 and hf["vocab_size"] == 320 and not hf["tie_word_embeddings"]
    loaded = dict(G.iter_gguf(gpath))
    assert set(loaded) == set(stored)
    for k, v in stored.items():
        torch.testing.assert_close(loaded[k].float(), v, rtol=1e-6, atol=1e-7, msg=k)

    # the same (dequantised) weights as a safetensors checkpoint: both engines must produce the same greedy tokens
    ref_dir = tmp_path / "ref"
    ref_dir.mkdir()
    save_file({k: v.contiguous() for k, v in stored.items()}, str(ref_dir / "model.safetensors"))
    (ref_dir / "config.json").write_text(json.dumps(CFG))
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(3, 320, (n,), generator=g).tolist() for n in (9, 33)]
    sp = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)
    outs = []
    for model in (gpath, str(ref_dir)):
        llm = LLM(model=model, device="cpu", dtype="float32", max_model_len=128)
        outs.append([o.outputs[0].token_ids for o in llm.generate(prompts, sp)])
        llm.shutdown()
    assert outs[0] == outs[1]
