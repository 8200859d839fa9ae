"""Mamba-2 mixers: the chunked scan against the token-by-token recurrence, and Bamba (attention + Mamba-2 hybrid) and Mamba2ForCausalLM
served through the engine against Hugging Face (greedy tokens, chunked prefill included)."""
import json

import pytest
import torch

from onecat_vllm import LLM, SamplingParams
from onecat_vllm.ops import ref


def test_chunked_scan_equals_the_recurrence():
    torch.manual_seed(0)
    H, P, G, N = 4, 8, 2, 16
    lens = [1, 70, 5, 130]
    T = sum(lens)
    x, dt = torch.randn(T, H, P), torch.nn.functional.softplus(torch.randn(T, H))
    A, B, C, D = -torch.rand(H) - 0.1, torch.randn(T, G, N), torch.randn(T, G, N), torch.randn(H)
    st = torch.randn(6, H, P, N)
    st2 = st.clone()
    qsl = torch.tensor([0] + torch.tensor(lens).cumsum(0).tolist(), dtype=torch.int32)
    slots, hi = torch.tensor([3, 1, 0, 5]), torch.tensor([1, 0, 1, 1])
    y = ref.mamba2_scan(x, dt, A, B, C, D, st, qsl, slots, hi)
    want, o = torch.zeros(T, H, P), 0
    for r, L in enumerate(lens):
        h = st2[slots[r]].clone() if hi[r] else torch.zeros(H, P, N)
        for t in range(o, o + L):
            Bt, Ct = B[t].repeat_interleave(H // G, 0), C[t].repeat_interleave(H // G, 0)
            h = h * torch.exp(dt[t] * A).view(H, 1, 1) + (dt[t].view(H, 1) * x[t]).unsqueeze(-1) * Bt.unsqueeze(1)
            want[t] = torch.einsum("hpn,hn->hp", h, Ct) + D.view(H, 1) * x[t]
        st2[slots[r]] = h
        o += L
    assert torch.allclose(y, want, atol=5e-4, rtol=5e-4) and torch.allclose(st, st2, atol=1e-4, rtol=1e-4)


def _save(hf, path, arch):
    hf.save_pretrained(str(path), safe_serialization=True)
    d = json.loads((path / "config.json").read_text())
    d["architectures"] = [arch]
    (path / "config.json").write_text(json.dumps(d))


def _prompts(vocab, lens=(5, 23, 70)):
    g = torch.Generator().manual_seed(3)
    return [torch.randint(3, vocab, (n,), generator=g).tolist() for n in lens]


def _hf_greedy(hf, prompts, n):
    out = []
    with torch.no_grad():
        for p in prompts:
            ids = torch.tensor([p])
            o = hf.generate(input_ids=ids, attention_mask=torch.ones_like(ids), max_new_tokens=n, do_sample=False, eos_token_id=None, pad_token_id=0)
            out.append(o[0, len(p):].tolist())
    return out


@pytest.mark.parametrize("budget", [8192, 32])
def test_bamba_matches_hugging_face(tmp_path, budget):
    tr = pytest.importorskip("transformers")
    try:
        from transformers import BambaConfig, BambaForCausalLM
    except Exception as e:  # pragma: no cover
        pytest.skip(f"transformers has no Bamba: {e}")
    cfg = BambaConfig(vocab_size=300, hidden_size=64, intermediate_size=128, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2,
                      attn_layer_indices=[1, 3], mamba_n_heads=8, mamba_d_head=16, mamba_n_groups=1, mamba_d_state=16, mamba_d_conv=4,
                      mamba_expand=2, mamba_chunk_size=16, max_position_embeddings=512, tie_word_embeddings=False, pad_token_id=0)
    torch.manual_seed(0)
    hf = BambaForCausalLM(cfg).float().eval()
    for n, p in hf.named_parameters():
        if "norm" not in n and "A_log" not in n and "dt_bias" not in n and n.rsplit(".", 1)[-1] != "D":
            torch.nn.init.normal_(p, std=0.15)
    _save(hf, tmp_path, "BambaForCausalLM")
    # Bamba rotates the first half of each head (partial_rotary_factor 0.5, ``attn_rotary_emb`` in the original config). The rotary
    # module of this transformers version builds its frequencies over the whole head; give it the half-width table the model defines
    rd = 8
    inv = 1.0 / (10000.0 ** (torch.arange(0, rd, 2, dtype=torch.float32) / rd))
    hf.model.rotary_emb.inv_freq = inv
    hf.model.rotary_emb.original_inv_freq = inv.clone()
    prompts = _prompts(300)
    want = _hf_greedy(hf, prompts, 12)
    llm = LLM(model=str(tmp_path), device="cpu", dtype="float32", max_model_len=256, max_num_batched_tokens=budget)
    got = [o.outputs[0].token_ids for o in llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True))]
    llm.shutdown()
    assert got == want


def test_mamba2_matches_hugging_face(tmp_path):
    tr = pytest.importorskip("transformers")
    try:
        from transformers import Mamba2Config, Mamba2ForCausalLM
    except Exception as e:  # pragma: no cover
        pytest.skip(f"transformers has no Mamba2: {e}")
    cfg = Mamba2Config(vocab_size=300, hidden_size=64, num_hidden_layers=3, num_heads=8, head_dim=16, state_size=16, n_groups=1, expand=2,
                       conv_kernel=4, chunk_size=16, tie_word_embeddings=True, pad_token_id=0, bos_token_id=1, eos_token_id=2)
    torch.manual_seed(0)
    hf = Mamba2ForCausalLM(cfg).float().eval()
    for n, p in hf.named_parameters():
        if "norm" not in n and "A_log" not in n and "dt_bias" not in n and n.rsplit(".", 1)[-1] != "D":
            torch.nn.init.normal_(p, std=0.15)
    _save(hf, tmp_path, "Mamba2ForCausalLM")
    prompts = _prompts(300)
    want = _hf_greedy(hf, prompts, 12)
    llm = LLM(model=str(tmp_path), device="cpu", dtype="float32", max_model_len=256, max_num_batched_tokens=48)
    got = [o.outputs[0].token_ids for o in llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True))]
    llm.shutdown()
    assert got == want


@pytest.mark.parametrize("falcon", [False, True])
def test_mamba1_matches_hugging_face(tmp_path, falcon):
    tr = pytest.importorskip("transformers")
    try:
        from transformers import FalconMambaConfig, FalconMambaForCausalLM, MambaConfig, MambaForCausalLM
    except Exception as e:  # pragma: no cover
        pytest.skip(f"transformers has no Mamba: {e}")
    Cfg, Model = (FalconMambaConfig, FalconMambaForCausalLM) if falcon else (MambaConfig, MambaForCausalLM)
    cfg = Cfg(vocab_size=300, hidden_size=64, num_hidden_layers=3, state_size=8, expand=2, conv_kernel=4, time_step_rank=6,
              tie_word_embeddings=True, pad_token_id=0, bos_token_id=1, eos_token_id=2)
    torch.manual_seed(0)
    hf = Model(cfg).float().eval()
    for n, p in hf.named_parameters():
        if "norm" not in n and "A_log" not in n and n.rsplit(".", 1)[-1] != "D" and "dt_proj.bias" not in n:
            torch.nn.init.normal_(p, std=0.15)
    _save(hf, tmp_path, "FalconMambaForCausalLM" if falcon else "MambaForCausalLM")
    prompts = _prompts(300)
    want = _hf_greedy(hf, prompts, 12)
    llm = LLM(model=str(tmp_path), device="cpu", dtype="float32", max_model_len=256, max_num_batched_tokens=48)
    got = [o.outputs[0].token_ids for o in llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True))]
    llm.shutdown()
    assert got == want


@pytest.mark.parametrize("experts", [0, 4])
def test_granite_hybrid_matches_hugging_face(tmp_path, experts):
    tr = pytest.importorskip("transformers")
    try:
        from transformers import GraniteMoeHybridConfig, GraniteMoeHybridForCausalLM
    except Exception as e:  # pragma: no cover
        pytest.skip(f"transformers has no GraniteMoeHybrid: {e}")
    cfg = GraniteMoeHybridConfig(vocab_size=300, hidden_size=64, intermediate_size=48, shared_intermediate_size=96, num_hidden_layers=4,
                                 num_attention_heads=4, num_key_value_heads=2, layer_types=["mamba", "attention", "mamba", "attention"],
                                 num_local_experts=experts, num_experts_per_tok=2 if experts else 0, mamba_n_heads=8, mamba_d_head=16,
                                 mamba_n_groups=1, mamba_d_state=16, mamba_d_conv=4, mamba_expand=2, mamba_chunk_size=16,
                                 embedding_multiplier=3.0, residual_multiplier=0.5, attention_multiplier=0.2, logits_scaling=4.0,
                                 position_embedding_type="nope", max_position_embeddings=512, tie_word_embeddings=False, pad_token_id=0)
    torch.manual_seed(0)
    hf = GraniteMoeHybridForCausalLM(cfg).float().eval()
    for n, p in hf.named_parameters():
        if "norm" not in n and "A_log" not in n and "dt_bias" not in n and n.rsplit(".", 1)[-1] != "D":
            torch.nn.init.normal_(p, std=0.15)
    _save(hf, tmp_path, "GraniteMoeHybridForCausalLM")
    prompts = _prompts(300)
    want = _hf_greedy(hf, prompts, 12)
    llm = LLM(model=str(tmp_path), device="cpu", dtype="float32", max_model_len=256, max_num_batched_tokens=48)
    got = [o.outputs[0].token_ids for o in llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True))]
    llm.shutdown()
    assert got == want


def test_jamba_matches_hugging_face(tmp_path):
    tr = pytest.importorskip("transformers")
    try:
        from transformers import JambaConfig, JambaForCausalLM
    except Exception as e:  # pragma: no cover
        pytest.skip(f"transformers has no Jamba: {e}")
    cfg = JambaConfig(vocab_size=300, hidden_size=64, intermediate_size=96, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2,
                      num_experts=4, num_experts_per_tok=2, attn_layer_period=2, attn_layer_offset=1, expert_layer_period=2, expert_layer_offset=1,
                      mamba_d_state=8, mamba_d_conv=4, mamba_expand=2, mamba_dt_rank=6, use_mamba_kernels=False, max_position_embeddings=512,
                      tie_word_embeddings=False, pad_token_id=0)
    torch.manual_seed(0)
    hf = JambaForCausalLM(cfg).float().eval()
    for n, p in hf.named_parameters():
        if "norm" not in n and "A_log" not in n and n.rsplit(".", 1)[-1] != "D" and "dt_proj.bias" not in n:
            torch.nn.init.normal_(p, std=0.15)
    _save(hf, tmp_path, "JambaForCausalLM")
    prompts = _prompts(300)
    want = _hf_greedy(hf, prompts, 12)
    llm = LLM(model=str(tmp_path), device="cpu", dtype="float32", max_model_len=256, max_num_batched_tokens=48)
    got = [o.outputs[0].token_ids for o in llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True))]
    llm.shutdown()
    assert got == want


def test_lfm2_short_conv_matches_hugging_face(tmp_path):
    tr = pytest.importorskip("transformers")
    try:
        from transformers import Lfm2Config, Lfm2ForCausalLM
    except Exception as e:  # pragma: no cover
        pytest.skip(f"transformers has no LFM2: {e}")
    cfg = Lfm2Config(vocab_size=300, hidden_size=64, intermediate_size=200, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2,
                     layer_types=["conv", "conv", "full_attention", "conv"], block_multiple_of=16, max_position_embeddings=512, pad_token_id=0)
    torch.manual_seed(0)
    hf = Lfm2ForCausalLM(cfg).float().eval()
    for n, p in hf.named_parameters():
        if "norm" not in n:
            torch.nn.init.normal_(p, std=0.15)
    _save(hf, tmp_path, "Lfm2ForCausalLM")
    prompts = _prompts(300)
    want = _hf_greedy(hf, prompts, 12)
    llm = LLM(model=str(tmp_path), device="cpu", dtype="float32", max_model_len=256, max_num_batched_tokens=48)
    got = [o.outputs[0].token_ids for o in llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True))]
    llm.shutdown()
    assert got == want


def test_lfm2_moe_matches_hugging_face(tmp_path):
    tr = pytest.importorskip("transformers")
    try:
        from transformers import Lfm2MoeConfig, Lfm2MoeForCausalLM
    except Exception as e:  # pragma: no cover
        pytest.skip(f"transformers has no LFM2-MoE: {e}")
    cfg = Lfm2MoeConfig(vocab_size=300, hidden_size=64, intermediate_size=128, moe_intermediate_size=48, num_hidden_layers=4, num_attention_heads=4,
                        num_key_value_heads=2, layer_types=["conv", "full_attention", "conv", "conv"], num_dense_layers=1, num_experts=4,
                        num_experts_per_tok=2, routed_scaling_factor=1.5, max_position_embeddings=512, pad_token_id=0)
    torch.manual_seed(0)
    hf = Lfm2MoeForCausalLM(cfg).float().eval()
    for n, p in hf.named_parameters():
        if "norm" not in n:
            torch.nn.init.normal_(p, std=0.15)
    for n, b in hf.named_buffers():
        if n.endswith("expert_bias"):
            b.normal_(0.0, 0.1, generator=torch.Generator().manual_seed(4))
    _save(hf, tmp_path, "Lfm2MoeForCausalLM")
    prompts = _prompts(300)
    want = _hf_greedy(hf, prompts, 12)
    llm = LLM(model=str(tmp_path), device="cpu", dtype="float32", max_model_len=256, max_num_batched_tokens=48)
    got = [o.outputs[0].token_ids for o in llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True))]
    llm.shutdown()
    assert got == want
