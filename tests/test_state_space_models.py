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


def test_nemotron_h_matches_hugging_face(tmp_path):
    """NemotronH: each block is one mixer. The installed transformers builds Mamba-2, attention (without positions) and expert blocks;
    the feed-forward blocks of the dense checkpoints are covered by the test below."""
    tr = pytest.importorskip("transformers")
    try:
        from transformers import NemotronHConfig, NemotronHForCausalLM
    except Exception as e:  # pragma: no cover
        pytest.skip(f"transformers has no NemotronH: {e}")
    cfg = NemotronHConfig(vocab_size=300, hidden_size=64, layers_block_type=["mamba", "attention", "mamba", "mamba", "attention"], num_attention_heads=4,
                          num_key_value_heads=2, head_dim=16, intermediate_size=128, ssm_state_size=16, mamba_num_heads=8, mamba_head_dim=16,
                          n_groups=2, conv_kernel=4, chunk_size=16, max_position_embeddings=256, tie_word_embeddings=False, pad_token_id=0,
                          bos_token_id=1, eos_token_id=2, use_mamba_kernels=False)
    torch.manual_seed(0)
    hf = NemotronHForCausalLM(cfg).float().eval()
    for n, p in hf.named_parameters():
        if "norm" not in n and "A_log" not in n and "dt_bias" not in n and n.rsplit(".", 1)[-1] != "D":
            torch.nn.init.normal_(p, std=0.15)
    _save(hf, tmp_path, "NemotronHForCausalLM")
    prompts = _prompts(300)
    llm = LLM(model=str(tmp_path), device="cpu", dtype="float32", max_model_len=256, max_num_batched_tokens=48)
    got = [o.outputs[0].token_ids for o in llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True))]
    llm.shutdown()
    # this random model's logits are flat (top-two gaps of 2e-4 occur, which fp32 rounding decides either way), so the check follows
    # the engine's own path: at every step its token must be Hugging Face's arg-max, or within 1e-3 of it in log-probability
    exact = 0
    for p, toks in zip(prompts, got):
        with torch.no_grad():
            lp = torch.log_softmax(hf(torch.tensor([p + toks])).logits[0, len(p) - 1: -1].float(), -1)
        for t, tok in enumerate(toks):
            assert lp[t, tok].item() >= lp[t].max().item() - 1e-3, (len(p), t, tok, int(lp[t].argmax()))
            exact += int(lp[t].argmax()) == tok
    assert exact >= 33     # of 36 steps


def test_nemotron_h_feed_forward_blocks(tmp_path):
    """The dense NemotronH pattern (M = Mamba-2, - = feed-forward, * = attention): a checkpoint under the family's own names loads
    completely, and the engine's tokens equal a plain forward over the same modules, whole prompt at once, with chunked prefill."""
    from onecat_vllm.config import ModelConfig
    from onecat_vllm.loader.weights import dummy_init, save_pretrained
    from onecat_vllm.models import build_model
    cfg = dict(architectures=["NemotronHForCausalLM"], vocab_size=300, hidden_size=64, hybrid_override_pattern="M-*-M-", num_attention_heads=4,
               num_key_value_heads=2, head_dim=16, intermediate_size=128, ssm_state_size=16, mamba_num_heads=8, mamba_head_dim=16, n_groups=2,
               conv_kernel=4, chunk_size=16, max_position_embeddings=256, tie_word_embeddings=False, mlp_hidden_act="relu2")
    mc = ModelConfig.from_hf_dict(cfg, dtype=torch.float32)
    assert [mc.layer_type(i) for i in range(6)] == ["mamba2", "ffn", "full_attention", "ffn", "mamba2", "ffn"]
    m = build_model(mc, "cpu")
    dummy_init(m, 0, std=0.15)
    save_pretrained(m, cfg, str(tmp_path))
    prompts = _prompts(300, (9, 70))
    sp = SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True)
    outs = []
    for budget in (8192, 32):
        llm = LLM(model=str(tmp_path), device="cpu", dtype="float32", max_model_len=256, max_num_batched_tokens=budget)
        outs.append([o.outputs[0].token_ids for o in llm.generate(prompts, sp)])
        llm.shutdown()
    assert outs[0] == outs[1]
    # the first generated token against a cache-free forward written out here: h += mixer(norm(h)) per block
    import torch.nn.functional as F
    layers = m.model.layers
    for p, got in zip(prompts, outs[0]):
        T = len(p)
        h = m.model.embed_tokens(torch.tensor(p))
        for i, layer in enumerate(layers):
            x = layer.input_layernorm(h, None)[0]
            kind = mc.layer_type(i)
            if kind == "ffn":
                y = layer.linear_attn.down_proj(F.relu(layer.linear_attn.up_proj(x)) ** 2)
            elif kind == "full_attention":
                a = layer.self_attn
                qkv = a.qkv_proj(x)
                q, k, v = qkv.split([a.Hq * a.D, a.Hkv * a.D, a.Hkv * a.D], -1)
                q, k, v = (t.view(T, -1, a.D).transpose(0, 1) for t in (q, k, v))
                o = F.scaled_dot_product_attention(q[None], k[None], v[None], is_causal=True, enable_gqa=True)[0]
                y = a.o_proj(o.transpose(0, 1).reshape(T, -1))
            else:
                mx = layer.linear_attn
                from types import SimpleNamespace
                md = SimpleNamespace(query_start_loc=torch.tensor([0, T]), state_slots=torch.tensor([0]), has_initial_state=torch.tensor([False]),
                                     gdn_record=None)
                (cd, kw), (hh, pp, nn_) = mx.state_shapes()
                y = mx(x, md, (torch.zeros(1, cd, kw), torch.zeros(1, hh, pp, nn_)))
            h = h + y
        logits = m.compute_logits(m.model.norm(h, None)[0][-1:])
        assert int(logits[0, :300].argmax()) == got[0]


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
