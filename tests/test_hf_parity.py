"""Checkpoint-format and model-math parity with Hugging Face transformers on CPU: a tiny randomly initialised HF model is saved with
``save_pretrained`` and loaded by this engine; greedy continuations and first-token log-probabilities must match
(reference test model: tests/models/language/generation/test_common.py — vLLM vs HF runner)."""
import pytest
import torch

transformers = pytest.importorskip("transformers")

BASE = dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, vocab_size=320,
            max_position_embeddings=256, rms_norm_eps=1e-6, tie_word_embeddings=False)
CASES = {
    "LlamaForCausalLM": dict(BASE, model_type="llama", rope_theta=10000.0),
    "MistralForCausalLM": dict(BASE, model_type="mistral", rope_theta=10000.0, sliding_window=None),
    "Qwen2ForCausalLM": dict(BASE, model_type="qwen2", rope_theta=1e6),
    "Qwen3ForCausalLM": dict(BASE, model_type="qwen3", head_dim=32, rope_theta=1e6),
    "Qwen3MoeForCausalLM": dict(BASE, model_type="qwen3_moe", head_dim=32, rope_theta=1e6, num_experts=8, num_experts_per_tok=2,
                                moe_intermediate_size=64, norm_topk_prob=True, decoder_sparse_step=1, mlp_only_layers=[]),
    "MixtralForCausalLM": dict(BASE, model_type="mixtral", rope_theta=1e6, num_local_experts=4, num_experts_per_tok=2),
    "Qwen2MoeForCausalLM": dict(BASE, model_type="qwen2_moe", rope_theta=1e6, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=64,
                                shared_expert_intermediate_size=96, norm_topk_prob=False, decoder_sparse_step=1, mlp_only_layers=[]),
    "DeepseekV3ForCausalLM": dict(BASE, model_type="deepseek_v3", num_key_value_heads=4, rope_theta=10000.0, q_lora_rank=32, kv_lora_rank=32,
                                  qk_nope_head_dim=16, qk_rope_head_dim=16, v_head_dim=16, n_routed_experts=8, n_shared_experts=1,
                                  num_experts_per_tok=2, moe_intermediate_size=48, n_group=2, topk_group=1, routed_scaling_factor=1.5,
                                  norm_topk_prob=True, first_k_dense_replace=1, scoring_func="sigmoid", rope_scaling=None),
    "Qwen3_5ForCausalLM": dict(BASE, model_type="qwen3_5_text", head_dim=32, num_hidden_layers=4, full_attention_interval=2,
                               linear_num_key_heads=2, linear_num_value_heads=4, linear_key_head_dim=16, linear_value_head_dim=16,
                               linear_conv_kernel_dim=4, rope_parameters={"rope_type": "default", "rope_theta": 1e6, "partial_rotary_factor": 0.5}),
    "Qwen3_5MoeForCausalLM": dict(BASE, model_type="qwen3_5_moe_text", head_dim=32, num_hidden_layers=4, full_attention_interval=2,
                                  linear_num_key_heads=2, linear_num_value_heads=4, linear_key_head_dim=16, linear_value_head_dim=16,
                                  linear_conv_kernel_dim=4, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=64,
                                  shared_expert_intermediate_size=64,
                                  rope_parameters={"rope_type": "default", "rope_theta": 1e6, "partial_rotary_factor": 0.5}),
    "DeepseekV2ForCausalLM": dict(BASE, model_type="deepseek_v2", num_key_value_heads=4, rope_theta=10000.0, q_lora_rank=None, kv_lora_rank=32,
                                  qk_nope_head_dim=16, qk_rope_head_dim=16, v_head_dim=16, n_routed_experts=4, n_shared_experts=1,
                                  num_experts_per_tok=2, moe_intermediate_size=48, n_group=1, topk_group=1, routed_scaling_factor=1.0,
                                  norm_topk_prob=False, first_k_dense_replace=1, scoring_func="softmax", topk_method="greedy", rope_scaling=None),
    "Phi3ForCausalLM": dict(BASE, model_type="phi3", rope_theta=10000.0, pad_token_id=0),
    "SeedOssForCausalLM": dict(BASE, model_type="seed_oss", head_dim=16, rope_theta=10000.0),
    "Qwen3NextForCausalLM": dict(BASE, model_type="qwen3_next", head_dim=32, rope_theta=1e6, partial_rotary_factor=0.5, num_hidden_layers=4,
                                 full_attention_interval=2, linear_num_key_heads=2, linear_num_value_heads=4, linear_key_head_dim=16,
                                 linear_value_head_dim=16, linear_conv_kernel_dim=4, num_experts=4, num_experts_per_tok=2,
                                 moe_intermediate_size=64, shared_expert_intermediate_size=64, norm_topk_prob=True, decoder_sparse_step=1,
                                 mlp_only_layers=[]),
    "GemmaForCausalLM": dict(BASE, model_type="gemma", head_dim=32, rope_theta=10000.0, tie_word_embeddings=True),
    "Gemma2ForCausalLM": dict(BASE, model_type="gemma2", head_dim=32, rope_theta=10000.0, tie_word_embeddings=True, num_hidden_layers=4,
                              sliding_window=16, query_pre_attn_scalar=24, attn_logit_softcapping=5.0, final_logit_softcapping=8.0),
    "Gemma3ForCausalLM": dict(BASE, model_type="gemma3_text", head_dim=32, tie_word_embeddings=True, num_hidden_layers=4, sliding_window=16,
                              query_pre_attn_scalar=24, layer_types=["sliding_attention", "sliding_attention", "sliding_attention", "full_attention"],
                              rope_parameters={"sliding_attention": {"rope_type": "default", "rope_theta": 10000.0},
                                               "full_attention": {"rope_type": "linear", "factor": 4.0, "rope_theta": 1e6}}),
    "GlmForCausalLM": dict(BASE, model_type="glm", head_dim=16, rope_theta=10000.0, partial_rotary_factor=0.5, attention_bias=True, pad_token_id=0),
    "Glm4ForCausalLM": dict(BASE, model_type="glm4", head_dim=16, rope_theta=10000.0, partial_rotary_factor=0.5, attention_bias=True, pad_token_id=0),
    "Glm4MoeForCausalLM": dict(BASE, model_type="glm4_moe", head_dim=16, rope_theta=10000.0, partial_rotary_factor=0.5, n_routed_experts=8,
                               n_shared_experts=1, num_experts_per_tok=2, moe_intermediate_size=48, n_group=1, topk_group=1,
                               routed_scaling_factor=1.5, norm_topk_prob=True, first_k_dense_replace=1, use_qk_norm=True, pad_token_id=0),
    "GraniteForCausalLM": dict(BASE, model_type="granite", rope_theta=10000.0, embedding_multiplier=6.0, residual_multiplier=0.3,
                               attention_multiplier=0.2, logits_scaling=4.0),
    "LlamaForCausalLM+llama3-rope": dict(BASE, model_type="llama", rope_parameters={"rope_type": "llama3", "rope_theta": 10000.0, "factor": 8.0,
                                         "low_freq_factor": 1.0, "high_freq_factor": 4.0, "original_max_position_embeddings": 32}),
    "LlamaForCausalLM+yarn-rope": dict(BASE, model_type="llama", rope_parameters={"rope_type": "yarn", "rope_theta": 10000.0, "factor": 4.0,
                                       "original_max_position_embeddings": 32}),
    "DeepseekV3ForCausalLM+yarn": dict(BASE, model_type="deepseek_v3", num_key_value_heads=4, q_lora_rank=32, kv_lora_rank=32,
                                       qk_nope_head_dim=16, qk_rope_head_dim=16, v_head_dim=16, n_routed_experts=8, n_shared_experts=1,
                                       num_experts_per_tok=2, moe_intermediate_size=48, n_group=2, topk_group=1, routed_scaling_factor=1.5,
                                       norm_topk_prob=True, first_k_dense_replace=1, scoring_func="sigmoid",
                                       rope_parameters={"rope_type": "yarn", "rope_theta": 10000.0, "factor": 8.0, "beta_fast": 32, "beta_slow": 1,
                                                        "mscale": 1.0, "mscale_all_dim": 1.0, "original_max_position_embeddings": 32}),
    "SmolLM3ForCausalLM": dict(BASE, model_type="smollm3", num_hidden_layers=4, no_rope_layers=[1, 1, 1, 0], rope_theta=10000.0, pad_token_id=0),
    "Olmo2ForCausalLM": dict(BASE, model_type="olmo2", rope_theta=10000.0, pad_token_id=0),
    "Olmo3ForCausalLM": dict(BASE, model_type="olmo3", num_hidden_layers=4, sliding_window=16, rope_theta=10000.0, pad_token_id=0,
                             layer_types=["sliding_attention", "sliding_attention", "sliding_attention", "full_attention"]),
    "OlmoeForCausalLM": dict(BASE, model_type="olmoe", rope_theta=10000.0, num_experts=8, num_experts_per_tok=2, norm_topk_prob=False, pad_token_id=0),
    "Ernie4_5ForCausalLM": dict(BASE, model_type="ernie4_5", head_dim=16, rope_theta=10000.0, use_bias=False, pad_token_id=0),
    "Exaone4ForCausalLM": dict(BASE, model_type="exaone4", head_dim=16, num_hidden_layers=4, sliding_window=16, sliding_window_pattern=4,
                               layer_types=["sliding_attention", "sliding_attention", "sliding_attention", "full_attention"], rope_theta=10000.0, pad_token_id=0),
    "MinistralForCausalLM": dict(BASE, model_type="ministral", head_dim=16, num_hidden_layers=4, sliding_window=16, rope_theta=10000.0, pad_token_id=0,
                                 layer_types=["sliding_attention", "full_attention", "sliding_attention", "full_attention"]),
    "Dots1ForCausalLM": dict(BASE, model_type="dots1", head_dim=16, rope_theta=10000.0, n_routed_experts=8, n_shared_experts=1, num_experts_per_tok=2,
                             moe_intermediate_size=48, n_group=1, topk_group=1, routed_scaling_factor=1.5, norm_topk_prob=True,
                             first_k_dense_replace=1, pad_token_id=0),
    "HeliumForCausalLM": dict(BASE, model_type="helium", head_dim=16, rope_theta=10000.0, pad_token_id=0),
    "CwmForCausalLM": dict(BASE, model_type="cwm", head_dim=16, num_hidden_layers=4, sliding_window=16, pad_token_id=0,
                           layer_types=["full_attention", "sliding_attention", "sliding_attention", "sliding_attention"],
                           rope_parameters={"rope_type": "llama3", "rope_theta": 10000.0, "factor": 4.0, "high_freq_factor": 4.0,
                                            "low_freq_factor": 1.0, "original_max_position_embeddings": 32}),
    "HunYuanDenseV1ForCausalLM": dict(BASE, model_type="hunyuan_v1_dense", head_dim=16, rope_theta=10000.0, use_qk_norm=True, pad_token_id=0),
    "GraniteMoeForCausalLM": dict(BASE, model_type="granitemoe", intermediate_size=48, rope_theta=10000.0, num_local_experts=4, num_experts_per_tok=2,
                                  embedding_multiplier=6.0, residual_multiplier=0.3, attention_multiplier=0.2, logits_scaling=4.0, pad_token_id=0),
    "Ernie4_5_MoeForCausalLM": dict(BASE, model_type="ernie4_5_moe", head_dim=16, num_hidden_layers=3, rope_theta=10000.0, moe_intermediate_size=48,
                                    moe_num_experts=8, moe_k=2, moe_num_shared_experts=1, moe_layer_start_index=1, moe_layer_end_index=2,
                                    moe_layer_interval=1, use_bias=False, pad_token_id=0),
    "GptOssForCausalLM": dict(BASE, model_type="gpt_oss", head_dim=16, num_hidden_layers=4, intermediate_size=48, num_local_experts=4,
                              num_experts_per_tok=2, sliding_window=16, pad_token_id=0,
                              layer_types=["sliding_attention", "full_attention", "sliding_attention", "full_attention"],
                              rope_parameters={"rope_type": "yarn", "rope_theta": 10000.0, "factor": 4.0, "beta_fast": 32.0, "beta_slow": 1.0,
                                               "truncate": False, "original_max_position_embeddings": 32}),
    "Phi3ForCausalLM+window": dict(BASE, model_type="phi3", rope_theta=10000.0, pad_token_id=0, sliding_window=16),
    "Phi3ForCausalLM+longrope": dict(BASE, model_type="phi3", pad_token_id=0, max_position_embeddings=512, original_max_position_embeddings=256,
                                     rope_parameters={"rope_type": "longrope", "rope_theta": 10000.0, "original_max_position_embeddings": 256,
                                                      "short_factor": [1.0 + 0.1 * i for i in range(8)], "long_factor": [2.0 + 0.3 * i for i in range(8)]}),
    "LlamaForCausalLM+attention-bias": dict(BASE, model_type="llama", rope_theta=10000.0, attention_bias=True),
    "Qwen3ForCausalLM+attention-bias": dict(BASE, model_type="qwen3", head_dim=32, rope_theta=1e6, attention_bias=True),
    "SeedOssForCausalLM+out-bias": dict(BASE, model_type="seed_oss", head_dim=16, rope_theta=10000.0, attention_bias=True, attention_out_bias=True),
    "LlamaForCausalLM+mlp-bias": dict(BASE, model_type="llama", rope_theta=10000.0, mlp_bias=True),
    "MistralForCausalLM+window": dict(BASE, model_type="mistral", rope_theta=10000.0, sliding_window=16),
    "GraniteMoeSharedForCausalLM": dict(BASE, model_type="granitemoeshared", intermediate_size=48, shared_intermediate_size=80, rope_theta=10000.0,
                                        num_local_experts=4, num_experts_per_tok=2, embedding_multiplier=6.0, residual_multiplier=0.3,
                                        attention_multiplier=0.2, logits_scaling=4.0, pad_token_id=0),
    "HunYuanMoEV1ForCausalLM": dict(BASE, model_type="hunyuan_v1_moe", head_dim=16, rope_theta=10000.0, num_experts=4, moe_topk=2, pad_token_id=0),
    "Ministral3ForCausalLM": dict(BASE, model_type="ministral3", head_dim=16, pad_token_id=0),
    "VaultGemmaForCausalLM": dict(BASE, model_type="vaultgemma", head_dim=16, pad_token_id=0),
    "FlexOlmoForCausalLM": dict(BASE, model_type="flex_olmo", num_experts=4, num_experts_per_tok=2, pad_token_id=0),
    "ExaoneMoeForCausalLM": dict(BASE, model_type="exaone_moe", head_dim=16, num_hidden_layers=4, num_experts=8, num_experts_per_tok=2,
                                 moe_intermediate_size=48, n_group=2, topk_group=1, routed_scaling_factor=1.5, sliding_window=16, sliding_window_pattern=2,
                                 layer_types=["sliding_attention", "full_attention", "sliding_attention", "full_attention"],
                                 mlp_layer_types=["dense", "sparse", "sparse", "sparse"], pad_token_id=0),
    "SolarOpenForCausalLM": dict(BASE, model_type="solar_open", head_dim=16, n_routed_experts=8, num_experts_per_tok=2, moe_intermediate_size=48,
                                 n_group=2, topk_group=1, routed_scaling_factor=1.5, pad_token_id=0),
    "Glm4MoeLiteForCausalLM": dict(BASE, model_type="glm4_moe_lite", num_key_value_heads=4, q_lora_rank=32, kv_lora_rank=32, qk_nope_head_dim=16,
                                   qk_rope_head_dim=16, v_head_dim=16, n_routed_experts=8, num_experts_per_tok=2, moe_intermediate_size=48,
                                   routed_scaling_factor=1.5, mlp_layer_types=["dense", "sparse"], pad_token_id=0),
    "ArceeForCausalLM": dict(BASE, model_type="arcee", head_dim=16, rope_theta=10000.0, pad_token_id=0),
    # mean-and-variance layer norms: without parameters (OLMo, with the q/k/v clamp), with weight and bias, with the weight stored minus one
    "OlmoForCausalLM": dict(BASE, model_type="olmo", clip_qkv=0.8, pad_token_id=0),
    "StableLmForCausalLM": dict(BASE, model_type="stablelm", use_qkv_bias=True, partial_rotary_factor=0.25, pad_token_id=0),
    "Starcoder2ForCausalLM": dict(BASE, model_type="starcoder2", sliding_window=16, use_bias=True, pad_token_id=0),
    "NemotronForCausalLM": dict(BASE, model_type="nemotron", partial_rotary_factor=0.5, pad_token_id=0),
    # attention and feed-forward in parallel off one layer norm; in the second form only the sliding-window layers rotate
    "CohereForCausalLM": dict(BASE, model_type="cohere", logit_scale=0.25, pad_token_id=0, tie_word_embeddings=True),
    "Cohere2ForCausalLM": dict(BASE, model_type="cohere2", num_hidden_layers=4, logit_scale=0.25, sliding_window=16, pad_token_id=0, tie_word_embeddings=True,
                               layer_types=["sliding_attention", "sliding_attention", "sliding_attention", "full_attention"]),
    "Jais2ForCausalLM": dict(BASE, model_type="jais2", attention_bias=True, mlp_bias=True, pad_token_id=0),
    "MiniMaxM2ForCausalLM": dict(BASE, model_type="minimax_m2", head_dim=16, intermediate_size=48, num_local_experts=8, num_experts_per_tok=2,
                                 pad_token_id=0),
}


@pytest.mark.timeout(600)
@pytest.mark.parametrize("arch", list(CASES))
def test_greedy_tokens_and_logprobs_match_transformers(arch, tmp_path):
    from onecat_vllm import LLM, SamplingParams
    cfg_cls = transformers.AutoConfig.for_model(CASES[arch]["model_type"], **{k: v for k, v in CASES[arch].items() if k != "model_type"})
    case, arch = arch, arch.split("+")[0]
    cfg_cls.architectures = [arch]
    torch.manual_seed(0)
    hf = getattr(transformers, arch)(cfg_cls).eval().float()
    for p in hf.parameters():  # widen the logit gaps so that greedy choices are not near-ties
        if p.dim() >= 2:
            p.data.mul_(3.0)
    gb = torch.Generator().manual_seed(6)
    for n, p in hf.named_parameters():   # biases and attention sinks start at zero or tiny: make them matter
        if (n.endswith("bias") or n.endswith("sinks")) and "e_score_correction_bias" not in n:
            p.data.normal_(0.0, 0.2, generator=gb)
    for n, p in list(hf.named_parameters()) + list(hf.named_buffers()):
        if "e_score_correction_bias" in n:  # zero at initialisation: give the router's selection bias something to do
            p.data.normal_(0.0, 0.05, generator=torch.Generator().manual_seed(4))
    hf.save_pretrained(str(tmp_path), safe_serialization=True)
    hf.generation_config.eos_token_id = None   # the engine runs with ignore_eos
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(1, 300, (n,), generator=g).tolist() for n in (5, 23, 40)]
    llm = LLM(model=str(tmp_path), device="cpu", dtype="float32", max_model_len=128)
    outs = llm.generate([{"prompt_token_ids": p} for p in prompts], SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True, logprobs=0))
    llm.shutdown()
    for p, o in zip(prompts, outs):
        ids = torch.tensor([p])
        with torch.no_grad():
            ref = hf.generate(ids, max_new_tokens=8, do_sample=False, pad_token_id=0)[0, len(p):].tolist()
            lp = torch.log_softmax(hf(ids).logits[0, -1].float(), -1)
        got = o.outputs[0].token_ids
        assert got == ref, f"{arch}: {got} vs {ref}"
        first = o.outputs[0].logprobs[0][got[0]].logprob
        assert abs(first - lp[ref[0]].item()) < 2e-3, (arch, first, lp[ref[0]].item())


@pytest.mark.timeout(900)
def test_cpu_plumbing_run_matches_transformers():
    """The benchmark plan's CPU plumbing configuration: tiny Llama-style fp32 decoder (4 layers, hidden 256, 8 q / 2 kv heads of 32,
    FFN 688, vocab 32000, untied head, RoPE theta 1e6, N(0, 0.02) weights from seed 0), 32 requests with prompts of 16..128 random
    tokens, 64 greedy tokens each with ignore_eos, through the engine (continuous batching, paged KV, block 16) against
    ``transformers`` greedy generation."""
    import tempfile
    from onecat_vllm import LLM, SamplingParams
    cfg = transformers.LlamaConfig(hidden_size=256, intermediate_size=688, num_hidden_layers=4, num_attention_heads=8, num_key_value_heads=2,
                                   head_dim=32, vocab_size=32000, rms_norm_eps=1e-6, rope_theta=1e6, max_position_embeddings=512,
                                   tie_word_embeddings=False, initializer_range=0.02)
    cfg.architectures = ["LlamaForCausalLM"]
    torch.manual_seed(0)
    hf = transformers.LlamaForCausalLM(cfg).eval().float()
    g = torch.Generator().manual_seed(0)
    lens = torch.randint(16, 129, (32,), generator=g).tolist()
    prompts = [torch.randint(0, 32000, (n,), generator=g).tolist() for n in lens]
    with tempfile.TemporaryDirectory() as d:
        hf.save_pretrained(d, safe_serialization=True)
        llm = LLM(model=d, device="cpu", dtype="float32", max_model_len=256, block_size=16, max_num_seqs=32, max_num_batched_tokens=512)
        outs = llm.generate([{"prompt_token_ids": p} for p in prompts], SamplingParams(temperature=0.0, max_tokens=64, ignore_eos=True))
        llm.shutdown()
    exact = total = 0
    for p, o in zip(prompts, outs):
        with torch.no_grad():
            ref = hf.generate(torch.tensor([p]), max_new_tokens=64, do_sample=False, pad_token_id=0)[0, len(p):].tolist()
        got = o.outputs[0].token_ids
        assert len(got) == 64
        n = next((i for i, (a, b) in enumerate(zip(got, ref)) if a != b), 64)
        exact += n == 64
        total += n
    # N(0, 0.02) weights make the logits nearly flat, so a last-bit difference in summation order can flip a greedy choice;
    # everything before the first such flip must agree
    assert exact >= 30 and total >= 0.97 * 32 * 64, (exact, total)


@pytest.mark.timeout(600)
def test_sequence_classification_matches_transformers(tmp_path):
    """A *ForSequenceClassification checkpoint: ``LLM.classify`` returns softmax(score(last hidden state)) as transformers does
    (reference: models/adapters.py ``as_seq_cls_model``; entrypoints/llm.py ``classify``)."""
    from onecat_vllm import LLM
    from onecat_vllm.sampling_params import PoolingParams
    cfg = transformers.Qwen2Config(**{k: v for k, v in BASE.items()}, rope_theta=1e6, num_labels=3, pad_token_id=0)
    cfg.architectures = ["Qwen2ForSequenceClassification"]
    torch.manual_seed(0)
    hf = transformers.Qwen2ForSequenceClassification(cfg).eval().float()
    for p in hf.parameters():
        if p.dim() >= 2:
            p.data.mul_(3.0)
    hf.save_pretrained(str(tmp_path), safe_serialization=True)
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(1, 300, (n,), generator=g).tolist() for n in (7, 33)]
    llm = LLM(model=str(tmp_path), device="cpu", dtype="float32", max_model_len=128)
    outs = llm.classify([{"prompt_token_ids": p} for p in prompts])
    raw = llm.encode([{"prompt_token_ids": prompts[0]}], PoolingParams(task="classify", normalize=False, use_activation=False))
    llm.shutdown()
    for p, o in zip(prompts, outs):
        with torch.no_grad():
            logits = hf(torch.tensor([p])).logits[0]
        assert torch.allclose(torch.tensor(o.outputs.data), torch.softmax(logits, -1), atol=2e-4), (o.outputs.data, logits)
    with torch.no_grad():
        assert torch.allclose(torch.tensor(raw[0].outputs.data), hf(torch.tensor([prompts[0]])).logits[0], atol=2e-3)


@pytest.mark.timeout(600)
def test_cross_encoder_score_matches_transformers(tmp_path):
    """A one-label sequence-classification checkpoint scores text pairs: ``LLM.score`` encodes ``text_1 <sep> text_2`` and returns
    sigmoid(score head), the value transformers gives for the same ids."""
    from onecat_vllm import LLM
    cfg = transformers.Qwen2Config(**{k: v for k, v in BASE.items()}, rope_theta=1e6, num_labels=1, pad_token_id=0, eos_token_id=257)
    cfg.architectures = ["Qwen2ForSequenceClassification"]
    torch.manual_seed(0)
    hf = transformers.Qwen2ForSequenceClassification(cfg).eval().float()
    for p in hf.parameters():
        if p.dim() >= 2:
            p.data.mul_(3.0)
    hf.save_pretrained(str(tmp_path), safe_serialization=True)
    llm = LLM(model=str(tmp_path), device="cpu", dtype="float32", max_model_len=128, tokenizer="byte")
    tok = llm.get_tokenizer()
    got = llm.score("what is a cat?", ["a small feline", "the stock market"])
    llm.shutdown()
    assert len(got) == 2 and got[0] != got[1]
    for g, doc in zip(got, ["a small feline", "the stock market"]):
        ids = list(tok.encode("what is a cat?")) + [257] + list(tok.encode(doc, add_special_tokens=False))
        with torch.no_grad():
            want = torch.sigmoid(hf(torch.tensor([ids])).logits[0, 0]).item()
        assert abs(g - want) < 2e-4, (g, want)
