"""End-to-end on a GPU: the engine with the sm_100a kernels against the fp32 CPU path on the same checkpoint."""
import json
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

CFG = dict(architectures=["Qwen3ForCausalLM"], hidden_size=512, intermediate_size=1024, num_hidden_layers=3, num_attention_heads=4,
           num_key_value_heads=2, head_dim=128, rms_norm_eps=1e-6, rope_theta=1e6, vocab_size=2048, max_position_embeddings=2048,
           tie_word_embeddings=False)


# Gemma2-style: sandwich norms, GeGLU, scaled embeddings, sliding window on alternate layers, score and logit soft-capping, D = 256
CFG_GEMMA2 = dict(architectures=["Gemma2ForCausalLM"], hidden_size=512, intermediate_size=1024, num_hidden_layers=4, num_attention_heads=4,
                  num_key_value_heads=2, head_dim=256, rms_norm_eps=1e-6, rope_theta=1e4, vocab_size=2048, max_position_embeddings=2048,
                  tie_word_embeddings=True, hidden_activation="gelu_pytorch_tanh", query_pre_attn_scalar=256, sliding_window=64,
                  layer_types=["sliding_attention", "full_attention", "sliding_attention", "full_attention"],
                  attn_logit_softcapping=50.0, final_logit_softcapping=30.0)


# OLMo-3-style: no pre-norms, normalised sub-block outputs, q / k norm over the whole projection, sliding layers
CFG_OLMO3 = dict(architectures=["Olmo3ForCausalLM"], hidden_size=512, intermediate_size=1024, num_hidden_layers=4, num_attention_heads=4,
                 num_key_value_heads=2, head_dim=128, rms_norm_eps=1e-6, rope_theta=1e4, vocab_size=2048, max_position_embeddings=2048,
                 tie_word_embeddings=False, sliding_window=64, layer_types=["sliding_attention", "sliding_attention", "sliding_attention", "full_attention"])
# SmolLM3-style: every fourth layer without rotary embedding; head size 64
CFG_SMOLLM3 = dict(architectures=["SmolLM3ForCausalLM"], hidden_size=512, intermediate_size=1024, num_hidden_layers=4, num_attention_heads=8,
                   num_key_value_heads=2, head_dim=64, rms_norm_eps=1e-6, rope_theta=1e4, vocab_size=2048, max_position_embeddings=2048,
                   tie_word_embeddings=True, no_rope_layers=[1, 1, 1, 0])


# HunYuan-style: per-head q / k norm applied after the rotation (two passes of the rope + insert kernel)
CFG_HUNYUAN = dict(architectures=["HunYuanDenseV1ForCausalLM"], hidden_size=512, intermediate_size=1024, num_hidden_layers=3, num_attention_heads=4,
                   num_key_value_heads=2, head_dim=128, rms_norm_eps=1e-6, rope_theta=1e4, vocab_size=2048, max_position_embeddings=2048,
                   tie_word_embeddings=False, use_qk_norm=True)


# GPT-OSS-style: attention sinks, alternating sliding layers, yarn, biases everywhere, experts with the clamped gated activation (served by
# one pair of dense GEMMs per expert), head size 64
CFG_GPTOSS = dict(architectures=["GptOssForCausalLM"], hidden_size=512, intermediate_size=512, num_hidden_layers=4, num_attention_heads=8,
                  num_key_value_heads=2, head_dim=64, rms_norm_eps=1e-5, vocab_size=2048, max_position_embeddings=2048, tie_word_embeddings=False,
                  num_local_experts=32, num_experts_per_tok=4, sliding_window=64,
                  layer_types=["sliding_attention", "full_attention", "sliding_attention", "full_attention"],
                  rope_parameters={"rope_type": "yarn", "rope_theta": 150000.0, "factor": 4.0, "beta_fast": 32.0, "beta_slow": 1.0, "truncate": False,
                                   "original_max_position_embeddings": 512})


def _make_checkpoint(tmp_path, cfg=CFG):
    from onecat_vllm.config import ModelConfig
    from onecat_vllm.loader.weights import dummy_init, save_pretrained
    from onecat_vllm.models import build_model
    mc = ModelConfig.from_hf_dict(cfg, dtype=torch.bfloat16)
    m = build_model(mc, "cpu")
    dummy_init(m, 0, std=0.05)
    save_pretrained(m, cfg, str(tmp_path))
    return str(tmp_path)


@pytest.mark.parametrize("eager,cfg,kvd", [(True, CFG, "auto"), (False, CFG, "auto"), (False, CFG_GEMMA2, "auto"), (False, CFG, "fp8"),
                                           (False, CFG_OLMO3, "auto"), (False, CFG_SMOLLM3, "auto"), (False, CFG_HUNYUAN, "auto"), (True, CFG_GPTOSS, "auto")],
                         ids=["eager", "graphs", "gemma2-graphs", "fp8kv-graphs", "olmo3-graphs", "smollm3-d64-graphs", "hunyuan-graphs", "gptoss-eager"])
def test_engine_gpu_matches_cpu(tmp_path, eager, cfg, kvd):
    from onecat_vllm import LLM, SamplingParams
    path = _make_checkpoint(tmp_path, cfg)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 2048, (int(n),), generator=g).tolist() for n in (5, 40, 130, 17, 64, 300)]
    sp = SamplingParams(temperature=0.0, max_tokens=24, ignore_eos=True, logprobs=0)
    gpu = LLM(model=path, device="cuda", dtype="bfloat16", max_model_len=1024, max_num_batched_tokens=256, max_num_seqs=8,
              gpu_memory_utilization=0.3, enforce_eager=eager, kv_cache_dtype=kvd)
    og = gpu.generate(prompts, sp)
    runner = gpu.llm_engine.engine_core.core.executor.worker.runner
    if not eager:
        assert runner.graphs is not None and runner.graphs.hits + runner.graphs.misses > 0, "decode must replay CUDA graphs"
    from onecat_vllm.ops import cuda as K
    assert K.check_status() == 0
    allowed = {"moe_expert_loop"} if cfg is CFG_GPTOSS else set()   # GPT-OSS experts: dense GEMMs per expert, activation in PyTorch
    assert K.TORCH_STANDINS <= allowed, f"ops fell back to device-side PyTorch: {K.TORCH_STANDINS}"
    K.TORCH_STANDINS.clear()
    gpu.shutdown()
    cpu = LLM(model=path, device="cpu", dtype="float32", max_model_len=1024, max_num_batched_tokens=256, max_num_seqs=8, kv_cache_dtype=kvd)
    if cfg is CFG_GPTOSS:
        # top-4 of 32 experts with random weights: a near-tie in the router forks the greedy path within a few tokens, so compare
        # teacher-forced instead: the fp32 model scores the GPU's own tokens, and those scores must match what the GPU reported
        diffs = []
        for p, o in zip(prompts, og):
            toks = o.outputs[0].token_ids
            assert len(toks) == 24
            r = cpu.generate([{"prompt_token_ids": p + toks}], SamplingParams(temperature=0.0, max_tokens=1, prompt_logprobs=0))[0]
            for i, t in enumerate(toks):
                diffs.append(abs(o.outputs[0].logprobs[i][t].logprob - r.prompt_logprobs[len(p) + i][t].logprob))
        cpu.shutdown()
        diffs.sort()
        # bf16 against fp32 through four routed layers: typical differences are ~0.1 nat, a flipped expert costs up to ~1.5
        assert diffs[len(diffs) // 2] < 0.2 and sum(diffs) / len(diffs) < 0.3 and diffs[-1] < 3.0, (diffs[len(diffs) // 2], sum(diffs) / len(diffs), diffs[-5:])
        return
    # teacher-forced agreement: feed the GPU's own tokens to the CPU model and require each GPU token to be near the top
    # random weights give nearly flat logits, so greedy paths may fork on near-ties: require (a) close log-probabilities of the
    # first generated token wherever both runs picked the same one, (b) a reasonable common prefix overall
    agree = total = first_same = 0
    for p, o in zip(prompts, og):
        toks = o.outputs[0].token_ids
        assert len(toks) == 24
        ref = cpu.generate([p], sp)[0].outputs[0]
        oc = ref.token_ids
        n = next((i for i, (a, b) in enumerate(zip(toks, oc)) if a != b), 24)
        agree += n
        total += 24
        if toks[0] == oc[0]:
            first_same += 1
            lg = o.outputs[0].logprobs[0][toks[0]].logprob
            lc = ref.logprobs[0][oc[0]].logprob
            assert abs(lg - lc) < 0.25, f"first-token logprob differs: gpu {lg} cpu {lc}"
    cpu.shutdown()
    assert first_same >= len(prompts) - 2, f"only {first_same}/{len(prompts)} prompts agree on the first generated token"
    assert agree / total > 0.35, f"GPU and CPU greedy decodes diverge too early: {agree}/{total} tokens before first difference"


def test_features_on_gpu_lora_offload_structured_embeds(tmp_path):
    """The engine features that only add host logic or small device ops run on the GPU path too: a LoRA adapter changes the first-token
    log-probability the same way as on the CPU path, the CPU tier of the prefix cache restores evicted blocks, a grammar constrains the
    output, prompt embeddings reproduce their token prompt."""
    import json as _json
    from safetensors.torch import save_file
    from onecat_vllm import LLM, SamplingParams
    from onecat_vllm.lora import LoRARequest
    from onecat_vllm.sampling_params import StructuredOutputsParams
    base = _make_checkpoint(tmp_path / "base")
    g = torch.Generator().manual_seed(5)
    ad = {}
    for l in range(CFG["num_hidden_layers"]):
        for name, (i, o) in {"self_attn.q_proj": (512, 512), "self_attn.o_proj": (512, 512), "mlp.gate_proj": (512, 1024), "mlp.down_proj": (1024, 512)}.items():
            ad[f"base_model.model.model.layers.{l}.{name}.lora_A.weight"] = torch.randn(8, i, generator=g) * 0.1
            ad[f"base_model.model.model.layers.{l}.{name}.lora_B.weight"] = torch.randn(o, 8, generator=g) * 0.1
    os.makedirs(tmp_path / "ad", exist_ok=True)
    save_file(ad, str(tmp_path / "ad" / "adapter_model.safetensors"))
    _json.dump({"r": 8, "lora_alpha": 16}, open(tmp_path / "ad" / "adapter_config.json", "w"))
    req = LoRARequest("ad", 1, str(tmp_path / "ad"))
    prompt = {"prompt_token_ids": torch.randint(0, 2048, (40,), generator=g).tolist()}
    sp = SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True, logprobs=0)
    res = {}
    for dev, dt in (("cpu", "float32"), ("cuda", "bfloat16")):
        llm = LLM(model=base, device=dev, dtype=dt, max_model_len=512, max_num_seqs=8, gpu_memory_utilization=0.3, enable_lora=True,
                  num_gpu_blocks_override=40, num_cpu_blocks_override=64, tokenizer="byte")
        plain = llm.generate([prompt], sp)[0].outputs[0]
        lora = llm.generate([prompt], sp, lora_request=req)[0].outputs[0]
        res[dev] = (plain.logprobs[0][plain.token_ids[0]].logprob, lora.logprobs[0][lora.token_ids[0]].logprob, plain.token_ids[0], lora.token_ids[0])
        if dev == "cuda":
            # CPU tier: push the prompt's blocks out of the 40-block pool with other traffic, then hit them again
            tier = llm.llm_engine.engine_core.core.scheduler.kv_cache_manager.offload
            for j in range(6):
                llm.generate([{"prompt_token_ids": torch.randint(0, 2048, (200,), generator=g).tolist()}], sp)
            again = llm.generate([prompt], sp)[0]
            assert tier.restored >= 2 and again.num_cached_tokens >= 32 and again.outputs[0].token_ids[0] == plain.token_ids[0]
            # grammar: the answer is one of the choices
            ch = llm.generate(["pick:"], SamplingParams(temperature=0.0, max_tokens=8, structured_outputs=StructuredOutputsParams(choice=["red", "blue"])))[0]
            assert ch.outputs[0].text in ("red", "blue")
            # prompt embeddings
            table = llm.llm_engine.engine_core.core.executor.worker.runner.model.model.embed_tokens.weight.detach()
            emb = llm.generate([{"prompt_embeds": table[torch.tensor(prompt["prompt_token_ids"], device=table.device)].cpu()}], sp)[0]
            assert emb.outputs[0].token_ids[0] == plain.token_ids[0]
            from onecat_vllm.ops import cuda as K
            assert K.check_status() == 0
        llm.shutdown()
    assert abs(res["cpu"][0] - res["cuda"][0]) < 0.15, res
    if res["cpu"][3] == res["cuda"][3]:
        assert abs(res["cpu"][1] - res["cuda"][1]) < 0.15, res
    assert abs(res["cuda"][0] - res["cuda"][1]) > 1e-3 or res["cuda"][2] != res["cuda"][3], "the adapter must change the GPU output"


# Qwen3.5-style hybrid: three Gated-DeltaNet layers to one gated full-attention layer (head size 256, partial rotary)
CFG_HYBRID = dict(architectures=["Qwen3_5ForCausalLM"], hidden_size=512, intermediate_size=1024, num_hidden_layers=4, num_attention_heads=4,
                  num_key_value_heads=2, head_dim=256, rms_norm_eps=1e-6, rope_theta=1e6, vocab_size=2048, max_position_embeddings=2048,
                  tie_word_embeddings=False, linear_num_key_heads=2, linear_num_value_heads=4, linear_key_head_dim=128, linear_value_head_dim=128,
                  linear_conv_kernel_dim=4, full_attention_interval=4, attn_output_gate=True, partial_rotary_factor=0.25)
# Qwen3-MoE-style: softmax top-4 of 32 experts through the routing kernel, the device-built work list and the grouped GEMM
CFG_QWEN_MOE = dict(architectures=["Qwen3MoeForCausalLM"], hidden_size=512, intermediate_size=1024, num_hidden_layers=3, num_attention_heads=4,
                    num_key_value_heads=2, head_dim=128, rms_norm_eps=1e-6, rope_theta=1e6, vocab_size=2048, max_position_embeddings=2048,
                    tie_word_embeddings=False, num_experts=32, num_experts_per_tok=4, moe_intermediate_size=256, norm_topk_prob=True)
# DeepSeek-V3-style: latent attention (512 + 64 wide cache), one dense layer, then grouped sigmoid routing with a shared expert
CFG_DSV3 = dict(architectures=["DeepseekV3ForCausalLM"], hidden_size=512, intermediate_size=1024, num_hidden_layers=3, num_attention_heads=4,
                num_key_value_heads=4, vocab_size=2048, rope_theta=10000.0, rms_norm_eps=1e-6, max_position_embeddings=2048, tie_word_embeddings=False,
                q_lora_rank=128, kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128, n_routed_experts=32, n_shared_experts=1,
                num_experts_per_tok=4, moe_intermediate_size=256, n_group=4, topk_group=2, routed_scaling_factor=1.5, norm_topk_prob=True,
                first_k_dense_replace=1, scoring_func="sigmoid")


@pytest.mark.parametrize("cfg", [CFG_HYBRID, CFG_QWEN_MOE, CFG_DSV3], ids=["hybrid-gdn", "qwen-moe", "deepseek-mla"])
def test_hybrid_moe_mla_engines_on_gpu_match_the_fp32_cpu_engine(tmp_path, cfg):
    """The engines whose mixers are not plain attention (Gated-DeltaNet state slots, routed experts, latent attention): decode must
    replay CUDA graphs, no op may fall back to device-side PyTorch, and the GPU's tokens, scored teacher-forced by the fp32 CPU engine,
    must carry the log-probabilities the GPU reported."""
    from onecat_vllm import LLM, SamplingParams
    from onecat_vllm.ops import cuda as K
    path = _make_checkpoint(tmp_path, cfg)
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, 2048, (int(n),), generator=g).tolist() for n in (7, 40, 130, 64, 290)]
    sp = SamplingParams(temperature=0.0, max_tokens=16, ignore_eos=True, logprobs=0)
    K.TORCH_STANDINS.clear()
    gpu = LLM(model=path, device="cuda", dtype="bfloat16", max_model_len=1024, max_num_batched_tokens=256, max_num_seqs=8, gpu_memory_utilization=0.3)
    og = gpu.generate(prompts, sp)
    runner = gpu.llm_engine.engine_core.core.executor.worker.runner
    assert runner.graphs is not None and runner.graphs.eligible and runner.graphs.hits + runner.graphs.misses > 0, "decode must replay CUDA graphs"
    assert K.check_status() == 0
    assert not K.TORCH_STANDINS, f"ops fell back to device-side PyTorch: {K.TORCH_STANDINS}"
    gpu.shutdown()
    cpu = LLM(model=path, device="cpu", dtype="float32", max_model_len=1024, max_num_batched_tokens=256, max_num_seqs=8)
    diffs = []
    for p, o in zip(prompts, og):
        toks = o.outputs[0].token_ids
        assert len(toks) == 16
        r = cpu.generate([{"prompt_token_ids": p + toks}], SamplingParams(temperature=0.0, max_tokens=1, prompt_logprobs=0))[0]
        for i, t in enumerate(toks):
            diffs.append(abs(o.outputs[0].logprobs[i][t].logprob - r.prompt_logprobs[len(p) + i][t].logprob))
    cpu.shutdown()
    diffs.sort()
    assert diffs[len(diffs) // 2] < 0.2 and sum(diffs) / len(diffs) < 0.3 and diffs[-1] < 3.0, (diffs[len(diffs) // 2], sum(diffs) / len(diffs), diffs[-5:])
