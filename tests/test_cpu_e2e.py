"""CPU plumbing slice: the tiny fp32 Llama/Qwen-style decoder served through the whole engine must reproduce a
plain HF Transformers greedy decode token for token (32 requests, prompts 16..128 tokens, 64 output tokens)."""
import torch
import pytest

from onecat_vllm import LLM, SamplingParams


def _hf_model_from(llm, cfg):
    from transformers import LlamaConfig, LlamaForCausalLM
    hc = LlamaConfig(hidden_size=cfg["hidden_size"], intermediate_size=cfg["intermediate_size"], num_hidden_layers=cfg["num_hidden_layers"],
                     num_attention_heads=cfg["num_attention_heads"], num_key_value_heads=cfg["num_key_value_heads"], head_dim=cfg["head_dim"],
                     rms_norm_eps=cfg["rms_norm_eps"], rope_theta=cfg["rope_theta"], vocab_size=cfg["vocab_size"],
                     max_position_embeddings=cfg["max_position_embeddings"], tie_word_embeddings=False, attention_bias=False)
    hf = LlamaForCausalLM(hc).float().eval()
    m = llm.llm_engine.engine_core.core.executor.worker.runner.model
    sd = {}
    H, D = cfg["num_attention_heads"], cfg["head_dim"]
    KV = cfg["num_key_value_heads"]
    for k, v in m.state_dict().items():
        if ".qkv_proj.weight" in k:
            q, kk, vv = v.split([H * D, KV * D, KV * D], dim=0)
            sd[k.replace("qkv_proj", "q_proj")] = q
            sd[k.replace("qkv_proj", "k_proj")] = kk
            sd[k.replace("qkv_proj", "v_proj")] = vv
        elif ".gate_up_proj.weight" in k:
            g, u = v.chunk(2, dim=0)
            sd[k.replace("gate_up_proj", "gate_proj")] = g
            sd[k.replace("gate_up_proj", "up_proj")] = u
        elif k.startswith("lm_head.weight") or "embed_tokens" in k:
            sd[k] = v[: cfg["vocab_size"]]
        else:
            sd[k] = v
    missing, unexpected = hf.load_state_dict(sd, strict=False)
    assert not [x for x in missing if "rotary" not in x], missing
    assert not unexpected, unexpected
    return hf


def _workload(n, seed=0, lo=16, hi=128, vocab=32000):
    g = torch.Generator().manual_seed(seed)
    lens = torch.randint(lo, hi + 1, (n,), generator=g)
    return [torch.randint(0, vocab, (int(l),), generator=g).tolist() for l in lens]


@pytest.mark.parametrize("budget,prefix", [(8192, True), (96, False)])
def test_tiny_llama_token_exact_vs_hf(tiny_llama_cfg, budget, prefix):
    cfg = tiny_llama_cfg
    llm = LLM(hf_config=cfg, max_model_len=512, dtype="float32", device="cpu", max_num_batched_tokens=budget, max_num_seqs=16,
              enable_prefix_caching=prefix, seed=0)
    prompts = _workload(32 if budget == 8192 else 6)
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=64, ignore_eos=True))
    assert len(outs) == len(prompts)
    hf = _hf_model_from(llm, cfg)
    with torch.no_grad():
        for p, o in zip(prompts, outs):
            ref = hf.generate(torch.tensor([p]), max_new_tokens=64, do_sample=False, pad_token_id=0, eos_token_id=None)[0, len(p):].tolist()
            assert o.outputs[0].token_ids == ref, f"prompt len {len(p)}"
            assert o.outputs[0].finish_reason == "length"
    llm.shutdown()


def test_prefix_cache_hit_gives_same_tokens(tiny_llama_cfg):
    llm = LLM(hf_config=tiny_llama_cfg, max_model_len=512, dtype="float32", device="cpu")
    p = _workload(1, seed=3, lo=100, hi=100)[0]
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    a = llm.generate([p], sp)[0]
    b = llm.generate([p + [5, 6, 7]], sp)[0]
    c = llm.generate([p], sp)[0]
    assert a.outputs[0].token_ids == c.outputs[0].token_ids
    assert c.num_cached_tokens == 96  # 6 full blocks of 16; the last token is always recomputed
    assert b.num_cached_tokens == 96
    llm.shutdown()


def test_seeded_sampling_is_reproducible(tiny_llama_cfg):
    llm = LLM(hf_config=tiny_llama_cfg, max_model_len=256, dtype="float32", device="cpu")
    p = _workload(2, seed=1)
    sp = SamplingParams(temperature=0.8, top_p=0.9, top_k=50, seed=7, max_tokens=12, ignore_eos=True)
    a = llm.generate(p, sp)
    b = llm.generate(p, sp)
    assert [o.outputs[0].token_ids for o in a] == [o.outputs[0].token_ids for o in b]
    sp2 = SamplingParams(temperature=0.8, seed=8, max_tokens=12, ignore_eos=True, n=2, logprobs=3)
    c = llm.generate(p[:1], sp2)[0]
    assert len(c.outputs) == 2 and c.outputs[0].token_ids != c.outputs[1].token_ids
    assert len(c.outputs[0].logprobs) == 12 and all(len(d) >= 3 for d in c.outputs[0].logprobs)
    llm.shutdown()


def test_embed_matches_direct_forward_and_survives_chunked_prefill():
    """LLM.embed (last / mean / cls pooling) equals pooling the model's own final hidden states, also when the prompt is
    prefilled in several chunks (reference test model: tests/models/language/pooling/)."""
    import torch
    from onecat_vllm import LLM
    from onecat_vllm.sampling_params import PoolingParams
    cfg = dict(architectures=["Qwen3ForCausalLM"], hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
               num_key_value_heads=2, head_dim=16, vocab_size=300, max_position_embeddings=512)
    prompt = list(range(5, 5 + 50))
    ref = {}
    for chunk in (8192, 16):
        llm = LLM(hf_config=cfg, device="cpu", dtype="float32", max_model_len=256, max_num_batched_tokens=chunk, enable_prefix_caching=False,
                  tokenizer="byte")
        for kind in ("last", "mean", "cls"):
            out = llm.encode([{"prompt_token_ids": prompt}], PoolingParams(task="encode", normalize=False, pooling_type=kind))[0]
            v = torch.tensor(out.outputs.data)
            assert v.shape == (64,)
            if chunk == 8192:
                ref[kind] = v
            else:
                assert torch.allclose(v, ref[kind], atol=1e-4), kind
        e = llm.embed([{"prompt_token_ids": prompt}])[0].outputs.embedding
        assert abs(sum(x * x for x in e) - 1) < 1e-4
        sc = llm.score("ab", ["ab", "xyz"])
        assert abs(sc[0] - 1) < 1e-4 and sc[1] < 0.9999
    assert not torch.allclose(ref["last"], ref["mean"])


def test_cpu_offload_tier_restores_evicted_prefix_blocks():
    """A GPU pool too small to keep a long shared prefix across other traffic: with the CPU tier the prefix comes back from the
    host (prefix-cache hit, restore copies) and the tokens equal those of a run that recomputes it."""
    from onecat_vllm import LLM, SamplingParams
    cfg = dict(architectures=["Qwen3ForCausalLM"], hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
               num_key_value_heads=2, head_dim=16, vocab_size=300, max_position_embeddings=512)
    prefix = [(3 * i) % 290 + 1 for i in range(160)]           # 10 blocks
    a = [{"prompt_token_ids": prefix + [7, 8, 9]}]
    filler = [{"prompt_token_ids": [(11 * i + j) % 290 + 1 for i in range(150)]} for j in range(3)]
    b = [{"prompt_token_ids": prefix + [20, 21]}]
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    kw = dict(hf_config=cfg, device="cpu", dtype="float32", max_model_len=256, num_gpu_blocks_override=24, max_num_seqs=1)
    plain = LLM(**kw)
    want = [plain.generate(x, sp)[0].outputs[0].token_ids for x in (a, *[[f] for f in filler], b)]
    plain.shutdown()
    llm = LLM(num_cpu_blocks_override=64, **kw)
    tier = llm.llm_engine.engine_core.core.scheduler.kv_cache_manager.offload
    assert tier is not None and tier.capacity == 64
    got = [llm.generate(x, sp)[0] for x in (a, *[[f] for f in filler], b)]
    assert [g.outputs[0].token_ids for g in got] == want
    assert tier.stored >= 10 and tier.restored >= 10, (tier.stored, tier.restored)
    assert got[-1].num_cached_tokens >= 160, "the shared prefix must count as a cache hit although the GPU pool had dropped it"
    llm.shutdown()


def test_arc_offload_policy_keeps_reused_blocks_through_a_scan():
    """Unit behaviour of the adaptive-replacement tier: blocks seen twice survive a scan of one-off blocks that would flush an LRU
    tier of the same size; and the engine produces the same tokens with it."""
    from onecat_vllm.core.kv_offload import ARCOffloadTier, CPUOffloadTier
    hot = [bytes([1, i]) for i in range(4)]
    scan = [bytes([2, i]) for i in range(40)]
    survivors = {}
    for cls in (CPUOffloadTier, ARCOffloadTier):
        t = cls(8)
        for h in hot:
            t.on_evict(h, 0)
        for h in hot:
            assert t.lookup(h) is not None      # second sighting: frequent
        for h in scan:
            t.on_evict(h, 0)
            t.take_ops()
        survivors[cls.__name__] = sum(t.lookup(h) is not None for h in hot)
        blocks = [c for c in t.index.values()]
        assert len(blocks) == len(set(blocks)) and len(blocks) + len(t.free) == 8   # no host block is lost or handed out twice
    assert survivors["CPUOffloadTier"] == 0 and survivors["ARCOffloadTier"] == 4, survivors
    from onecat_vllm import LLM, SamplingParams
    cfg = dict(architectures=["Qwen3ForCausalLM"], hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
               num_key_value_heads=2, head_dim=16, vocab_size=300, max_position_embeddings=512)
    prefix = [(3 * i) % 290 + 1 for i in range(160)]
    reqs = [[{"prompt_token_ids": prefix + [7, 8, 9]}]] + [[{"prompt_token_ids": [(11 * i + j) % 290 + 1 for i in range(150)]}] for j in range(3)] \
        + [[{"prompt_token_ids": prefix + [20, 21]}]]
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    kw = dict(hf_config=cfg, device="cpu", dtype="float32", max_model_len=256, num_gpu_blocks_override=24, max_num_seqs=1)
    plain = LLM(**kw)
    want = [plain.generate(x, sp)[0].outputs[0].token_ids for x in reqs]
    plain.shutdown()
    llm = LLM(num_cpu_blocks_override=64, kv_offloading_policy="arc", **kw)
    tier = llm.llm_engine.engine_core.core.scheduler.kv_cache_manager.offload
    assert isinstance(tier, ARCOffloadTier)
    got = [llm.generate(x, sp)[0] for x in reqs]
    assert [g.outputs[0].token_ids for g in got] == want
    assert tier.restored >= 10 and got[-1].num_cached_tokens >= 160
    llm.shutdown()


def test_shared_storage_connector_hands_prefill_kv_to_another_engine(tmp_path):
    """Disaggregated prefill / decode through the shared-storage KV connector: a producer engine runs the prompt once, a second
    (consumer) engine restores the blocks by hash and continues with the same tokens as an engine that computed everything itself."""
    from onecat_vllm import LLM, SamplingParams
    cfg = dict(architectures=["Qwen3ForCausalLM"], hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
               num_key_value_heads=2, head_dim=16, vocab_size=300, max_position_embeddings=512)
    prompt = [{"prompt_token_ids": [(5 * i) % 290 + 1 for i in range(100)]}]
    kw = dict(hf_config=cfg, device="cpu", dtype="float32", max_model_len=256)
    ktc = lambda role: {"kv_connector": "SharedStorageConnector", "kv_role": role, "kv_connector_extra_config": {"shared_storage_path": str(tmp_path)}}
    solo = LLM(**kw)
    want = solo.generate(prompt, SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))[0].outputs[0].token_ids
    solo.shutdown()
    prefill = LLM(kv_transfer_config=ktc("kv_producer"), **kw)
    first = prefill.generate(prompt, SamplingParams(temperature=0.0, max_tokens=1))[0].outputs[0].token_ids
    prefill.shutdown()
    import os
    assert len([f for f in os.listdir(tmp_path) if f.endswith(".kv")]) == 100 // 16
    decode = LLM(kv_transfer_config=ktc("kv_consumer"), **kw)
    out = decode.generate(prompt, SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))[0]
    tier = decode.llm_engine.engine_core.core.scheduler.kv_cache_manager.offload
    assert out.outputs[0].token_ids == want and first == want[:1]
    assert tier.restored == 100 // 16 and out.num_cached_tokens == 96 and tier.stored == 0
    decode.shutdown()


def test_beam_search_finds_a_sequence_at_least_as_likely_as_greedy():
    from onecat_vllm import LLM, SamplingParams
    from onecat_vllm.sampling_params import BeamSearchParams
    cfg = dict(architectures=["LlamaForCausalLM"], hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
               num_key_value_heads=2, head_dim=16, vocab_size=300, max_position_embeddings=256)
    llm = LLM(hf_config=cfg, device="cpu", dtype="float32", max_model_len=128)
    prompt = {"prompt_token_ids": [5, 9, 200, 33, 7]}
    greedy = llm.generate([prompt], SamplingParams(temperature=0.0, max_tokens=5, logprobs=0, ignore_eos=True))[0].outputs[0]
    res = llm.beam_search([prompt], BeamSearchParams(beam_width=3, max_tokens=5, ignore_eos=True))[0]["sequences"]
    assert len(res) == 3 and all(len(s["tokens"]) == 10 for s in res)
    assert res[0]["cum_logprob"] >= greedy.cumulative_logprob - 1e-4
    assert res[0]["cum_logprob"] >= res[1]["cum_logprob"] >= res[2]["cum_logprob"]
    one = llm.beam_search([prompt], BeamSearchParams(beam_width=1, max_tokens=5, ignore_eos=True))[0]["sequences"][0]
    assert one["tokens"][5:] == greedy.token_ids
    llm.shutdown()


def test_prompt_embeds_equal_token_prompts_and_can_be_chunked():
    """Feeding the embedding rows of a token prompt as ``prompt_embeds`` gives the same continuation as the token prompt, also when the
    prompt is prefilled in chunks and batched with ordinary requests."""
    import torch
    from onecat_vllm import LLM, SamplingParams
    cfg = dict(architectures=["Qwen3ForCausalLM"], hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
               num_key_value_heads=2, head_dim=16, vocab_size=300, max_position_embeddings=256)
    llm = LLM(hf_config=cfg, device="cpu", dtype="float32", max_model_len=128, max_num_batched_tokens=16)
    table = llm.llm_engine.engine_core.core.executor.worker.runner.model.model.embed_tokens.weight.detach().clone()
    ids = [(9 * i) % 290 + 1 for i in range(37)]
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    want = llm.generate([{"prompt_token_ids": ids}], sp)[0].outputs[0].token_ids
    outs = llm.generate([{"prompt_embeds": table[ids]}, {"prompt_token_ids": ids[:10]}], sp)
    assert outs[0].outputs[0].token_ids == want and len(outs[0].prompt_token_ids) == 37
    import pytest
    with pytest.raises(ValueError):
        llm.generate([{"prompt_embeds": torch.zeros(3, 5)}], sp)
    llm.shutdown()


@pytest.mark.parametrize("packed", [False, True])
def test_weights_handed_over_through_ipc_handles(packed):
    """RLHF-style in-place update: a second model's weights reach the engine as shared-memory handles (one per tensor, or one flat
    buffer per dtype) and the engine then decodes exactly like an engine built from that second model."""
    import torch
    from onecat_vllm import LLM, SamplingParams
    from onecat_vllm.config import ModelConfig
    from onecat_vllm.loader.weights import dummy_init, to_hf_state_dict
    from onecat_vllm.models import build_model
    from onecat_vllm.utils.weight_transfer import pack_ipc
    cfg = dict(architectures=["Qwen3ForCausalLM"], hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
               num_key_value_heads=2, head_dim=16, vocab_size=300, max_position_embeddings=256)
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    prompt = [{"prompt_token_ids": list(range(3, 30))}]
    other = build_model(ModelConfig.from_hf_dict(cfg, dtype=torch.float32, seed=5), "cpu")
    dummy_init(other, 5)
    want_llm = LLM(hf_config=cfg, device="cpu", dtype="float32", max_model_len=128, seed=5)
    want = want_llm.generate(prompt, sp)[0].outputs[0].token_ids
    want_llm.shutdown()
    llm = LLM(hf_config=cfg, device="cpu", dtype="float32", max_model_len=128, seed=0, enable_prefix_caching=False)
    before = llm.generate(prompt, sp)[0].outputs[0].token_ids
    n = llm.collective_rpc("update_weights_ipc", args=(pack_ipc(to_hf_state_dict(other).items(), packed=packed),))
    assert n[0] > 10
    after = llm.generate(prompt, sp)[0].outputs[0].token_ids
    llm.shutdown()
    assert before != want and after == want


def test_sliding_window_block_release_does_not_change_the_tokens():
    """An all-sliding model (Mistral-style) releases the blocks below its window while it decodes; the tokens must be those of the same
    engine with the release switched off, and the pool must really hold fewer blocks."""
    cfg = dict(architectures=["MistralForCausalLM"], hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
               num_key_value_heads=2, head_dim=16, vocab_size=500, max_position_embeddings=2048, sliding_window=48, rms_norm_eps=1e-6, rope_theta=1e4)
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, 500, (n,), generator=g).tolist() for n in (420, 333)]
    sp = SamplingParams(temperature=0.0, max_tokens=40, ignore_eos=True)
    kw = dict(hf_config=cfg, device="cpu", dtype="float32", max_model_len=1024, max_num_batched_tokens=128, enable_prefix_caching=False, seed=0)
    a = LLM(**kw)
    mgr = a.llm_engine.engine_core.core.scheduler.kv_cache_manager
    assert mgr.sliding_window == 48
    low = [1.0]
    orig = mgr.allocate_slots

    def spy(*args, **kwargs):
        out = orig(*args, **kwargs)
        low[0] = min(low[0], mgr.usage) if mgr.req_to_blocks and all(len(b) > 20 for b in mgr.req_to_blocks.values()) else low[0]
        return out
    mgr.allocate_slots = spy
    ta = [o.outputs[0].token_ids for o in a.generate(prompts, sp)]
    a.shutdown()
    b = LLM(**kw)
    b.llm_engine.engine_core.core.scheduler.kv_cache_manager.sliding_window = 0
    tb = [o.outputs[0].token_ids for o in b.generate(prompts, sp)]
    b.shutdown()
    assert ta == tb


def test_p2p_connector_serves_prefill_kv_to_a_decode_engine():
    """Disaggregated prefill / decode over the peer-to-peer connector: the producer keeps the prompt's blocks in host memory and serves
    them over a socket while it lives; the consumer restores them by hash and decodes the same tokens as a stand-alone engine."""
    from onecat_vllm import LLM, SamplingParams
    from onecat_vllm.executor.multiproc import _free_port
    cfg = dict(architectures=["Qwen3ForCausalLM"], hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
               num_key_value_heads=2, head_dim=16, vocab_size=300, max_position_embeddings=512)
    prompt = [{"prompt_token_ids": [(7 * i) % 290 + 1 for i in range(100)]}]
    kw = dict(hf_config=cfg, device="cpu", dtype="float32", max_model_len=256)
    port = _free_port()
    ktc = lambda role: {"kv_connector": "P2pConnector", "kv_role": role, "kv_connector_extra_config": {"host": "127.0.0.1", "port": port}}
    solo = LLM(**kw)
    want = solo.generate(prompt, SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))[0].outputs[0].token_ids
    solo.shutdown()
    prefill = LLM(kv_transfer_config=ktc("kv_producer"), **kw)
    first = prefill.generate(prompt, SamplingParams(temperature=0.0, max_tokens=1))[0].outputs[0].token_ids
    decode = LLM(kv_transfer_config=ktc("kv_consumer"), **kw)
    out = decode.generate(prompt, SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))[0]
    tier = decode.llm_engine.engine_core.core.scheduler.kv_cache_manager.offload
    assert out.outputs[0].token_ids == want and first == want[:1]
    assert tier.restored == 100 // 16 and out.num_cached_tokens == 96 and tier.stored == 0
    # a prompt the producer never saw finds nothing and is computed locally
    other = decode.generate([{"prompt_token_ids": [3] * 40}], SamplingParams(temperature=0.0, max_tokens=2))[0]
    assert other.num_cached_tokens == 0
    prefill.shutdown()
    decode.shutdown()
