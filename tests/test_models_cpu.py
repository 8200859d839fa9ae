"""Model families on CPU (fp32, random weights): chunked prefill must equal whole-prompt prefill (KV / recurrent state hand-off),
speculative decoding must be lossless under greedy sampling, quantised checkpoints must match their dequantised twins."""
import pytest
import torch

from onecat_vllm import LLM, SamplingParams

HYBRID = dict(architectures=["Qwen3NextForCausalLM"], hidden_size=128, intermediate_size=256, num_hidden_layers=4, num_attention_heads=4,
              num_key_value_heads=2, head_dim=32, vocab_size=500, max_position_embeddings=512, linear_num_key_heads=2, linear_num_value_heads=4,
              linear_key_head_dim=32, linear_value_head_dim=32, full_attention_interval=4, partial_rotary_factor=0.25)
MOE = dict(architectures=["Qwen3MoeForCausalLM"], hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
           num_key_value_heads=2, head_dim=16, vocab_size=300, max_position_embeddings=256, num_experts=8, num_experts_per_tok=2,
           moe_intermediate_size=32, shared_expert_intermediate_size=64, norm_topk_prob=True)
DSV3 = dict(architectures=["DeepseekV3ForCausalLM"], hidden_size=64, intermediate_size=128, num_hidden_layers=3, num_attention_heads=4,
            vocab_size=300, max_position_embeddings=256, q_lora_rank=32, kv_lora_rank=16, qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=16,
            n_routed_experts=8, num_experts_per_tok=2, moe_intermediate_size=32, n_shared_experts=1, n_group=4, topk_group=2,
            first_k_dense_replace=1, routed_scaling_factor=2.5, scoring_func="sigmoid")


def _prompts(vocab, lens=(20, 45, 9), seed=0):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lens]


def _gen(cfg, prompts, **kw):
    llm = LLM(hf_config=cfg, max_model_len=256, dtype="float32", device="cpu", **kw)
    out = [o.outputs[0].token_ids for o in llm.generate(prompts, SamplingParams(temperature=0, max_tokens=16, ignore_eos=True))]
    llm.shutdown()
    return out


@pytest.mark.parametrize("cfg", [HYBRID, MOE, DSV3], ids=["hybrid-gdn", "moe", "mla-moe"])
def test_chunked_prefill_equals_whole(cfg):
    p = _prompts(cfg["vocab_size"])
    assert _gen(cfg, p, max_num_batched_tokens=16) == _gen(cfg, p)


@pytest.mark.parametrize("method", ["ngram", "mtp"])
def test_spec_decode_lossless_on_hybrid(method):
    p = _prompts(500)
    ref = _gen(HYBRID, p)
    assert _gen(HYBRID, p, speculative_config=dict(method=method, num_speculative_tokens=3)) == ref


def test_spec_decode_verifies_against_the_constrained_distribution():
    """With top_k = 1 a random-temperature request is deterministic (the arg-max), with and without drafts: the verifier must judge
    the drafts against the filtered distribution, not the raw one. Penalties, a logit bias and bad words must carry over too."""
    p = _prompts(500)[:3]

    def run(sp, **kw):
        llm = LLM(hf_config=HYBRID, max_model_len=256, dtype="float32", device="cpu", **kw)
        out = [o.outputs[0].token_ids for o in llm.generate(p, sp)]
        llm.shutdown()
        return out
    spec = dict(speculative_config=dict(method="ngram", num_speculative_tokens=3))
    greedy = run(SamplingParams(temperature=0, max_tokens=24, ignore_eos=True))
    topk1 = SamplingParams(temperature=1.0, top_k=1, max_tokens=24, ignore_eos=True, seed=3)
    assert run(topk1, **spec) == greedy
    banned = greedy[0][3]
    shaped = SamplingParams(temperature=0, max_tokens=24, ignore_eos=True, repetition_penalty=1.3, logit_bias={7: 4.0},
                            bad_words_token_ids=[[banned]])
    want = run(shaped)
    assert want != greedy and all(banned not in o for o in want)
    assert run(shaped, **spec) == want


def test_verifier_applies_filters_and_processors_to_draft_rows():
    """The verifier on crafted logits: a draft with 38 % of the raw probability mass must never be accepted under top_k = 1 (the raw
    distribution would accept it about every third time), and a banned arg-max must not be what greedy verification emits."""
    from onecat_vllm.sample.metadata import SamplingMetadata
    llm = LLM(hf_config=HYBRID, max_model_len=256, dtype="float32", device="cpu", speculative_config=dict(method="ngram", num_speculative_tokens=3))
    runner = llm.llm_engine.engine_core.core.executor.worker.runner
    V, A, D = HYBRID["vocab_size"], 5, 9
    row = torch.full((V,), -8.0)
    row[A], row[D] = 2.0, 1.5
    logits = row.repeat(6, 1)                      # request 0: three drafts + bonus; request 1: one draft + bonus
    rows, drafts = [4, 2], [[D, D, D], [D]]

    def md(**kw):
        base = dict(temperature=torch.ones(2), all_greedy=False, all_random=True, top_p=None, top_k=None, min_p=None, generators={},
                    max_num_logprobs=None, no_penalties=True, output_token_ids=[[1, 2], [3]], logit_bias=[None, None],
                    allowed_token_ids=[None, None])
        base.update(kw)
        return SamplingMetadata(**base)
    accepted_raw = 0
    for _ in range(40):
        out = runner._verify(logits.clone(), md(), rows, drafts)
        accepted_raw += sum(1 for o in out if o[0] == D)
        out = runner._verify(logits.clone(), md(top_k=torch.tensor([1, 1])), rows, drafts)
        assert out == [[A], [A]]                   # first draft rejected, the recovered token is the only one left in the filter
    assert accepted_raw > 0                        # the crafted draft is plausible without the filter
    # a batch in which every request verified a full set of drafts takes the copy-free path: same rules, caller's logits untouched
    full = row.repeat(8, 1)
    keep = full.clone()
    assert runner._verify(full, md(top_k=torch.tensor([1, 1])), [4, 4], [[D, D, D], [D, D, D]]) == [[A], [A]]
    assert torch.equal(full, keep)
    assert runner._verify(full, md(temperature=None, all_greedy=True, all_random=False), [4, 4], [[A, A, A], [A, D, A]]) == [[A, A, A, A], [A, A]]
    greedy = dict(temperature=None, all_greedy=True, all_random=False)
    assert runner._verify(logits.clone(), md(**greedy), rows, [[A, A, A], [A]]) == [[A, A, A, A], [A, A]]
    out = runner._verify(logits.clone(), md(bad_words_token_ids={0: [[A]]}, **greedy), rows, [[A, A, A], [A]])
    assert out == [[D], [A, A]]                    # request 0 may not emit A anywhere: its first draft fails and D is recovered
    llm.shutdown()


def test_synthetic_acceptance_exercises_verifier():
    llm = LLM(hf_config=HYBRID, max_model_len=256, dtype="float32", device="cpu",
              speculative_config=dict(method="mtp", num_speculative_tokens=3, synthetic_acceptance_rate=0.7, synthetic_seed=1))
    outs = llm.generate(_prompts(500), SamplingParams(temperature=0, max_tokens=40, ignore_eos=True))
    assert all(len(o.outputs[0].token_ids) == 40 for o in outs)
    llm.shutdown()


def test_awq_checkpoint_matches_dequantised_weights(tmp_path):
    """An AWQ model and a dense model holding the dequantised weights must decode identically on the CPU path."""
    from onecat_vllm.config import ModelConfig
    from onecat_vllm.loader.weights import dummy_init, save_pretrained, to_hf_state_dict
    from onecat_vllm.models import build_model
    base = dict(architectures=["LlamaForCausalLM"], hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                num_key_value_heads=2, head_dim=32, vocab_size=300, max_position_embeddings=256)
    qcfg = dict(base, quantization_config=dict(quant_method="awq", bits=4, group_size=128, zero_point=True))
    m = build_model(ModelConfig.from_hf_dict(qcfg, dtype=torch.float32), "cpu")
    dummy_init(m, 0)
    save_pretrained(m, qcfg, str(tmp_path / "awq"))
    sd = {}
    for name, mod in m.named_modules():
        if hasattr(mod, "method") and mod.method.name == "awq":
            w = mod.method.dequantized_weight(mod).float()
            off = 0
            stacked = [(t, s) for o, t, s in m.stacked_params_mapping if name.endswith(o)]
            if stacked:
                ours = [o for o, t, s in m.stacked_params_mapping if name.endswith(o)][0]
                for theirs, sid in stacked:
                    n = mod.local_output_sizes[sid]
                    sd[name[: -len(ours)] + theirs + ".weight"] = w[off:off + n].contiguous()
                    off += n
            else:
                sd[name + ".weight"] = w.contiguous()
    for k, v in to_hf_state_dict(m).items():
        if not k.endswith((".qweight", ".qzeros", ".scales")):
            sd[k] = v
    from safetensors.torch import save_file
    import json, os
    os.makedirs(tmp_path / "dense")
    save_file({k: v.contiguous() for k, v in sd.items()}, str(tmp_path / "dense" / "model.safetensors"))
    json.dump(base, open(tmp_path / "dense" / "config.json", "w"))
    p = _prompts(300, (12, 30))
    sp = SamplingParams(temperature=0, max_tokens=10, ignore_eos=True)
    a = LLM(model=str(tmp_path / "awq"), device="cpu", dtype="float32", max_model_len=128)
    b = LLM(model=str(tmp_path / "dense"), device="cpu", dtype="float32", max_model_len=128)
    assert [o.outputs[0].token_ids for o in a.generate(p, sp)] == [o.outputs[0].token_ids for o in b.generate(p, sp)]
    a.shutdown(); b.shutdown()


def test_weight_packers_keep_every_value_addressable():
    """The tile layouts of the FP8 and MXFP4 packers: byte / nibble (n, k) of the source lands where the kernel reads it, and
    the scale words carry the bf16 bits of scale * 2**120 (fp8) and 2**(e - 1) (fp4)."""
    import torch
    from onecat_vllm.ops.cuda import _NIB_ORDER, pack_fp8, pack_mxfp4
    N, K = 256, 192
    g = torch.Generator().manual_seed(0)
    w8 = torch.randint(0, 256, (N, K), generator=g, dtype=torch.uint8)
    rs = torch.rand(N, K // 64, generator=g) * 1e-3 + 1e-5
    tiles, sz, npad = pack_fp8(w8, rs, 64)
    assert tiles.shape == (2, 3, 8192) and sz.shape == (3, 256) and npad == 256
    for n, k in [(0, 0), (5, 17), (130, 63), (255, 191), (129, 64)]:
        nt, r, kt, kk = n // 128, n % 128, k // 64, k % 64
        assert int(tiles[nt, kt, (kk // 16) * 2048 + r * 16 + kk % 16]) == int(w8[n, k])
        want = (rs[n, kt] * 2.0 ** 120).to(torch.bfloat16).view(torch.int16).int() & 0xFFFF
        assert int(sz[kt, n]) == int(want)
    packed = torch.randint(0, 256, (N, K // 2), generator=g, dtype=torch.uint8)
    e = torch.randint(100, 128, (N, K // 32), generator=g, dtype=torch.uint8)
    t4, sz4, _ = pack_mxfp4(packed, e)
    assert t4.shape == (2, 3, 4096) and sz4.shape == (3, 256)
    words = t4.view(2, 3, 2, 128, 4, 4)  # [nt][kt][half][row][word][byte]
    for n, k in [(0, 0), (3, 9), (200, 100), (255, 191)]:
        nt, r, kt, kk = n // 128, n % 128, k // 64, k % 64
        c, j = kk // 8, kk % 8
        b = words[nt, kt, c // 4, r, c % 4]
        word = int(b[0]) | int(b[1]) << 8 | int(b[2]) << 16 | int(b[3]) << 24
        nib = (word >> (4 * _NIB_ORDER.index(j))) & 0xF
        src = int(packed[n, k // 2])
        assert nib == ((src >> 4) if k % 2 else (src & 0xF))
        half = (int(sz4[kt, n]) >> (16 * (kk // 32))) & 0xFFFF
        want = torch.tensor(2.0 ** (int(e[n, k // 32]) - 1)).to(torch.bfloat16).view(torch.int16).int() & 0xFFFF
        assert half == int(want)


def test_nvfp4_packer_round_trips_through_the_kernel_layout():
    """Rebuild the weights from the NVFP4 tiles and scale words exactly as the kernel reads them (word c of a row's 8 words holds
    k = 8c..8c+7; group g = c // 2 takes the g-th bf16 of the row's two scale words) and compare with the reference dequantisation."""
    import torch
    from onecat_vllm.ops import ref
    from onecat_vllm.ops.cuda import _NIB_ORDER, pack_nvfp4
    N, K = 128, 128
    g = torch.Generator().manual_seed(3)
    packed = torch.randint(0, 256, (N, K // 2), generator=g, dtype=torch.uint8)
    sc = (torch.rand(N, K // 16, generator=g) * 3 + 0.25).to(torch.float8_e4m3fn)
    gs = torch.tensor([0.02])
    tiles, sz, npad = pack_nvfp4(packed, sc, gs)
    assert tiles.shape == (1, 2, 4096) and sz.shape == (2, 128, 2)
    want = ref.nvfp4_dequantize(packed, sc, gs)
    lut = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])
    words = tiles.view(1, 2, 2, 128, 4, 4).to(torch.int64)  # [nt][kt][half][row][word][byte]
    got = torch.zeros(N, K)
    for kt in range(2):
        for r in range(N):
            for c in range(8):
                b = words[0, kt, c // 4, r, c % 4]
                word = int(b[0]) | int(b[1]) << 8 | int(b[2]) << 16 | int(b[3]) << 24
                szw = int(sz[kt, r, c // 4]) & 0xFFFFFFFF
                half = (szw >> 16) & 0xFFFF if (c & 2) else szw & 0xFFFF
                s = torch.tensor([half << 16], dtype=torch.int32).view(torch.float32).item() / 2.0 ** 126
                for j in range(8):
                    nib = (word >> (4 * _NIB_ORDER.index(j))) & 0xF
                    v = lut[nib & 7].item() * (-1.0 if nib & 8 else 1.0)
                    got[r, kt * 64 + c * 8 + j] = v * s
    assert torch.allclose(got, want, rtol=2 ** -7, atol=1e-6)


@pytest.mark.parametrize("layout", ["qwen", "deepseek"])
def test_mtp_head_weights_load_from_checkpoint(tmp_path, layout):
    """The draft head's tensors come from the target's checkpoint: ``mtp.*`` (Qwen3-Next / Qwen3.5) or decoder layer
    ``num_hidden_layers`` with enorm / hnorm / eh_proj / shared_head.norm (DeepSeek-V3)."""
    import dataclasses
    from safetensors.torch import save_file
    from onecat_vllm.config import ModelConfig
    from onecat_vllm.loader.weights import dummy_init, save_pretrained, to_hf_state_dict
    from onecat_vllm.models import build_model
    from onecat_vllm.models.decoder import MTPHead
    cfg = HYBRID if layout == "qwen" else DSV3
    mc = ModelConfig.from_hf_dict(cfg, dtype=torch.float32)
    m = build_model(mc, "cpu")
    dummy_init(m, 0)
    save_pretrained(m, cfg, str(tmp_path))
    head = MTPHead(mc, m, "cpu")
    dummy_init(head, 77)
    sd = {}
    L = mc.num_hidden_layers
    ds = {"pre_fc_norm_embedding.": "enorm.", "pre_fc_norm_hidden.": "hnorm.", "fc.": "eh_proj.", "norm.": "shared_head.norm."}
    for name, w in to_hf_state_dict(head).items():
        if layout == "qwen":
            name = "mtp." + (("layers.0." + name[len("layer."):]) if name.startswith("layer.") else name)
        else:
            for ours, theirs in ds.items():
                if name.startswith(ours):
                    name = theirs + name[len(ours):]
                    break
            else:
                name = name[len("layer."):]
            name = f"model.layers.{L}." + name
        sd[name] = w.contiguous()
    save_file(sd, str(tmp_path / "model-mtp.safetensors"))
    llm = LLM(model=str(tmp_path), max_model_len=128, dtype="float32", device="cpu", speculative_config=dict(method="mtp", num_speculative_tokens=2))
    got = llm.llm_engine.engine_core.core.executor.worker.runner.mtp
    want = dict(head.named_parameters())
    n = 0
    for name, p in got.named_parameters():
        assert torch.equal(p, want[name]), name
        n += 1
    assert n >= 8
    out = llm.generate(_prompts(cfg["vocab_size"])[:2], SamplingParams(temperature=0, max_tokens=8, ignore_eos=True))
    assert all(len(o.outputs[0].token_ids) == 8 for o in out)
    llm.shutdown()


def test_eagle_head_is_lossless_and_loads_its_checkpoint(tmp_path):
    """EAGLE-1 drafting: greedy output equals plain decoding whatever the head proposes, and the head's tensors come from its own
    checkpoint directory (``fc`` with bias, ``embed_tokens``, ``layers.0`` without an input norm)."""
    from safetensors.torch import save_file
    from onecat_vllm.config import ModelConfig
    from onecat_vllm.loader.weights import dummy_init, to_hf_state_dict
    from onecat_vllm.models import build_model
    from onecat_vllm.models.decoder import EagleHead
    dense = dict(architectures=["LlamaForCausalLM"], hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                 num_key_value_heads=2, head_dim=16, vocab_size=500, max_position_embeddings=256)
    mc = ModelConfig.from_hf_dict(dense, dtype=torch.float32)
    head = EagleHead(mc, build_model(mc, "cpu"), "cpu")
    dummy_init(head, 5)
    sd = {}
    for name, w in to_hf_state_dict(head).items():
        if "input_layernorm" in name:
            continue
        sd[("layers.0." + name[len("layer."):]) if name.startswith("layer.") else name] = w.contiguous()
    save_file(sd, str(tmp_path / "model.safetensors"))
    p = _prompts(500)
    ref = _gen(dense, p)
    llm = LLM(hf_config=dense, max_model_len=256, dtype="float32", device="cpu",
              speculative_config=dict(method="eagle", num_speculative_tokens=3, model=str(tmp_path)))
    got = llm.llm_engine.engine_core.core.executor.worker.runner.mtp
    assert got.own_embedding
    want = dict(head.named_parameters())
    for name, q in got.named_parameters():
        if "input_layernorm" not in name:
            assert torch.equal(q[:500], want[name][:500]), name   # embedding rows past the vocabulary are padding
    out = [o.outputs[0].token_ids for o in llm.generate(p, SamplingParams(temperature=0, max_tokens=16, ignore_eos=True))]
    llm.shutdown()
    assert out == ref


def test_eagle3_head_is_lossless_loads_its_checkpoint_and_matches_plain_torch(tmp_path):
    """EAGLE-3 drafting: the target records its residual stream at three depths, the head (own final norm, LM head over a reduced
    vocabulary with ``d2t`` offsets) loads ``fc`` / ``midlayer.*`` / ``norm`` / ``lm_head`` / ``d2t``, greedy output equals plain
    decoding, and the head's first pass equals a plain-PyTorch restatement of the layer."""
    import json
    from safetensors.torch import save_file
    from onecat_vllm.config import ModelConfig
    from onecat_vllm.loader.weights import dummy_init, to_hf_state_dict
    from onecat_vllm.models import build_model
    from onecat_vllm.models.decoder import Eagle3Head
    from onecat_vllm.ops import ref
    from onecat_vllm.worker.attn_metadata import AttentionMetadata
    H, V, DV = 64, 500, 120
    dense = dict(architectures=["LlamaForCausalLM"], hidden_size=H, intermediate_size=128, num_hidden_layers=8, num_attention_heads=4,
                 num_key_value_heads=2, head_dim=16, vocab_size=V, max_position_embeddings=256, rms_norm_eps=1e-6, rope_theta=10000.0)
    mc = ModelConfig.from_hf_dict(dense, dtype=torch.float32)
    mc.max_model_len = 256
    head = Eagle3Head(mc, build_model(mc, "cpu"), "cpu", DV)
    dummy_init(head, 5, std=0.2)
    sd = {}
    for name, w in to_hf_state_dict(head).items():
        if name.startswith("embed_tokens."):
            continue                                   # this checkpoint shares the target's embedding
        name = "midlayer." + name[len("layer."):] if name.startswith("layer.") else ("midlayer." + name if name.startswith("hidden_norm.") else name)
        sd[name] = w.contiguous()
    targets = torch.sort(torch.randperm(V, generator=torch.Generator().manual_seed(2))[:DV]).values
    sd["d2t"] = targets - torch.arange(DV)
    sd["t2d"] = torch.zeros(V, dtype=torch.bool)
    save_file(sd, str(tmp_path / "model.safetensors"))
    (tmp_path / "config.json").write_text(json.dumps({"draft_vocab_size": DV}))

    p = _prompts(V)
    want = _gen(dense, p)
    llm = LLM(hf_config=dense, max_model_len=256, dtype="float32", device="cpu",
              speculative_config=dict(method="eagle3", num_speculative_tokens=3, model=str(tmp_path)))
    runner = llm.llm_engine.engine_core.core.executor.worker.runner
    got = runner.mtp
    assert got.own_lm_head and not got.own_embedding and got.draft_vocab == DV and torch.equal(got.d2t, sd["d2t"])
    assert runner.model.model.aux_hidden_layers == (2, 4, 5)
    src = dict(head.named_parameters())
    for name, q in got.named_parameters():
        if not name.startswith("embed_tokens."):
            assert torch.equal(q, src[name]), name
    out = [o.outputs[0].token_ids for o in llm.generate(p, SamplingParams(temperature=0, max_tokens=16, ignore_eos=True))]
    assert out == want
    assert len(runner.model.model.last_aux) == 3 and all(a.shape[-1] == H for a in runner.model.model.last_aux)

    # ---- the head's first pass on one 7-token sequence against plain PyTorch
    T = 7
    g = torch.Generator().manual_seed(9)
    ids = torch.randint(0, V, (T,), generator=g, dtype=torch.int32)
    aux = torch.randn(T, 3 * H, generator=g)
    cache = torch.zeros(4, 2, 2, 16, 16)
    md = AttentionMetadata(1, T, torch.tensor([0, T], dtype=torch.int32), torch.tensor([T], dtype=torch.int32), torch.tensor([[1]], dtype=torch.int32),
                           torch.arange(16, 16 + T, dtype=torch.int32), torch.arange(T, dtype=torch.int32), T, T, query_lens_cpu=[T], seq_lens_cpu=[T])
    with torch.no_grad():
        h_out = got(ids, aux, md, cache)
        logits = got.compute_logits(h_out)

        def rms(x, w):
            return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * w
        L = got.layer
        hidden = aux @ got.fc.weight.t()
        emb = runner.model.model.embed_tokens.weight[ids.long()]
        x = torch.cat([rms(emb, L.input_layernorm.weight), rms(hidden, got.hidden_norm.weight)], -1)
        qkv = x @ L.self_attn.qkv_proj.weight.t()
        q, k, v = qkv[:, :64].view(T, 4, 16), qkv[:, 64:96].view(T, 2, 16), qkv[:, 96:].view(T, 2, 16)
        cs = ref.build_cos_sin_cache(16, 256, 10000.0, "cpu")[:T]
        rot = lambda t: torch.cat([t[..., :8] * cs[:, None, :8] - t[..., 8:] * cs[:, None, 8:], t[..., 8:] * cs[:, None, :8] + t[..., :8] * cs[:, None, 8:]], -1)
        q, k = rot(q), rot(k)
        k, v = k.repeat_interleave(2, 1), v.repeat_interleave(2, 1)
        att = torch.einsum("thd,shd->hts", q, k) * 16 ** -0.5
        att = att.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf")).softmax(-1)
        o = torch.einsum("hts,shd->thd", att, v).reshape(T, 64) @ L.self_attn.o_proj.weight.t()
        r = hidden + o
        x2 = rms(r, L.post_attention_layernorm.weight)
        gu = x2 @ L.mlp.gate_up_proj.weight.t()
        want_h = r + (torch.nn.functional.silu(gu[:, :128]) * gu[:, 128:]) @ L.mlp.down_proj.weight.t()
        want_lg = rms(want_h, got.norm.weight) @ got.lm_head.weight.t()
    assert torch.allclose(h_out, want_h, atol=2e-4, rtol=2e-4), float((h_out - want_h).abs().max())
    assert logits.shape == (T, V) and torch.isinf(logits[:, [i for i in range(V) if i not in set(targets.tolist())]]).all()
    assert torch.allclose(logits[:, targets], want_lg, atol=2e-3, rtol=2e-3)
    llm.shutdown()


def test_draft_model_proposer_is_lossless_and_a_twin_draft_is_always_accepted(tmp_path):
    """A separate draft model under the target's block ids. With the target's own weights as the draft every proposed token is
    accepted (which pins the position and slot bookkeeping of the drafting passes); with another model the output is still the
    target's greedy decode."""
    from onecat_vllm.config import ModelConfig
    from onecat_vllm.loader.weights import dummy_init, save_pretrained
    from onecat_vllm.models import build_model
    big = dict(architectures=["LlamaForCausalLM"], hidden_size=64, intermediate_size=128, num_hidden_layers=3, num_attention_heads=4,
               num_key_value_heads=2, head_dim=16, vocab_size=500, max_position_embeddings=256)
    small = dict(big, hidden_size=32, intermediate_size=64, num_hidden_layers=1, num_attention_heads=2, num_key_value_heads=1)
    for name, cfg, seed in (("big", big, 0), ("small", small, 7)):
        m = build_model(ModelConfig.from_hf_dict(cfg, dtype=torch.float32), "cpu")
        dummy_init(m, seed, std=0.1)
        save_pretrained(m, cfg, str(tmp_path / name))
    p = _prompts(500)
    sp = SamplingParams(temperature=0, max_tokens=20, ignore_eos=True)

    def run(**kw):
        llm = LLM(model=str(tmp_path / "big"), max_model_len=256, dtype="float32", device="cpu", max_num_batched_tokens=64, disable_log_stats=False, **kw)
        out = [o.outputs[0].token_ids for o in llm.generate(p, sp)]
        mt = llm.llm_engine.get_metrics()
        acc = (mt.get("vllm:spec_decode_num_accepted_tokens_total"), mt.get("vllm:spec_decode_num_draft_tokens_total"))
        llm.shutdown()
        return out, acc
    want, _ = run()
    twin, acc = run(speculative_config=dict(method="draft_model", num_speculative_tokens=3, model=str(tmp_path / "big")))
    assert twin == want
    assert acc[1] and acc[0] == acc[1], acc     # every draft of the twin was accepted
    other, _ = run(speculative_config=dict(method="draft_model", num_speculative_tokens=3, model=str(tmp_path / "small")))
    assert other == want


def test_medusa_heads_are_lossless_and_load(tmp_path):
    from safetensors.torch import save_file
    from onecat_vllm.spec_decode.proposers import MedusaHeads
    dense = dict(architectures=["LlamaForCausalLM"], hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                 num_key_value_heads=2, head_dim=16, vocab_size=500, max_position_embeddings=256)
    src = MedusaHeads(64, 500, 3, 1, torch.float32)
    sd = {}
    for name, w in src.state_dict().items():   # the serving layout: blocks.{i}.layers.{j}.*, lm_heads.{i}.weight
        parts = name.split(".")
        sd[f"blocks.{parts[1]}.layers.{parts[2]}.{parts[3]}" if parts[0] == "blocks" else name] = w.contiguous()
    save_file(sd, str(tmp_path / "model.safetensors"))
    p = _prompts(500)
    ref = _gen(dense, p)
    llm = LLM(hf_config=dense, max_model_len=256, dtype="float32", device="cpu",
              speculative_config=dict(method="medusa", num_speculative_tokens=3, model=str(tmp_path)))
    heads = llm.llm_engine.engine_core.core.executor.worker.runner.proposer.heads
    for name, w in src.state_dict().items():
        assert torch.equal(heads.state_dict()[name], w), name
    out = [o.outputs[0].token_ids for o in llm.generate(p, SamplingParams(temperature=0, max_tokens=16, ignore_eos=True))]
    llm.shutdown()
    assert out == ref


def test_native_ngram_lookup_matches_python_and_suffix_cache_drafts_across_requests():
    import numpy as np
    from onecat_vllm.spec_decode.proposers import NgramProposer
    p = NgramProposer(3, 2, 4)
    assert p._native is not None, "the native module must be built"
    rng = np.random.default_rng(0)
    for _ in range(200):
        toks = rng.integers(0, 6, size=int(rng.integers(1, 60))).tolist()
        assert list(p.propose_one(toks)) == p.propose_one_py(toks), toks
    # suffix cache: the second run of the same prompt drafts the first run's answer and accepts it
    dense = dict(architectures=["LlamaForCausalLM"], hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                 num_key_value_heads=2, head_dim=16, vocab_size=500, max_position_embeddings=256)
    prompts = _prompts(500)[:2]
    ref = _gen(dense, prompts)
    llm = LLM(hf_config=dense, max_model_len=256, dtype="float32", device="cpu", enable_prefix_caching=False,
              speculative_config=dict(method="suffix", num_speculative_tokens=3))
    sp = SamplingParams(temperature=0, max_tokens=16, ignore_eos=True)
    first = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
    second = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
    prop = llm.llm_engine.engine_core.core.executor.worker.runner.proposer
    assert prop.index.num_sequences >= 2
    seq = list(prompts[0]["prompt_token_ids"] if isinstance(prompts[0], dict) else prompts[0]) + first[0]
    cut = len(seq) - 10
    assert list(prop.index.propose(np.asarray(seq[cut - 4:cut], dtype=np.int32), 3)) == seq[cut:cut + 3]
    llm.shutdown()
    assert first == ref and second == ref


@pytest.mark.parametrize("scheme", ["int4-group", "fp8-channel", "fp8-tensor"])
def test_compressed_tensors_checkpoints_match_their_dequantised_weights(tmp_path, scheme):
    """llm-compressor layouts: pack-quantized symmetric int4 (``weight_packed`` / ``weight_scale``) and float-quantized FP8 with one
    scale per tensor or per output channel. A dense checkpoint holding the dequantised weights must decode identically."""
    import json
    from safetensors.torch import save_file
    from onecat_vllm.config import ModelConfig
    from onecat_vllm.loader.weights import dummy_init, to_hf_state_dict
    from onecat_vllm.models import build_model
    base = dict(architectures=["LlamaForCausalLM"], hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                num_key_value_heads=2, head_dim=32, vocab_size=300, max_position_embeddings=256)
    m = build_model(ModelConfig.from_hf_dict(base, dtype=torch.float32), "cpu")
    dummy_init(m, 0, std=0.05)
    dense, quant = {}, {}
    for name, w in to_hf_state_dict(m).items():
        if not name.endswith("proj.weight"):
            dense[name] = quant[name] = w.contiguous()
            continue
        stem = name[: -len(".weight")]
        if scheme == "int4-group":
            g = 128
            wg = w.float().view(w.shape[0], -1, g)
            scale = (wg.abs().amax(-1) / 7.0).clamp_min(1e-8).half()
            codes = (torch.round(wg / scale.float().unsqueeze(-1)).clamp(-8, 7) + 8).to(torch.int32).view(w.shape[0], -1)
            packed = torch.zeros(w.shape[0], w.shape[1] // 8, dtype=torch.int32)
            for j in range(8):
                packed |= codes[:, j::8] << (4 * j)
            quant[stem + ".weight_packed"], quant[stem + ".weight_scale"] = packed, scale
            quant[stem + ".weight_shape"] = torch.tensor(list(w.shape))
            dense[name] = ((codes.float() - 8.0).view(w.shape[0], -1, g) * scale.float().unsqueeze(-1)).view_as(w).contiguous()
        else:
            scale = (w.float().abs().amax(-1, keepdim=True) if scheme == "fp8-channel" else w.float().abs().amax().view(1)) / 448.0
            w8 = (w.float() / scale).to(torch.float8_e4m3fn)
            quant[name], quant[stem + ".weight_scale"] = w8, scale.float()
            quant[stem + ".input_scale"] = torch.ones(1)
            dense[name] = (w8.float() * scale).contiguous()
    weights = ({"num_bits": 4, "type": "int", "symmetric": True, "strategy": "group", "group_size": 128} if scheme == "int4-group" else
               {"num_bits": 8, "type": "float", "symmetric": True, "strategy": scheme.split("-")[1]})
    qcfg = {"quant_method": "compressed-tensors", "format": "pack-quantized" if scheme == "int4-group" else "float-quantized",
            "ignore": ["lm_head"], "config_groups": {"group_0": {"targets": ["Linear"], "weights": weights, "input_activations": None}}}
    outs = []
    for tag, sd, cfg in (("dense", dense, base), ("quant", quant, dict(base, quantization_config=qcfg))):
        d = tmp_path / tag
        d.mkdir()
        save_file(sd, str(d / "model.safetensors"))
        (d / "config.json").write_text(json.dumps(cfg))
        llm = LLM(model=str(d), max_model_len=128, dtype="float32", device="cpu")
        outs.append([o.outputs[0].token_ids for o in llm.generate(_prompts(300), SamplingParams(temperature=0, max_tokens=10, ignore_eos=True))])
        llm.shutdown()
    assert outs[0] == outs[1]


def test_gpt_oss_mxfp4_release_format_matches_its_dequantised_checkpoint(tmp_path):
    """GPT-OSS experts in the MXFP4 release layout (``*_blocks`` / ``*_scales``, alternating gate / up rows) against a bf16-layout
    checkpoint (``[E, H, 2I]`` with alternating columns) holding the dequantised values."""
    import json
    from safetensors.torch import save_file
    from onecat_vllm.config import ModelConfig
    from onecat_vllm.loader.weights import dummy_init, to_hf_state_dict
    from onecat_vllm.models import build_model
    from onecat_vllm.ops import ref
    base = dict(architectures=["GptOssForCausalLM"], hidden_size=64, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
                num_key_value_heads=2, head_dim=16, vocab_size=300, max_position_embeddings=256, num_local_experts=4, num_experts_per_tok=2,
                sliding_window=16, layer_types=["sliding_attention", "full_attention"], tie_word_embeddings=False)
    m = build_model(ModelConfig.from_hf_dict(base, dtype=torch.float32), "cpu")
    dummy_init(m, 0, std=0.05)
    common = {k: v.contiguous() for k, v in to_hf_state_dict(m).items() if ".mlp.experts." not in k}
    g = torch.Generator().manual_seed(1)
    E, H, I = 4, 64, 64
    dense, quant = dict(common), dict(common)
    for layer in range(2):
        pre = f"model.layers.{layer}.mlp.experts."
        gu_b = torch.randint(0, 256, (E, 2 * I, H // 32, 16), generator=g, dtype=torch.uint8)
        gu_s = torch.randint(118, 123, (E, 2 * I, H // 32), generator=g, dtype=torch.uint8)
        dn_b = torch.randint(0, 256, (E, H, I // 32, 16), generator=g, dtype=torch.uint8)
        dn_s = torch.randint(118, 123, (E, H, I // 32), generator=g, dtype=torch.uint8)
        gu_bias, dn_bias = torch.randn(E, 2 * I, generator=g) * 0.1, torch.randn(E, H, generator=g) * 0.1
        quant.update({pre + "gate_up_proj_blocks": gu_b, pre + "gate_up_proj_scales": gu_s, pre + "down_proj_blocks": dn_b,
                      pre + "down_proj_scales": dn_s, pre + "gate_up_proj_bias": gu_bias, pre + "down_proj_bias": dn_bias})
        gu = ref.mxfp4_dequantize(gu_b.reshape(E, 2 * I, H // 2), gu_s)      # [E, 2I, H], rows alternate gate / up
        dn = ref.mxfp4_dequantize(dn_b.reshape(E, H, I // 2), dn_s)          # [E, H, I]
        dense.update({pre + "gate_up_proj": gu.transpose(1, 2).contiguous(), pre + "down_proj": dn.transpose(1, 2).contiguous(),
                      pre + "gate_up_proj_bias": gu_bias, pre + "down_proj_bias": dn_bias})
    qcfg = {"quant_method": "mxfp4", "modules_to_not_convert": ["model.layers.*.self_attn", "model.layers.*.mlp.router", "model.embed_tokens", "lm_head"]}
    outs = []
    for tag, sd, cfg in (("dense", dense, base), ("quant", quant, dict(base, quantization_config=qcfg))):
        d = tmp_path / tag
        d.mkdir()
        save_file(sd, str(d / "model.safetensors"))
        (d / "config.json").write_text(json.dumps(cfg))
        llm = LLM(model=str(d), max_model_len=128, dtype="float32", device="cpu")
        outs.append([o.outputs[0].token_ids for o in llm.generate(_prompts(300), SamplingParams(temperature=0, max_tokens=10, ignore_eos=True))])
        llm.shutdown()
    assert outs[0] == outs[1]


def test_deepseek_v32_is_limited_to_contexts_where_dense_attention_is_exact():
    """The V3.2 indexer keeps index_topk keys per query; this engine runs dense attention, which is the same thing only up to that
    many tokens: longer contexts are refused, the default context is cut to the limit."""
    import pytest
    from onecat_vllm.config import EngineArgs
    cfg = dict(architectures=["DeepseekV32ForCausalLM"], hidden_size=256, num_hidden_layers=2, num_attention_heads=4, vocab_size=1000, q_lora_rank=64,
               kv_lora_rank=32, qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=16, n_routed_experts=4, num_experts_per_tok=2,
               moe_intermediate_size=64, index_topk=128, max_position_embeddings=4096)
    with pytest.raises(ValueError, match="indexer"):
        EngineArgs(hf_config=cfg, device="cpu", max_model_len=512).create_engine_config()
    assert EngineArgs(hf_config=cfg, device="cpu").create_engine_config().model_config.max_model_len == 128
    assert EngineArgs(hf_config=cfg, device="cpu", max_model_len=100).create_engine_config().model_config.max_model_len == 100
