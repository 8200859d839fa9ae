"""Multimodal inputs on CPU: placeholder expansion and hashing, the encoder cache's budget logic, the scheduler cutting a prefill
chunk at an item that does not fit, the runner replacing placeholder rows by (cached) encoder outputs, and the Qwen2-VL vision
tower against Hugging Face's."""
import pytest
import torch

from onecat_vllm import LLM, SamplingParams

IMG = 250
CFG = dict(architectures=["Qwen2VLForConditionalGeneration"], hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
           num_key_value_heads=2, head_dim=16, vocab_size=300, max_position_embeddings=1024, rms_norm_eps=1e-6, rope_theta=1e4,
           image_token_id=IMG)


def test_processor_expands_placeholders_and_hashes_items():
    from onecat_vllm.multimodal import MultiModalProcessor
    p = MultiModalProcessor({"image": IMG}, 64)
    a, b = torch.randn(5, 64), torch.randn(3, 64)
    out = p.apply([1, IMG, 2, 3, IMG, 4], {"image": [a, {"image_embeds": b}]})
    assert out.token_ids == [1] + [IMG] * 5 + [2, 3] + [IMG] * 3 + [4]
    assert [(f.offset, f.length, f.kind) for f in out.features] == [(1, 5, "embeds"), (8, 3, "embeds")]
    assert out.features[0].mm_hash != out.features[1].mm_hash
    assert p.apply([IMG], {"image": a.clone()}).features[0].mm_hash == out.features[0].mm_hash      # content, not identity
    px = {"pixel_values": torch.randn(16, 12), "image_grid_thw": (1, 4, 4)}
    assert p.apply([IMG], {"image": px}).features[0].length == 4 and p.apply([IMG], {"image": px}).features[0].kind == "pixels"
    with pytest.raises(ValueError):
        p.apply([1, 2], {"image": a})
    with pytest.raises(ValueError):
        p.apply([IMG, IMG], {"image": a})


def test_encoder_cache_manager_shares_and_evicts():
    from types import SimpleNamespace
    from onecat_vllm.core.encoder_cache_manager import EncoderCacheManager
    from onecat_vllm.multimodal import MultiModalFeature
    m = EncoderCacheManager(10)
    f = lambda h, n: MultiModalFeature("image", h, 0, n, "embeds")
    r1 = SimpleNamespace(request_id="a", mm_features=[f("x", 6)])
    r2 = SimpleNamespace(request_id="b", mm_features=[f("x", 6), f("y", 5)])
    assert not m.check_and_update_cache(r1, 0) and m.can_allocate(r1, 0, 100)
    m.allocate(r1, 0)
    assert m.check_and_update_cache(r2, 0)                       # same image: shared entry
    assert not m.can_allocate(r2, 1, 100)                        # 6 + 5 > 10 and nothing is freeable
    m.free_encoder_input(r1, 0)
    assert not m.can_allocate(r2, 1, 100)                        # r2 still references x
    m.free_encoder_input(r2, 0)
    assert m.num_freeable_slots == 10 and m.num_free_slots == 4  # x is unreferenced but still cached
    r3 = SimpleNamespace(request_id="c", mm_features=[f("x", 6)])
    assert m.check_and_update_cache(r3, 0)                       # ... and can be picked up again
    m.free(r3)
    assert m.can_allocate(r2, 1, 100) and m.get_freed_mm_hashes() == ["x"]   # evicted to make room
    assert not m.can_allocate(r2, 1, 4)                          # the per-step encoder budget binds too


def _embed_table(llm):
    return llm.llm_engine.engine_core.core.executor.worker.runner.model.model.embed_tokens.weight.detach().clone()


def test_image_embeddings_replace_placeholder_rows_end_to_end():
    """An image given as embeddings equal to the embedding-table rows of some token ids must behave exactly like those token ids;
    a different image must change the output; a small encoder budget splits the prefill at the item without changing the tokens."""
    sp = SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True)
    kw = dict(hf_config=CFG, device="cpu", dtype="float32", max_model_len=512, seed=0)
    llm = LLM(**kw)
    tab = _embed_table(llm)
    stand_in = [11, 12, 13, 14, 15, 16]
    img = tab[stand_in]
    text = llm.generate([[5, 6] + stand_in + [7, 8, 9]], sp)[0].outputs[0].token_ids
    mm = llm.generate([{"prompt_token_ids": [5, 6, IMG, 7, 8, 9], "multi_modal_data": {"image": img}}], sp)[0]
    assert mm.outputs[0].token_ids == text and len(mm.prompt_token_ids) == 11
    other = llm.generate([{"prompt_token_ids": [5, 6, IMG, 7, 8, 9], "multi_modal_data": {"image": torch.randn(6, 64) * 0.3}}], sp)[0]
    assert other.outputs[0].token_ids != text
    runner = llm.llm_engine.engine_core.core.executor.worker.runner
    sched = llm.llm_engine.engine_core.core.scheduler
    assert sched.encoder_cache_manager.num_freeable_slots == sched.encoder_cache_manager.cache_size   # nothing is referenced any more
    # two requests with the same image in one batch: one encoder-cache entry
    outs = llm.generate([{"prompt_token_ids": [5, 6, IMG, 7, 8, 9], "multi_modal_data": {"image": img}},
                         {"prompt_token_ids": [5, 6, IMG, 7, 8, 9], "multi_modal_data": {"image": img.clone()}}], sp)
    assert [o.outputs[0].token_ids for o in outs] == [text, text]
    assert len([h for h in runner.encoder_cache]) <= 2
    llm.shutdown()
    # chunked prefill through the item (budget of 4 tokens per step) and an encoder cache that holds one item at a time
    small = LLM(max_num_batched_tokens=4, **kw)
    small.llm_engine.engine_core.core.scheduler.encoder_cache_manager.__init__(8)
    long_img = tab[[21, 22, 23, 24, 25, 26, 27]]
    want = small.generate([[5, 6] + stand_in + [7] + [21, 22, 23, 24, 25, 26, 27] + [8, 9]], sp)[0].outputs[0].token_ids
    got = small.generate([{"prompt_token_ids": [5, 6, IMG, 7, IMG, 8, 9], "multi_modal_data": {"image": [img, long_img]}}], sp)[0].outputs[0].token_ids
    assert got == want
    small.shutdown()


def test_vision_tower_matches_hugging_face():
    tr = pytest.importorskip("transformers")
    try:
        from transformers.models.qwen2_vl.configuration_qwen2_vl import Qwen2VLVisionConfig
        from transformers.models.qwen2_vl.modeling_qwen2_vl import Qwen2VisionTransformerPretrainedModel
    except Exception as e:  # pragma: no cover
        pytest.skip(f"transformers has no Qwen2-VL vision tower: {e}")
    vc = dict(depth=2, embed_dim=32, hidden_size=48, num_heads=4, mlp_ratio=2, patch_size=4, spatial_merge_size=2, temporal_patch_size=2, in_channels=3)
    hf = Qwen2VisionTransformerPretrainedModel(Qwen2VLVisionConfig(**vc)).float().eval()
    for p in hf.parameters():
        torch.nn.init.normal_(p, std=0.2)
    from onecat_vllm.models.vision import VisionTower
    ours = VisionTower(vc, torch.float32).eval()
    used = sum(ours.load_weight("visual." + n, p.detach()) for n, p in hf.named_parameters())
    assert used == len(list(hf.named_parameters()))
    t, h, w = 2, 4, 6
    pix = torch.randn(t * h * w, 3 * 2 * 4 * 4)
    with torch.no_grad():
        ref = hf(pix, grid_thw=torch.tensor([[t, h, w]]))
        ref = ref[0] if isinstance(ref, (tuple, list)) else getattr(ref, "pooler_output", ref)
        got = ours(pix, (t, h, w))
    assert got.shape == (t * h * w // 4, 48)
    assert torch.allclose(got, ref, atol=2e-4, rtol=2e-4), float((got - ref).abs().max())


def test_qwen2_vl_with_an_image_matches_hugging_face(tmp_path):
    """The whole model on a prompt with an image: vision tower, placeholder rows, and the (temporal, height, width) rotary positions
    of the image grid and of the text after it. Greedy tokens must equal Hugging Face's."""
    tr = pytest.importorskip("transformers")
    try:
        from transformers import Qwen2VLConfig, Qwen2VLForConditionalGeneration
    except Exception as e:  # pragma: no cover
        pytest.skip(f"transformers has no Qwen2-VL: {e}")
    vc = dict(depth=2, embed_dim=32, hidden_size=64, num_heads=4, mlp_ratio=2, patch_size=4, spatial_merge_size=2, temporal_patch_size=2, in_channels=3)
    text = dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, vocab_size=300,
                max_position_embeddings=1024, rms_norm_eps=1e-6, rope_theta=1e4, rope_scaling={"type": "mrope", "mrope_section": [2, 3, 3]},
                tie_word_embeddings=False)
    cfg = Qwen2VLConfig(text_config=text, vision_config=vc, image_token_id=IMG, video_token_id=251, vision_start_token_id=252, vision_end_token_id=253)
    torch.manual_seed(0)
    hf = Qwen2VLForConditionalGeneration(cfg).float().eval()
    for n, p in hf.named_parameters():
        torch.nn.init.normal_(p, std=0.5 if "norm" not in n else 0.1)
        if "norm" in n and n.endswith("weight"):
            p.data.add_(1.0)
    hf.save_pretrained(str(tmp_path), safe_serialization=True)
    import json
    d = json.loads((tmp_path / "config.json").read_text())
    d["architectures"] = ["Qwen2VLForConditionalGeneration"]
    (tmp_path / "config.json").write_text(json.dumps(d))

    t, h, w = 1, 4, 6                     # 24 patches -> 6 positions on a 2 x 3 grid
    pix = torch.randn(t * h * w, 3 * 2 * 4 * 4)
    n_img = t * h * w // 4
    prompt = [5, 6, 252, IMG, 253, 7, 8, 9]
    ids = torch.tensor([[5, 6, 252] + [IMG] * n_img + [253, 7, 8, 9]])
    with torch.no_grad():
        ref = hf.generate(input_ids=ids, attention_mask=torch.ones_like(ids), pixel_values=pix, image_grid_thw=torch.tensor([[t, h, w]]),
                          mm_token_type_ids=(ids == IMG).long(), max_new_tokens=10, do_sample=False, eos_token_id=None, pad_token_id=0)[0, ids.shape[1]:].tolist()
    llm = LLM(model=str(tmp_path), device="cpu", dtype="float32", max_model_len=128)
    assert llm.llm_engine.cfg.model_config.mrope_section == (2, 3, 3)
    sp = SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True)
    got = llm.generate([{"prompt_token_ids": prompt, "multi_modal_data": {"image": {"pixel_values": pix, "image_grid_thw": (t, h, w)}}}], sp)[0].outputs[0].token_ids
    # the same prompt without the rotary sections' grid would differ: text-only request through the same engine stays consistent
    plain = llm.generate([[5, 6, 7, 8, 9]], sp)[0].outputs[0].token_ids
    with torch.no_grad():
        ref_plain = hf.generate(input_ids=torch.tensor([[5, 6, 7, 8, 9]]), max_new_tokens=10, do_sample=False, eos_token_id=None, pad_token_id=0)[0, 5:].tolist()
    llm.shutdown()
    assert plain == ref_plain
    assert got == ref
    with torch.no_grad():  # ... and the grid matters: Hugging Face with sequential positions for the same inputs answers differently
        seq = hf(input_ids=ids, attention_mask=torch.ones_like(ids), pixel_values=pix, image_grid_thw=torch.tensor([[t, h, w]]),
                 mm_token_type_ids=(ids == IMG).long(), position_ids=torch.arange(ids.shape[1]).view(1, 1, -1).expand(3, 1, -1)).logits[0, -1].argmax().item()
    assert seq != ref[0]
