"""Tensor-parallel plumbing on CPU: two gloo ranks in worker processes must reproduce the single-rank greedy decode."""
import pytest
import torch

from onecat_vllm import LLM, SamplingParams

CFG = dict(architectures=["LlamaForCausalLM"], hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
           num_key_value_heads=2, head_dim=32, vocab_size=1000, max_position_embeddings=256)


def _ckpt(tmp_path):
    from onecat_vllm.config import ModelConfig
    from onecat_vllm.loader.weights import dummy_init, save_pretrained
    from onecat_vllm.models import build_model
    m = build_model(ModelConfig.from_hf_dict(CFG, dtype=torch.float32), "cpu")
    dummy_init(m, 0, std=0.05)
    save_pretrained(m, CFG, str(tmp_path))
    return str(tmp_path)


@pytest.mark.timeout(300)
def test_tp2_cpu_matches_tp1(tmp_path):
    path = _ckpt(tmp_path)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 1000, (n,), generator=g).tolist() for n in (9, 33, 70)]
    sp = SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True)
    one = LLM(model=path, device="cpu", dtype="float32", max_model_len=128)
    ref = [o.outputs[0].token_ids for o in one.generate(prompts, sp)]
    one.shutdown()
    two = LLM(model=path, device="cpu", dtype="float32", max_model_len=128, tensor_parallel_size=2, distributed_executor_backend="mp")
    got = [o.outputs[0].token_ids for o in two.generate(prompts, sp)]
    two.shutdown()
    assert got == ref


@pytest.mark.timeout(120)
def test_worker_death_is_detected(tmp_path):
    """A worker that exits is noticed by the monitor thread and the next step raises instead of hanging."""
    import os
    path = _ckpt(tmp_path)
    llm = LLM(model=path, device="cpu", dtype="float32", max_model_len=128, tensor_parallel_size=2, distributed_executor_backend="mp")
    ex = llm.llm_engine.engine_core.core.executor
    victim = ex.procs[1]
    victim.terminate()  # host-side failure: the exact child we started
    victim.join(5)
    import time
    t0 = time.time()
    while not ex.is_failed and time.time() - t0 < 10:
        time.sleep(0.05)
    assert ex.is_failed
    with pytest.raises(Exception):
        llm.generate([[1, 2, 3]], SamplingParams(max_tokens=2))
    llm.shutdown()


CFG4 = dict(CFG, num_hidden_layers=5)


@pytest.mark.timeout(600)
@pytest.mark.parametrize("tp,pp", [(1, 2), (2, 2), (1, 3)])
def test_pipeline_parallel_cpu_matches_single(tmp_path, tp, pp):
    """Pipeline stages (gloo send/recv of the block output and the residual) reproduce the single-process greedy decode,
    including uneven layer splits, chunked prefill and sampling with seeds."""
    from onecat_vllm.config import ModelConfig
    from onecat_vllm.loader.weights import dummy_init, save_pretrained
    from onecat_vllm.models import build_model
    from onecat_vllm.parallel.state import pp_layer_range
    assert [pp_layer_range(5, r, 3) for r in range(3)] == [(0, 2), (2, 4), (4, 5)]
    m = build_model(ModelConfig.from_hf_dict(CFG4, dtype=torch.float32), "cpu")
    dummy_init(m, 0, std=0.05)
    save_pretrained(m, CFG4, str(tmp_path))
    path = str(tmp_path)
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, 1000, (n,), generator=g).tolist() for n in (7, 40, 90)]
    sps = [SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True), SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True),
           SamplingParams(temperature=0.9, seed=3, max_tokens=8, ignore_eos=True)]
    kw = dict(model=path, device="cpu", dtype="float32", max_model_len=128, max_num_batched_tokens=48)
    one = LLM(**kw)
    ref = [o.outputs[0].token_ids for o in one.generate(prompts, sps)]
    one.shutdown()
    many = LLM(**kw, tensor_parallel_size=tp, pipeline_parallel_size=pp, distributed_executor_backend="mp")
    got = [o.outputs[0].token_ids for o in many.generate(prompts, sps)]
    many.shutdown()
    assert got == ref


@pytest.mark.timeout(300)
def test_row_parallel_biases_join_the_sum_once(tmp_path):
    """Biases on the output projection and the down projection (attention_bias / mlp_bias): with two ranks their partial outputs are
    summed, so the bias must come from one rank only; the decode must equal the single-rank one."""
    from onecat_vllm.config import ModelConfig
    from onecat_vllm.loader.weights import dummy_init, save_pretrained
    from onecat_vllm.models import build_model
    cfg = dict(CFG, attention_bias=True, mlp_bias=True)
    m = build_model(ModelConfig.from_hf_dict(cfg, dtype=torch.float32), "cpu")
    dummy_init(m, 0, std=0.05)
    for n, p in m.named_parameters():
        if n.endswith("bias"):
            p.data.normal_(0.0, 0.3, generator=torch.Generator().manual_seed(3))
    assert m.model.layers[0].self_attn.o_proj.bias is not None and m.model.layers[0].mlp.down_proj.bias is not None
    save_pretrained(m, cfg, str(tmp_path))
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 1000, (n,), generator=g).tolist() for n in (9, 33)]
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    one = LLM(model=str(tmp_path), device="cpu", dtype="float32", max_model_len=128)
    ref = [o.outputs[0].token_ids for o in one.generate(prompts, sp)]
    one.shutdown()
    two = LLM(model=str(tmp_path), device="cpu", dtype="float32", max_model_len=128, tensor_parallel_size=2, distributed_executor_backend="mp")
    got = [o.outputs[0].token_ids for o in two.generate(prompts, sp)]
    two.shutdown()
    assert got == ref


@pytest.mark.timeout(300)
@pytest.mark.parametrize("arch,extra", [("Starcoder2ForCausalLM", dict(use_bias=True, tie_word_embeddings=False)),
                                        ("CohereForCausalLM", dict(logit_scale=0.25, tie_word_embeddings=False))])
def test_layer_norm_families_on_two_ranks(tmp_path, arch, extra):
    """Mean-and-variance layer norms are not part of the fused reduce + add + norm: the reduction runs first and the norm after it.
    Starcoder2 adds biases on every projection of an ungated feed-forward; Cohere sums attention and feed-forward before one reduction."""
    from onecat_vllm.config import ModelConfig
    from onecat_vllm.loader.weights import dummy_init, save_pretrained
    from onecat_vllm.models import build_model
    cfg = dict(CFG, architectures=[arch], **extra)
    m = build_model(ModelConfig.from_hf_dict(cfg, dtype=torch.float32), "cpu")
    dummy_init(m, 0, std=0.05)
    gb = torch.Generator().manual_seed(3)
    for n, p in m.named_parameters():
        if n.endswith("bias"):
            p.data.normal_(0.0, 0.3, generator=gb)
    save_pretrained(m, cfg, str(tmp_path))
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 1000, (n,), generator=g).tolist() for n in (9, 33)]
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    outs = []
    for tp in (1, 2):
        kw = dict(tensor_parallel_size=2, distributed_executor_backend="mp") if tp == 2 else {}
        llm = LLM(model=str(tmp_path), device="cpu", dtype="float32", max_model_len=128, **kw)
        outs.append([o.outputs[0].token_ids for o in llm.generate(prompts, sp)])
        llm.shutdown()
    assert outs[0] == outs[1]


CFG_MOE = dict(architectures=["Qwen3MoeForCausalLM"], hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
               num_key_value_heads=2, head_dim=16, vocab_size=500, max_position_embeddings=256, num_experts=8, num_experts_per_tok=2,
               moe_intermediate_size=32, norm_topk_prob=True)


@pytest.mark.timeout(600)
@pytest.mark.parametrize("ep_comm", ["reduce", "a2a"])
def test_expert_parallel_two_ranks_match_one(tmp_path, monkeypatch, ep_comm):
    """Expert parallelism over two gloo ranks, with the experts' partial sums riding the reduction and with tokens exchanged between
    the ranks (each routes half of the batch): both must reproduce the single-rank tokens."""
    from onecat_vllm.config import ModelConfig
    from onecat_vllm.loader.weights import dummy_init, save_pretrained
    from onecat_vllm.models import build_model
    m = build_model(ModelConfig.from_hf_dict(CFG_MOE, dtype=torch.float32), "cpu")
    dummy_init(m, 0, std=0.05)
    save_pretrained(m, CFG_MOE, str(tmp_path))
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 500, (n,), generator=g).tolist() for n in (9, 33, 1, 20)]
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    kw = dict(model=str(tmp_path), device="cpu", dtype="float32", max_model_len=128)
    one = LLM(**kw)
    ref = [o.outputs[0].token_ids for o in one.generate(prompts, sp)]
    one.shutdown()
    monkeypatch.setenv("ONECAT_EP_COMM", ep_comm)
    two = LLM(tensor_parallel_size=2, distributed_executor_backend="mp", enable_expert_parallel=True, **kw)
    got = [o.outputs[0].token_ids for o in two.generate(prompts, sp)]
    two.shutdown()
    assert got == ref
