"""Async scheduling on the CPU engine: with one step in flight the outputs must be exactly those of the plain loop."""
import pytest
import torch

from onecat_vllm import LLM, SamplingParams

CFG = dict(architectures=["LlamaForCausalLM"], hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
           num_key_value_heads=2, head_dim=32, vocab_size=1000, max_position_embeddings=512)


def _prompts(seed=0, lens=(9, 33, 70, 5, 120, 17)):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, 1000, (n,), generator=g).tolist() for n in lens]


def _llm(**kw):
    return LLM(model="dummy", hf_config=CFG, device="cpu", dtype="float32", max_model_len=256, max_num_seqs=4, max_num_batched_tokens=64, **kw)


@pytest.mark.timeout(300)
def test_outputs_match_the_plain_loop_with_chunked_prefill_and_queueing():
    # six requests over four running slots with a 64-token step budget: chunked prefills, mixed steps, requests that finish by length
    # (predicted: no wasted step) and by EOS (found one step late: the extra token is dropped)
    sps = [SamplingParams(temperature=0.0, max_tokens=m, ignore_eos=(i % 2 == 0)) for i, m in enumerate((12, 30, 7, 1, 25, 16))]
    ref_llm = _llm()
    ref = [(o.outputs[0].token_ids, o.outputs[0].finish_reason) for o in ref_llm.generate(_prompts(), sps)]
    ref_llm.shutdown()
    a = _llm(async_scheduling=True)
    core = a.llm_engine.engine_core.core
    assert core.async_scheduling
    launched = []
    orig = core.executor.launch_model
    core.executor.launch_model = lambda so: (launched.append(so.total_num_scheduled_tokens), orig(so))[1]
    got = [(o.outputs[0].token_ids, o.outputs[0].finish_reason) for o in a.generate(_prompts(), sps)]
    assert got == ref
    assert len(launched) > 10, "steps must have gone through the launch / collect path"
    # a second batch on the same engine: nothing stale is left behind by the trailing step of the first
    again = [(o.outputs[0].token_ids, o.outputs[0].finish_reason) for o in a.generate(_prompts(), sps)]
    a.shutdown()
    assert again == ref


@pytest.mark.timeout(300)
def test_requests_that_need_their_tokens_on_the_host_run_the_plain_order():
    sp_plain = SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True)
    sp_pen = SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True, repetition_penalty=1.3, logprobs=2)
    ref_llm = _llm()
    ref = [o.outputs[0].token_ids for o in ref_llm.generate(_prompts(1, (20, 31)), [sp_plain, sp_pen])]
    ref_llm.shutdown()
    a = _llm(async_scheduling=True)
    outs = a.generate(_prompts(1, (20, 31)), [sp_plain, sp_pen])
    a.shutdown()
    assert [o.outputs[0].token_ids for o in outs] == ref and outs[1].outputs[0].logprobs is not None


@pytest.mark.timeout(300)
def test_seeded_sampling_is_unchanged():
    sp = SamplingParams(temperature=0.8, top_p=0.9, seed=7, max_tokens=14, ignore_eos=True)
    r = _llm()
    ref = [o.outputs[0].token_ids for o in r.generate(_prompts(2, (11, 40, 23)), sp)]
    r.shutdown()
    a = _llm(async_scheduling=True)
    got = [o.outputs[0].token_ids for o in a.generate(_prompts(2, (11, 40, 23)), sp)]
    a.shutdown()
    assert got == ref


@pytest.mark.timeout(300)
def test_a_stop_found_one_step_late_drops_the_extra_token():
    base = SamplingParams(temperature=0.0, max_tokens=20, ignore_eos=True)
    r = _llm()
    free = r.generate(_prompts(3, (15, 28, 9)), base)
    stops = [o.outputs[0].token_ids[6] for o in free]          # a token each request is known to produce mid-way
    sps = [SamplingParams(temperature=0.0, max_tokens=20, ignore_eos=True, stop_token_ids=[s]) for s in stops]
    ref = [(o.outputs[0].token_ids, o.outputs[0].finish_reason) for o in r.generate(_prompts(3, (15, 28, 9)), sps)]
    r.shutdown()
    assert all(len(t) < 20 and fr == "stop" for t, fr in ref)
    a = _llm(async_scheduling=True)
    got = [(o.outputs[0].token_ids, o.outputs[0].finish_reason) for o in a.generate(_prompts(3, (15, 28, 9)), sps)]
    # the engine stays consistent afterwards (blocks of the stopped requests were freed while a step that still wrote to them ran)
    more = [o.outputs[0].token_ids for o in a.generate(_prompts(3, (15, 28, 9)), base)]
    a.shutdown()
    assert got == ref and more == [o.outputs[0].token_ids for o in free]


@pytest.mark.parametrize("async_on", [False, True])
def test_a_request_that_can_never_be_scheduled_ends_with_an_error(async_on):
    """An idle engine whose scheduler keeps placing nothing for its first waiting request gives that request an error finish
    instead of spinning (host-side fault: the block pool is made to look too small for the prompt)."""
    import torch
    from onecat_vllm import LLM, SamplingParams
    cfg = dict(architectures=["LlamaForCausalLM"], hidden_size=64, intermediate_size=128, num_hidden_layers=1, num_attention_heads=4,
               num_key_value_heads=2, head_dim=16, vocab_size=300, max_position_embeddings=256)
    llm = LLM(hf_config=cfg, device="cpu", dtype="float32", max_model_len=128, async_scheduling=async_on)
    core = llm.llm_engine.engine_core.core
    km = core.scheduler.kv_cache_manager
    orig = km.allocate_slots
    km.allocate_slots = lambda *a, **k: None            # "no room", for every request, for ever
    outs = llm.generate([[1, 2, 3, 4, 5]], SamplingParams(temperature=0, max_tokens=4))
    assert outs[0].finished and outs[0].outputs[0].finish_reason == "error" and outs[0].outputs[0].token_ids == []
    km.allocate_slots = orig
    ok = llm.generate([[1, 2, 3, 4, 5]], SamplingParams(temperature=0, max_tokens=4, ignore_eos=True))
    assert len(ok[0].outputs[0].token_ids) == 4         # the engine is still good for other requests
    llm.shutdown()
