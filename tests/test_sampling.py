"""Sampler and rejection sampler semantics on CPU."""
import pytest
import torch

from onecat_vllm.ops import ref
from onecat_vllm.sample.metadata import SamplingMetadata
from onecat_vllm.sample.rejection_sampler import RejectionSampler
from onecat_vllm.sample.sampler import Sampler
from onecat_vllm.sampling_params import SamplingParams


def md(B, **kw):
    base = dict(temperature=None, all_greedy=True, all_random=False, top_p=None, top_k=None, min_p=None, generators={}, max_num_logprobs=None,
                no_penalties=True)
    base.update(kw)
    m = SamplingMetadata(**base)
    m.output_token_ids = kw.get("output_token_ids", [[] for _ in range(B)])
    m.logit_bias = [None] * B
    m.allowed_token_ids = [None] * B
    return m


def test_greedy_and_logprobs_from_raw_logits():
    lg = torch.tensor([[0.1, 2.0, -1.0, 0.5], [3.0, 0.0, 0.0, 0.0]])
    out = Sampler()(lg, md(2, max_num_logprobs=2))
    assert out.sampled_token_ids.tolist() == [1, 0]
    ids, vals, ranks = out.logprobs
    assert ids[0].tolist()[:2] == [1, 1] and ranks.tolist() == [1, 1]
    assert torch.allclose(vals[0, 0], torch.log_softmax(lg[0], -1)[1])


def test_top_k_top_p_min_p_masks():
    lg = torch.log(torch.tensor([[0.5, 0.3, 0.15, 0.05]]))
    k = ref.top_k_top_p_min_p(lg.clone(), torch.tensor([2]), None, None)
    assert torch.isinf(k[0, 2:]).all() and not torch.isinf(k[0, :2]).any()
    p = ref.top_k_top_p_min_p(lg.clone(), None, torch.tensor([0.7]), None)
    assert torch.isinf(p[0, 2:]).all() and not torch.isinf(p[0, :2]).any()
    m = ref.top_k_top_p_min_p(lg.clone(), None, None, torch.tensor([0.5]))
    assert torch.isinf(m[0, 2:]).all()


def test_seeded_random_sampling_reproducible_and_distribution():
    torch.manual_seed(0)
    lg = torch.log(torch.tensor([[0.7, 0.2, 0.1]])).repeat(4000, 1)
    g = {i: torch.Generator().manual_seed(i) for i in range(4000)}
    m = md(4000, temperature=torch.ones(4000), all_greedy=False, all_random=True, generators=g)
    a = Sampler()(lg, m).sampled_token_ids
    g2 = {i: torch.Generator().manual_seed(i) for i in range(4000)}
    b = Sampler()(lg, md(4000, temperature=torch.ones(4000), all_greedy=False, all_random=True, generators=g2)).sampled_token_ids
    assert torch.equal(a, b)
    freq = torch.bincount(a, minlength=3).float() / 4000
    assert abs(freq[0] - 0.7) < 0.03 and abs(freq[1] - 0.2) < 0.03


def test_penalties_and_logit_processors():
    lg = torch.zeros(1, 5)
    lg[0, 2] = 1.0
    m = md(1, no_penalties=False, presence_penalties=torch.tensor([2.0]), frequency_penalties=torch.tensor([0.0]),
           repetition_penalties=torch.tensor([1.0]), output_token_ids=[[2]])
    m.prompt_token_ids = [[]]
    assert Sampler()(lg.clone(), m).sampled_token_ids.item() != 2
    m2 = md(1)
    m2.allowed_token_ids = [[3, 4]]
    m2.logit_bias = [{4: 5.0}]
    assert Sampler()(lg.clone(), m2).sampled_token_ids.item() == 4
    m3 = md(1, output_token_ids=[[]])
    m3.min_tokens = {0: (2, {2})}
    assert Sampler()(lg.clone(), m3).sampled_token_ids.item() != 2
    m4 = md(1, output_token_ids=[[1]])
    m4.bad_words_token_ids = {0: [[1, 2]]}
    assert Sampler()(lg.clone(), m4).sampled_token_ids.item() != 2


def test_rejection_greedy_accepts_matching_prefix():
    V = 6
    tl = torch.full((2, 4, V), -5.0)
    for b, seq in enumerate([[1, 2, 3, 4], [1, 5, 0, 0]]):
        for i, t in enumerate(seq):
            tl[b, i, t] = 5.0
    draft = torch.tensor([[1, 2, 3], [1, 2, 3]])
    out = RejectionSampler()(draft, torch.tensor([3, 3]), tl, torch.tensor([4, 9]), md(2))
    assert RejectionSampler.parse_output(out) == [[1, 2, 3, 4], [1, 5]]


def test_rejection_random_is_unbiased_for_point_drafts():
    """With no draft probabilities the draft is a point mass: accept with prob p(x); the emitted token must follow p."""
    torch.manual_seed(0)
    p = torch.tensor([0.6, 0.3, 0.1])
    B = 6000
    tl = torch.log(p).view(1, 1, 3).repeat(B, 2, 1)
    draft = torch.zeros(B, 1, dtype=torch.long)
    m = md(B, temperature=torch.ones(B), all_greedy=False, all_random=True)
    out = RejectionSampler(seed=1)(draft, torch.ones(B, dtype=torch.long), tl, torch.full((B,), 2), m)
    first = out[:, 0]
    freq = torch.bincount(first, minlength=3).float() / B
    assert torch.allclose(freq, p, atol=0.03)
    accepted = (first == 0) & (out[:, 1] == 2)
    assert abs(accepted.float().mean() - 0.6) < 0.05  # bonus appended exactly when the draft was accepted


def test_rejection_synthetic_rate():
    B, k, V = 4000, 3, 8
    tl = torch.randn(B, k + 1, V)
    draft = torch.randint(0, V, (B, k))
    rs = RejectionSampler(synthetic_rates=[0.7, 0.7, 0.7], seed=3)
    out = rs(draft, torch.full((B,), k), tl, torch.zeros(B, dtype=torch.long), md(B))
    n_acc = torch.tensor([sum(1 for i in range(k) if row[i] == d[i]) for row, d in zip(out.tolist(), draft.tolist())]).float()
    lens = torch.tensor([len(r) for r in RejectionSampler.parse_output(out)]).float()
    # expected emitted tokens per step = 1 + 0.7 + 0.49 + 0.343
    assert abs(lens.mean() - 2.533) < 0.08
    rs2 = RejectionSampler(synthetic_rates=[0.7, 0.7, 0.7], seed=3)
    out2 = rs2(draft, torch.full((B,), k), tl, torch.zeros(B, dtype=torch.long), md(B))
    assert torch.equal(out, out2), "the seeded acceptance stream must be reproducible"


def test_sampling_params_validation():
    with pytest.raises(ValueError):
        SamplingParams(top_p=0.0)
    with pytest.raises(ValueError):
        SamplingParams(n=2, temperature=0.0)
    sp = SamplingParams(temperature=0.0, top_k=5, top_p=0.5)
    assert sp.top_k == 0 and sp.top_p == 1.0  # greedy neutralises the random knobs
    assert SamplingParams.from_dict(sp.to_dict()).temperature == 0.0


def test_prompt_logprobs_match_a_direct_forward_across_chunks():
    """prompt_logprobs=k returns, for every prompt position after the first, the log-probability of the actual token plus the top k,
    identical whether the prompt is prefilled in one chunk or several (reference test model: tests/v1/sample/test_logprobs.py)."""
    import torch
    from onecat_vllm import LLM, SamplingParams
    cfg = dict(architectures=["LlamaForCausalLM"], hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
               num_key_value_heads=2, head_dim=16, vocab_size=300, max_position_embeddings=256)
    prompt = [(7 * i) % 290 + 1 for i in range(45)]
    got = {}
    for chunk in (8192, 16):
        llm = LLM(hf_config=cfg, device="cpu", dtype="float32", max_model_len=128, max_num_batched_tokens=chunk)
        out = llm.generate([{"prompt_token_ids": prompt}], SamplingParams(temperature=0.0, max_tokens=2, prompt_logprobs=3, logprobs=1))[0]
        plp = out.prompt_logprobs
        assert plp[0] is None and len(plp) == len(prompt)
        for pos in range(1, len(prompt)):
            d = plp[pos]
            assert prompt[pos] in d and 3 <= len(d) <= 4
            assert all(v.logprob <= 0 for v in d.values())
        got[chunk] = [plp[pos][prompt[pos]].logprob for pos in range(1, len(prompt))]
        llm.shutdown()
    assert max(abs(a - b) for a, b in zip(got[8192], got[16])) < 1e-4
    # ranks: the actual token's rank is 1 exactly when it is the arg-max
    assert any(v.rank == 1 for d in plp[1:] for v in d.values())


def test_repetition_detection_and_thinking_budget():
    from onecat_vllm import LLM, SamplingParams
    from onecat_vllm.sampling_params import RepetitionDetectionParams
    r = RepetitionDetectionParams(max_pattern_size=3, min_pattern_size=2, min_count=3)
    assert r.hit([9, 1, 2, 1, 2, 1, 2]) and r.hit([5, 1, 2, 3, 1, 2, 3, 1, 2, 3]) and not r.hit([1, 2, 1, 2, 3, 1, 2]) and not r.hit([7, 7, 7])
    assert RepetitionDetectionParams(max_pattern_size=1, min_count=3).hit([4, 7, 7, 7])
    cfg = dict(architectures=["LlamaForCausalLM"], hidden_size=64, intermediate_size=128, num_hidden_layers=1, num_attention_heads=4,
               num_key_value_heads=2, head_dim=16, vocab_size=300, max_position_embeddings=256)
    llm = LLM(hf_config=cfg, device="cpu", dtype="float32", max_model_len=128, tokenizer="byte")
    # a random tiny model falls into a loop quickly under greedy decoding: detection stops it early with its own reason
    base = llm.generate(["abc"], SamplingParams(temperature=0.0, max_tokens=60, ignore_eos=True))[0].outputs[0]
    det = llm.generate(["abc"], SamplingParams(temperature=0.0, max_tokens=60, ignore_eos=True,
                                               repetition_detection=RepetitionDetectionParams(max_pattern_size=8, min_count=3)))[0].outputs[0]
    if r.__class__(max_pattern_size=8, min_count=3).hit(base.token_ids) or len(det.token_ids) < 60:
        assert det.stop_reason == "repetition" and det.finish_reason == "stop" and len(det.token_ids) < 60
        assert det.token_ids == base.token_ids[: len(det.token_ids)]
    # thinking budget: the byte tokenizer has no single-token <think>, so the request is refused
    import pytest
    with pytest.raises(ValueError):
        llm.generate(["x"], SamplingParams(max_tokens=4, thinking_token_budget=2))
    llm.shutdown()
    # the sampler forces the think-end token once the budget is used
    import torch
    from onecat_vllm.sample.metadata import SamplingMetadata
    from onecat_vllm.sample.sampler import Sampler
    md = SamplingMetadata(temperature=None, all_greedy=True, all_random=False, top_p=None, top_k=None, min_p=None, generators={},
                          max_num_logprobs=None, no_penalties=True, output_token_ids=[[5, 100, 7, 8], [5, 100, 7], [100, 1, 2, 101, 3, 4, 5]],
                          logit_bias=[None] * 3, allowed_token_ids=[None] * 3, thinking={0: (2, 100, 101), 1: (2, 100, 101), 2: (2, 100, 101)})
    lg = torch.zeros(3, 200)
    lg[:, 42] = 5.0
    out = Sampler()(lg, md).sampled_token_ids.tolist()
    assert out == [101, 42, 42]  # row 0 used its budget; row 1 has one token left; row 2 already closed its block


def test_user_logits_processor_is_applied_per_request():
    """An engine-level logits processor named by its import path sees every sampling step with per-request context
    (ids, extra_args) and can reshape the logits (reference: v1/sample/logits_processor/ custom processors)."""
    import torch
    from onecat_vllm import LLM, SamplingParams
    cfg = dict(architectures=["LlamaForCausalLM"], hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
               num_key_value_heads=2, head_dim=16, vocab_size=300, max_position_embeddings=256)
    llm = LLM(hf_config=cfg, device="cpu", dtype="float32", max_model_len=128, logits_processors=["tests.logits_processor_example:BanOrForce"])
    prompt = {"prompt_token_ids": list(range(3, 20))}
    plain = llm.generate([prompt], SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True))[0].outputs[0].token_ids
    banned = llm.generate([prompt], SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True, extra_args={"banned": plain}))[0].outputs[0].token_ids
    assert not set(banned) & set(plain)
    outs = llm.generate([prompt, prompt], [SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True, extra_args={"force": 7}),
                                           SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)])
    forced, other = outs[0].outputs[0].token_ids, outs[1].outputs[0].token_ids
    assert forced[1::2] == [7, 7, 7] and forced[0] == plain[0] and other == plain
    llm.shutdown()
