"""Scheduler / KV-cache manager / block pool logic on CPU with a fake model runner (no weights, no device)."""
import pytest

from onecat_vllm.config import CacheConfig, ModelConfig, SchedulerConfig, SpeculativeConfig, VllmConfig
from onecat_vllm.core.block_pool import BlockPool
from onecat_vllm.core.kv_cache_manager import KVCacheManager
from onecat_vllm.core.kv_cache_utils import FreeKVCacheBlockQueue, KVCacheBlock, hash_block_tokens, make_block_hasher
from onecat_vllm.core.sched_output import ModelRunnerOutput
from onecat_vllm.core.scheduler import Scheduler
from onecat_vllm.request import Request, RequestStatus
from onecat_vllm.sampling_params import SamplingParams


def make_scheduler(num_blocks=64, budget=64, max_seqs=8, max_len=256, policy="fcfs", spec=None, prefix=True, chunked=True):
    cfg = VllmConfig(ModelConfig(max_model_len=max_len), CacheConfig(block_size=16, enable_prefix_caching=prefix),
                     scheduler_config=SchedulerConfig(max_num_batched_tokens=budget, max_num_seqs=max_seqs, max_model_len=max_len, policy=policy,
                                                      enable_chunked_prefill=chunked),
                     speculative_config=spec or SpeculativeConfig(), device="cpu")
    return Scheduler(cfg, num_blocks)


def req(rid, n, max_tokens=8, priority=0, s=None, tokens=None, arrival=None):
    r = Request(rid, tokens or list(range(1, n + 1)), SamplingParams(max_tokens=max_tokens, ignore_eos=True, temperature=0.0), eos_token_id=0,
                priority=priority, arrival_time=arrival, block_hasher=s.block_hasher if s else None)
    return r


def fake_output(so, token=7, spec=None):
    ids = list(so.num_scheduled_tokens)
    return ModelRunnerOutput(req_ids=ids, sampled_token_ids=[[token] for _ in ids], spec_token_ids=spec)


def run_step(s, token=7):
    so = s.schedule()
    sampled = []
    for rid, n in so.num_scheduled_tokens.items():
        r = s.requests[rid]
        sampled.append([token] if r.num_computed_tokens >= r.num_tokens else [])
    out = s.update_from_output(so, ModelRunnerOutput(req_ids=list(so.num_scheduled_tokens), sampled_token_ids=sampled))
    return so, out


def test_free_queue_order_and_removal():
    blocks = [KVCacheBlock(i) for i in range(5)]
    q = FreeKVCacheBlockQueue(blocks)
    assert q.popleft().block_id == 0
    q.remove(blocks[2])
    q.append(blocks[0])
    assert [b.block_id for b in q.get_all_free_blocks()] == [1, 3, 4, 0]
    assert q.num_free_blocks == 4
    with pytest.raises(RuntimeError):
        q.remove(blocks[2])


def test_block_hash_chain_identifies_prefix():
    import hashlib
    fn = lambda b: hashlib.sha256(b).digest()
    h1 = hash_block_tokens(fn, None, (1, 2, 3))
    assert hash_block_tokens(fn, h1, (4, 5, 6)) != hash_block_tokens(fn, None, (4, 5, 6))
    assert hash_block_tokens(fn, None, (1, 2, 3), ("salt",)) != h1


def test_chunked_prefill_budget_and_decode():
    s = make_scheduler(budget=32)
    s.add_request(req("a", 50, s=s))
    s.add_request(req("b", 0, s=s, tokens=list(range(500, 520))))
    so, _ = run_step(s)
    assert so.num_scheduled_tokens == {"a": 32} and so.total_num_scheduled_tokens == 32
    so, _ = run_step(s)
    assert so.num_scheduled_tokens == {"a": 18, "b": 14}  # running first, waiting fills the rest
    so, outs = run_step(s)
    assert so.num_scheduled_tokens == {"a": 1, "b": 6}
    assert [o.request_id for o in outs[0].outputs] == ["a", "b"] or len(outs[0].outputs) >= 1
    so, _ = run_step(s)
    assert so.num_scheduled_tokens == {"a": 1, "b": 1}


def test_finish_by_length_frees_blocks():
    s = make_scheduler()
    s.add_request(req("a", 10, max_tokens=2, s=s))
    free0 = s.kv_cache_manager.block_pool.get_num_free_blocks()
    run_step(s)
    _, outs = run_step(s)
    assert outs[0].outputs[0].finish_reason is not None and str(outs[0].outputs[0].finish_reason) == "length"
    assert not s.has_unfinished_requests()
    assert s.kv_cache_manager.block_pool.get_num_free_blocks() == free0
    assert "a" in s.schedule().finished_req_ids


def test_stop_token_and_eos():
    s = make_scheduler()
    r = Request("a", [1, 2, 3], SamplingParams(max_tokens=10, stop_token_ids=[9]), eos_token_id=5)
    s.add_request(r)
    so = s.schedule()
    out = s.update_from_output(so, ModelRunnerOutput(req_ids=["a"], sampled_token_ids=[[9]]))
    assert out[0].outputs[0].stop_reason == 9 and str(out[0].outputs[0].finish_reason) == "stop"
    r2 = Request("b", [1, 2, 3], SamplingParams(max_tokens=10), eos_token_id=5)
    s.add_request(r2)
    so = s.schedule()
    out = s.update_from_output(so, ModelRunnerOutput(req_ids=["b"], sampled_token_ids=[[5]]))
    assert str(out[0].outputs[0].finish_reason) == "stop" and out[0].outputs[0].stop_reason is None


def test_prefix_cache_hit_and_last_token_recompute():
    s = make_scheduler(budget=256)
    toks = list(range(100, 148))  # 3 full blocks
    s.add_request(req("a", 0, max_tokens=1, s=s, tokens=toks))
    run_step(s)
    s.schedule()
    s.add_request(req("b", 0, max_tokens=1, s=s, tokens=toks))
    so = s.schedule()
    # 48 tokens cached, but at most num_tokens-1 may hit → 2 blocks (32 tokens), 16 recomputed
    assert so.num_scheduled_tokens["b"] == 16 and so.scheduled_new_reqs[0].num_computed_tokens == 32
    s.add_request(req("c", 0, max_tokens=1, s=s, tokens=toks + [1, 2, 3]))
    s.update_from_output(so, ModelRunnerOutput(req_ids=["b"], sampled_token_ids=[[1]]))
    so = s.schedule()
    assert so.scheduled_new_reqs[0].num_computed_tokens == 48


def test_preemption_fcfs_and_resume():
    s = make_scheduler(num_blocks=7, budget=256, prefix=False)  # 6 usable blocks
    s.add_request(req("a", 40, max_tokens=40, s=s))  # 3 blocks
    s.add_request(req("b", 40, max_tokens=40, s=s))  # 3 blocks
    run_step(s)
    preempted = False
    for _ in range(12):
        so, _ = run_step(s)
        if so.preempted_req_ids:
            assert so.preempted_req_ids == {"b"}  # newest running request goes first
            preempted = True
            break
    assert preempted and s.requests["b"].status == RequestStatus.PREEMPTED and s.requests["b"].num_computed_tokens == 0
    for _ in range(100):
        so, _ = run_step(s)
        if not s.has_unfinished_requests():
            break
    assert not s.has_unfinished_requests()


def test_priority_policy_orders_waiting_and_victims():
    s = make_scheduler(policy="priority", max_seqs=1)
    s.add_request(req("low", 5, priority=5, s=s, arrival=1.0))
    s.add_request(req("high", 5, priority=0, s=s, arrival=2.0))
    so = s.schedule()
    assert list(so.num_scheduled_tokens) == ["high"]


def test_abort_running_and_waiting():
    s = make_scheduler(max_seqs=1)
    s.add_request(req("a", 5, s=s))
    s.add_request(req("b", 5, s=s))
    s.schedule()
    s.finish_requests(["a", "b"], RequestStatus.FINISHED_ABORTED)
    assert not s.has_unfinished_requests() and s.finished_req_ids == {"a", "b"}


def test_spec_decode_accounting():
    spec = SpeculativeConfig(method="ngram", num_speculative_tokens=3)
    s = make_scheduler(spec=spec)
    s.add_request(req("a", 10, max_tokens=20, s=s))
    so = s.schedule()
    s.update_from_output(so, ModelRunnerOutput(req_ids=["a"], sampled_token_ids=[[7]], spec_token_ids=[[8, 9, 10]]))
    so = s.schedule()
    assert so.num_scheduled_tokens["a"] == 4 and so.scheduled_spec_decode_tokens["a"] == [8, 9, 10]
    r = s.requests["a"]
    assert r.num_computed_tokens == 14
    # two drafts accepted (+1 recovered token): one rejected draft is rolled back
    s.update_from_output(so, ModelRunnerOutput(req_ids=["a"], sampled_token_ids=[[8, 9, 42]], spec_token_ids=[[1, 2, 3]]))
    assert r.num_computed_tokens == 13 and r.output_token_ids == [7, 8, 9, 42]
    so = s.schedule()
    assert so.num_scheduled_tokens["a"] == 4


def test_kv_manager_lookahead_and_usage():
    m = KVCacheManager(num_blocks=10, block_size=16, max_model_len=256, enable_caching=False)
    r = Request("a", list(range(20)), SamplingParams(max_tokens=4))
    new = m.allocate_slots(r, 20, num_lookahead_tokens=13)
    assert len(new) == 3  # 33 tokens → 3 blocks
    assert m.usage == pytest.approx(3 / 9)
    m.free(r)
    assert m.usage == 0.0
    assert m.allocate_slots(Request("b", list(range(200)), SamplingParams()), 200) is None


def test_rejects_bad_requests():
    s = make_scheduler(max_len=32)
    with pytest.raises(ValueError):
        s.add_request(req("long", 40, s=s))
    s.add_request(req("x", 4, s=s))
    with pytest.raises(ValueError):
        s.add_request(req("x", 4, s=s))


def test_kv_events_are_published_over_zmq():
    """Block stored / removed events reach a ZMQ subscriber with increasing sequence numbers."""
    import msgpack
    import zmq
    from onecat_vllm import LLM, SamplingParams
    cfg = dict(architectures=["LlamaForCausalLM"], hidden_size=64, intermediate_size=128, num_hidden_layers=1, num_attention_heads=4,
               num_key_value_heads=2, head_dim=16, vocab_size=300, max_position_embeddings=256)
    ep = "ipc:///tmp/onecat-kv-events-test"
    llm = LLM(hf_config=cfg, device="cpu", dtype="float32", max_model_len=128, kv_events_config={"endpoint": ep, "topic": "kv"})
    sub = zmq.Context.instance().socket(zmq.SUB)
    sub.connect(ep)
    sub.setsockopt(zmq.SUBSCRIBE, b"kv")
    import time
    time.sleep(0.3)
    llm.generate([{"prompt_token_ids": list(range(1, 50))}], SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True))
    seqs, stored = [], 0
    while sub.poll(500):
        topic, seq, payload = sub.recv_multipart()
        seqs.append(int.from_bytes(seq, "big"))
        body = msgpack.unpackb(payload)
        stored += sum(1 for e in body["events"] if e["type"] == "BlockStored" and e["block_hash"])
    assert seqs == sorted(seqs) and len(seqs) >= 1 and stored >= 3
    sub.close(linger=0)
    llm.shutdown()


def test_general_plugins_run_once_and_register_models(monkeypatch):
    import onecat_vllm.utils.plugins as P
    from onecat_vllm.models import register_model, supported_architectures

    class EP:
        def __init__(self, name, fn):
            self.name, self._fn = name, fn

        def load(self):
            return self._fn

    calls = []
    eps = [EP("a", lambda: (calls.append("a"), register_model("MyOutOfTreeForCausalLM", "dense"))), EP("b", lambda: calls.append("b")),
           EP("broken", lambda: 1 / 0)]
    monkeypatch.setattr("importlib.metadata.entry_points", lambda group: eps if group == P.GENERAL_GROUP else [])
    monkeypatch.setattr(P, "_loaded", False)
    monkeypatch.setenv("ONECAT_PLUGINS", "a,broken")
    assert P.load_general_plugins() == ["a"] and calls == ["a"]
    assert "MyOutOfTreeForCausalLM" in supported_architectures()
    assert P.load_general_plugins() == []  # once per process


def test_older_gemma_config_formats_give_the_same_layer_layout():
    """Checkpoints written before ``layer_types`` / ``rope_parameters`` existed: Gemma2 alternates sliding and global layers, Gemma3
    makes every ``sliding_window_pattern``-th layer global and names its local rotary base ``rope_local_base_freq``."""
    from onecat_vllm.config import ModelConfig
    base = dict(hidden_size=64, num_attention_heads=4, num_key_value_heads=2, head_dim=16, query_pre_attn_scalar=16)
    g2 = ModelConfig.from_hf_dict(dict(base, architectures=["Gemma2ForCausalLM"], num_hidden_layers=4, sliding_window=4096))
    assert g2.sliding_layers == (0, 2) and g2.sliding_window == 4096 and g2.sandwich_norm and g2.hidden_act == "gelu_tanh"
    g3 = ModelConfig.from_hf_dict(dict(base, architectures=["Gemma3ForCausalLM"], num_hidden_layers=12, sliding_window=1024, sliding_window_pattern=6,
                                       rope_local_base_freq=10000.0, rope_theta=1e6, rope_scaling={"rope_type": "linear", "factor": 8.0},
                                       hidden_activation="gelu_pytorch_tanh"))
    assert g3.sliding_layers == (0, 1, 2, 3, 4, 6, 7, 8, 9, 10) and g3.rope_local_theta == 10000.0 and g3.rope_theta == 1e6
    assert g3.rope_scaling == {"rope_type": "linear", "factor": 8.0} and g3.hidden_act == "gelu_tanh" and g3.qk_norm
    new = ModelConfig.from_hf_dict(dict(base, architectures=["Gemma3ForCausalLM"], num_hidden_layers=4, sliding_window=16,
                                        layer_types=["sliding_attention", "full_attention", "sliding_attention", "full_attention"]))
    assert new.sliding_layers == (0, 2)


def test_rotary_scaling_rules_build_tables():
    """Every supported context-extension rule yields a finite [max_pos, rotary_dim] table; linear scaling equals position / factor
    and the dynamic rule equals the plain rule with its NTK-adjusted base."""
    import torch
    from onecat_vllm.ops import ref
    plain = ref.build_cos_sin_cache(16, 64, 1e4)
    lin = ref.build_cos_sin_cache(16, 64, 1e4, None, {"rope_type": "linear", "factor": 4.0})
    assert torch.allclose(lin[4::4][:8], plain[1:9], atol=1e-6)
    for sc in ({"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0, "original_max_position_embeddings": 32},
               {"rope_type": "yarn", "factor": 4.0, "original_max_position_embeddings": 32},
               {"type": "mrope", "mrope_section": [2, 3, 3]},
               {"rope_type": "longrope", "short_factor": [1.0] * 8, "long_factor": [2.0] * 8, "original_max_position_embeddings": 32},
               {"rope_type": "dynamic", "factor": 2.0, "original_max_position_embeddings": 32}):
        t = ref.build_cos_sin_cache(16, 64, 1e4, None, sc)
        assert t.shape == (64, 16) and torch.isfinite(t).all()
    dyn = ref.build_cos_sin_cache(16, 64, 1e4, None, {"rope_type": "dynamic", "factor": 2.0, "original_max_position_embeddings": 32})
    base = 1e4 * ((2.0 * 64 / 32) - 1.0) ** (16 / 14)
    assert torch.allclose(dyn, ref.build_cos_sin_cache(16, 64, base), atol=1e-6)
    assert torch.equal(ref.build_cos_sin_cache(16, 64, 1e4, None, {"type": "mrope"}), plain)


def test_cpu_tier_restore_after_partial_eviction_keeps_block_ids_unique():
    """A prefix whose tail blocks were evicted to the CPU tier: the surviving GPU hits sit at the head of the free queue, and the
    restore must not hand those very blocks out again."""
    from types import SimpleNamespace
    m = KVCacheManager(num_blocks=31, block_size=16, max_model_len=4096)
    m.enable_cpu_offload(32)
    hasher = make_block_hasher(16)
    a = Request("a", list(range(1, 161)), SamplingParams(max_tokens=1), eos_token_id=0, block_hasher=hasher)
    assert m.allocate_slots(a, 160) is not None
    a.num_computed_tokens = 160
    m.free(a)  # ten cached blocks, tail first in the free queue
    # evict the prefix's last five blocks (they are the oldest free cached blocks) by taking fresh blocks
    other = SimpleNamespace(request_id="o", num_computed_tokens=0, num_tokens=16 * 25, block_hashes=[], sampling_params=None)
    free_before = m.block_pool.get_num_free_blocks()
    taken = m.block_pool.get_new_blocks(free_before - 5)
    assert len(m.offload.index) == 5
    m.block_pool.free_blocks(taken)
    b = Request("b", list(range(1, 162)), SamplingParams(max_tokens=1), eos_token_id=0, block_hasher=hasher)
    hit, n = m.get_computed_blocks(b)
    ids = [x.block_id for x in hit]
    assert n == 160 and len(set(ids)) == 10, ids
    assert [x.block_hash for x in hit] == b.block_hashes[:10]
    _, swap_in = m.offload.take_ops()
    assert sorted(g for _, g in swap_in) == sorted(ids[5:])        # only the evicted half is copied back
    assert not set(g for _, g in swap_in) & set(ids[:5])            # and never into a surviving hit
    assert m.allocate_slots(b, 1, n, hit) is not None
    assert m.get_block_ids("b")[:10] == ids


def test_requests_that_edit_logits_get_no_drafts():
    """Drafts are verified against the temperature-only distribution, so a request with allowed ids, penalties or a random top-k must
    not receive them."""
    from onecat_vllm.config import SpeculativeConfig
    s = make_scheduler(spec=SpeculativeConfig(method="ngram", num_speculative_tokens=2))
    plain = Request("p", [1, 2, 3], SamplingParams(max_tokens=8, temperature=0.0, top_k=5), eos_token_id=0)
    masked = Request("m", [1, 2, 3], SamplingParams(max_tokens=8, temperature=0.0, allowed_token_ids=[4, 5]), eos_token_id=0)
    topk = Request("k", [1, 2, 3], SamplingParams(max_tokens=8, temperature=1.0, top_k=1), eos_token_id=0)
    assert plain.spec_decode_ok and not masked.spec_decode_ok and not topk.spec_decode_ok
    for r in (plain, masked, topk):
        s.add_request(r)
    so = s.schedule()
    s.update_from_output(so, ModelRunnerOutput(req_ids=list(so.num_scheduled_tokens), sampled_token_ids=[[7]] * 3, spec_token_ids=[[8, 9]] * 3))
    assert plain.spec_token_ids == [8, 9] and masked.spec_token_ids == [] and topk.spec_token_ids == []
    s.update_draft_token_ids(["p", "m", "k"], [[1, 1], [1, 1], [1, 1]])
    assert plain.spec_token_ids == [1, 1] and masked.spec_token_ids == [] and topk.spec_token_ids == []


def test_sliding_window_blocks_are_released_while_the_request_runs():
    """All-sliding models: blocks wholly below the window (minus the slack the kernels' key tiles need) go back to the pool; their
    table entries become the placeholder block, so positions keep their indices."""
    m = KVCacheManager(num_blocks=200, block_size=16, max_model_len=8192, enable_caching=False, sliding_window=256)
    r = Request("w", list(range(1, 1025)), SamplingParams(max_tokens=4), eos_token_id=0)
    assert m.allocate_slots(r, 1024) is not None
    r.num_computed_tokens = 1024
    used_before = 200 - m.block_pool.get_num_free_blocks()
    assert m.allocate_slots(r, 1) is not None            # next query sits at position 1024: keys <= 768 are out of its window
    ids = m.get_block_ids("w")
    n_gone = (1024 - 256 + 1 - 128) // 16
    assert ids[:n_gone] == [0] * n_gone and all(i != 0 for i in ids[n_gone:]) and len(ids) == 65
    assert 200 - m.block_pool.get_num_free_blocks() == used_before + 1 - n_gone
    m.free(r)
    assert m.block_pool.get_num_free_blocks() == 199       # everything but the placeholder block is back
    full = KVCacheManager(num_blocks=200, block_size=16, max_model_len=8192, enable_caching=False)
    r2 = Request("f", list(range(1, 1025)), SamplingParams(max_tokens=4), eos_token_id=0)
    full.allocate_slots(r2, 1024)
    r2.num_computed_tokens = 1024
    full.allocate_slots(r2, 1)
    assert 0 not in full.get_block_ids("f")
