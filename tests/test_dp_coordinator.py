"""The data-parallel coordinator: wave bookkeeping on the bare state machine, and the process with two engine reporters and two
front-end subscribers over ZMQ."""
import time

import pytest

from onecat_vllm.engine.coordinator import CoordinatorState, DPCoordinator, EngineReporter, FrontendSubscriber


def test_wave_state_machine():
    st = CoordinatorState(2)
    assert st.snapshot() == {"counts": [[0, 0], [0, 0]], "wave": 0, "running": False}
    assert st.on_first_req({"wave": 0, "engine": 1}) == {"start_wave": 0, "exclude": 1} and st.running
    assert st.on_first_req({"wave": 0, "engine": 0}) is None                  # already running
    st.on_engine({"engine": 0, "stats": [3, 1]})
    assert st.dirty and st.snapshot()["counts"] == [[3, 1], [0, 0]]
    st.on_engine({"engine": 0, "wave_complete": 0})
    assert st.running                                                            # one replica is still busy
    st.on_engine({"engine": 1, "wave_complete": 0})
    assert not st.running and st.wave == 1
    st.on_engine({"engine": 1, "wave_complete": 0})                              # a late note for the finished wave changes nothing
    assert st.wave == 1 and not st.running
    assert st.on_first_req({"wave": 0, "engine": 0}) == {"start_wave": 1, "exclude": 0}   # raced with the end of wave 0: starts wave 1
    assert st.on_engine({"engine": 1, "start_wave": 1}) is None                 # an engine noticing the same thing adds nothing


def _until(cond, timeout=5.0):
    t0 = time.time()
    while time.time() - t0 < timeout:
        if cond():
            return True
        time.sleep(0.02)
    return False


@pytest.mark.timeout(60)
def test_coordinator_process_links_engines_and_front_ends():
    co = DPCoordinator(2)
    engines = [EngineReporter(i, co.addresses) for i in range(2)]
    fronts = [FrontendSubscriber(co.addresses) for _ in range(2)]
    try:
        time.sleep(0.3)                                                          # SUB sockets join late by nature
        engines[0].report(5, 2)
        engines[1].report(0, 1)
        assert _until(lambda: all(f.counts() == [[5, 2], [0, 1]] for f in fronts))   # both front ends see both engines' load
        fronts[0].request_routed(1)                                              # idle group: this wakes it
        assert _until(lambda: engines[0].poll_start_wave() == 0)
        assert engines[1].poll_start_wave() is None                              # the engine that got the request is not told twice
        engines[1].running = True
        assert _until(lambda: all(f.state["running"] for f in fronts))
        fronts[1].request_routed(0)                                              # running group: no further broadcast
        time.sleep(0.3)
        assert engines[0].poll_start_wave() is None
        for e in engines:
            e.became_idle()
        assert _until(lambda: all((not f.state["running"]) and f.state["wave"] == 1 for f in fronts))
        engines[0].became_busy()                                                 # work that reached an engine directly starts the next wave
        assert _until(lambda: engines[1].poll_start_wave() == 1)
    finally:
        for x in engines + fronts:
            x.close()
        co.close()
    assert not co.proc.is_alive()


@pytest.mark.timeout(600)
def test_engine_replicas_report_to_the_coordinator(monkeypatch):
    """Two CPU replicas with the coordinator switched on: requests complete with the single-engine tokens, the coordinator's table
    reaches the client, and after the work is done the group is idle again in a later wave."""
    import time as _t
    from onecat_vllm import LLM, SamplingParams
    cfg = dict(architectures=["LlamaForCausalLM"], hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
               num_key_value_heads=2, head_dim=16, vocab_size=300, max_position_embeddings=256)
    prompts = [[(7 * i + j) % 290 + 1 for j in range(5 + i)] for i in range(6)]
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    one = LLM(hf_config=cfg, device="cpu", dtype="float32", max_model_len=128)
    ref = [o.outputs[0].token_ids for o in one.generate([{"prompt_token_ids": p} for p in prompts], sp)]
    one.shutdown()
    monkeypatch.setenv("ONECAT_DP_COORDINATOR", "1")
    two = LLM(hf_config=cfg, device="cpu", dtype="float32", max_model_len=128, data_parallel_size=2)
    client = two.llm_engine.engine_core
    assert client.coordinator is not None and client._coord_sub is not None
    seen = []
    orig = client._coord_sub.on_update
    client._coord_sub.on_update = lambda m: (seen.append(m), orig(m))
    got = [o.outputs[0].token_ids for o in two.generate([{"prompt_token_ids": p} for p in prompts], sp)]
    assert got == ref
    assert _until(lambda: bool(seen) and not client._coord_sub.state["running"] and client._coord_sub.state["wave"] >= 1, 10)
    assert any(m["running"] for m in seen)                          # the group was seen running in between
    assert all(len(m["counts"]) == 2 for m in seen)
    proc = client.coordinator.proc
    two.shutdown()
    assert not proc.is_alive()
