"""Engine core in its own process: wire codec round trip, sync client through LLMEngine, asyncio streaming, death detection."""
import asyncio

import pytest
import torch

from onecat_vllm.config import EngineArgs
from onecat_vllm.engine import serial
from onecat_vllm.sampling_params import RequestOutputKind, SamplingParams

CFG = dict(architectures=["LlamaForCausalLM"], hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
           num_key_value_heads=2, head_dim=16, vocab_size=300, max_position_embeddings=256)


def test_serial_roundtrip_with_oob_buffers():
    big = torch.arange(1000, dtype=torch.float32).reshape(10, 100)
    msg = {"a": [1, 2, {"t": big, "s": torch.tensor([1, 2], dtype=torch.int32)}], "b": torch.ones(300, dtype=torch.bfloat16), "c": {3, 1}}
    frames = serial.encode(msg)
    assert len(frames) == 3  # body + two out-of-band buffers (the small tensor is inline)
    back = serial.decode([bytes(f) for f in frames])
    assert torch.equal(back["a"][2]["t"], big) and back["a"][2]["s"].tolist() == [1, 2]
    assert back["b"].dtype == torch.bfloat16 and float(back["b"].float().sum()) == 300.0 and back["c"] == {1, 3}


@pytest.mark.timeout(180)
def test_sync_mp_client_matches_inproc():
    from onecat_vllm.engine.llm_engine import LLMEngine
    args = EngineArgs(hf_config=CFG, device="cpu", dtype="float32", max_model_len=128)
    prompts = [[5, 6, 7, 8, 9], list(range(20, 60))]
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True, output_kind=RequestOutputKind.FINAL_ONLY)
    res = {}
    for mp_mode in (False, True):
        eng = LLMEngine(args.create_engine_config(), multiprocess=mp_mode)
        for i, p in enumerate(prompts):
            eng.add_request(str(i), p, sp)
        outs = {}
        while eng.has_unfinished_requests():
            for o in eng.step():
                if o.finished:
                    outs[o.request_id] = o.outputs[0].token_ids
        if mp_mode:
            assert eng.reset_prefix_cache() in (True, False)
        eng.shutdown()
        res[mp_mode] = outs
    assert res[False] == res[True] and len(res[True]) == 2


@pytest.mark.timeout(180)
def test_async_llm_streams_and_detects_death():
    from onecat_vllm.engine.async_llm import AsyncLLM
    from onecat_vllm.engine.core import EngineDeadError
    args = EngineArgs(hf_config=CFG, device="cpu", dtype="float32", max_model_len=128, disable_log_stats=True)

    async def main():
        eng = AsyncLLM.from_engine_args(args)
        sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True, output_kind=RequestOutputKind.DELTA)

        async def run(rid, p):
            toks = []
            async for o in eng.generate(p, sp, rid):
                toks.extend(o.outputs[0].token_ids)
            return toks

        a, b = await asyncio.gather(run("a", [1, 2, 3]), run("b", list(range(30))))
        assert len(a) == 6 and len(b) == 6
        # host-side failure: terminate the engine process we started; pending and new requests must raise, not hang
        eng.engine_core.proc.terminate()
        eng.engine_core.proc.join(5)
        await asyncio.sleep(0.5)
        with pytest.raises(EngineDeadError):
            await asyncio.wait_for(run("c", [4, 5, 6]), 20)
        eng.shutdown()

    asyncio.run(main())


@pytest.mark.timeout(600)
def test_data_parallel_replicas_balance_and_match_single():
    """Two engine-core replicas behind one client: every request completes with the single-engine tokens, both replicas
    get work, aborts reach the owning replica, utility calls fan out to all replicas."""
    from onecat_vllm import LLM, SamplingParams
    cfg = dict(architectures=["LlamaForCausalLM"], hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
               num_key_value_heads=2, head_dim=16, vocab_size=300, max_position_embeddings=256)
    prompts = [[(7 * i + j) % 290 + 1 for j in range(5 + i)] for i in range(8)]
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    one = LLM(hf_config=cfg, device="cpu", dtype="float32", max_model_len=128)
    ref = [o.outputs[0].token_ids for o in one.generate([{"prompt_token_ids": p} for p in prompts], sp)]
    one.shutdown()
    two = LLM(hf_config=cfg, device="cpu", dtype="float32", max_model_len=128, data_parallel_size=2)
    client = two.llm_engine.engine_core
    assert client.num_engines == 2
    sent = []
    orig = client._route
    client._route = lambda req: (lambda e: (sent.append(e), e)[1])(orig(req))
    got = [o.outputs[0].token_ids for o in two.generate([{"prompt_token_ids": p} for p in prompts], sp)]
    assert got == ref
    assert len(set(sent)) == 2 and abs(sent.count(sent[0]) - len(sent) / 2) <= 1  # both replicas used, evenly
    assert client._inflight == [0, 0] and not client._owner
    assert two.reset_prefix_cache() == [True, True]
    two.shutdown()


@pytest.mark.timeout(300)
def test_forward_error_kills_the_engine_cleanly():
    """A model forward that starts raising (host-side fault injection) surfaces as an error on that step and as ``EngineDeadError``
    on every later call, in-process; through the engine-core process the client reports the dead engine instead of hanging
    (reference test model: tests/v1/shutdown/test_forward_error.py)."""
    from onecat_vllm import LLM, SamplingParams
    from onecat_vllm.engine.core import EngineDeadError
    cfg = dict(architectures=["LlamaForCausalLM"], hidden_size=64, intermediate_size=128, num_hidden_layers=1, num_attention_heads=4,
               num_key_value_heads=2, head_dim=16, vocab_size=300, max_position_embeddings=256)
    llm = LLM(hf_config=cfg, device="cpu", dtype="float32", max_model_len=128)
    runner = llm.llm_engine.engine_core.core.executor.worker.runner
    calls = {"n": 0}
    orig = runner.model.forward

    def boom(*a, **k):
        calls["n"] += 1
        if calls["n"] > 3:
            raise RuntimeError("injected forward failure")
        return orig(*a, **k)

    runner.model.forward = boom
    with pytest.raises(RuntimeError, match="injected"):
        llm.generate([{"prompt_token_ids": [1, 2, 3]}], SamplingParams(max_tokens=20, ignore_eos=True))
    with pytest.raises(EngineDeadError):
        llm.llm_engine.engine_core.core.step()
    llm.shutdown()
