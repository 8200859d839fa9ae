"""gRPC endpoint against the CPU engine: streaming deltas, token-id prompts, abort on cancel, tokenizer and health calls."""
import asyncio

import pytest

CFG = dict(architectures=["LlamaForCausalLM"], hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
           num_key_value_heads=2, head_dim=16, vocab_size=300, max_position_embeddings=256)


@pytest.mark.timeout(180)
def test_generate_stream_tokenize_health_and_cancel():
    from onecat_vllm.config import EngineArgs
    from onecat_vllm.engine.async_llm import AsyncLLM
    from onecat_vllm.entrypoints.grpc_server import EngineClient, serve_grpc

    async def main():
        eng = AsyncLLM.from_engine_args(EngineArgs(hf_config=CFG, device="cpu", dtype="float32", max_model_len=256, tokenizer="byte"))
        server, port = await serve_grpc(eng, port=0)
        cli = EngineClient(f"127.0.0.1:{port}")
        try:
            assert (await cli.health())["ok"] is True
            assert (await cli.tokenize("hi", add_special_tokens=False))["token_ids"] == [104, 105]
            ids, texts, last = [], [], None
            async for d in cli.generate(prompt="hello", sampling_params={"temperature": 0.0, "max_tokens": 6, "ignore_eos": True}):
                ids += d["token_ids"]
                texts.append(d["text"])
                last = d
            assert len(ids) == 6 and last["finished"] and last["finish_reason"] == "length" and last["num_prompt_tokens"] == 6
            # the same prompt as token ids gives the same tokens
            ids2 = []
            async for d in cli.generate(prompt_token_ids=[256] + list(b"hello"), sampling_params={"temperature": 0.0, "max_tokens": 6, "ignore_eos": True}):
                ids2 += d["token_ids"]
            assert ids2 == ids
            # a cancelled call aborts its request in the engine
            call = cli.generate(request_id="long", prompt="abc", sampling_params={"temperature": 0.0, "max_tokens": 200, "ignore_eos": True})
            got = 0
            async for d in call:
                got += len(d["token_ids"])
                if got >= 3:
                    call.cancel()
                    break
            for _ in range(100):
                if (await cli.health())["unfinished"] == 0:
                    break
                await asyncio.sleep(0.05)
            assert (await cli.health())["unfinished"] == 0
            assert (await cli.abort("nope")) == {"aborted": False}
            import grpc
            with pytest.raises(grpc.aio.AioRpcError) as e:
                async for _ in cli.generate(sampling_params={"max_tokens": 1}):
                    pass
            assert e.value.code() == grpc.StatusCode.INVALID_ARGUMENT
        finally:
            await cli.close()
            await server.stop(0.5)
            eng.shutdown()

    asyncio.run(main())
