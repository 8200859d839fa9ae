"""OpenAI-compatible server on CPU with the byte tokenizer: routes, streaming, stop strings, tool/reasoning parsers, metrics."""
import json
import os

import pytest

from onecat_vllm.entrypoints.parsers import DeepSeekV3ToolParser, HermesToolParser, Qwen3CoderToolParser, ReasoningParser

CFG = dict(architectures=["LlamaForCausalLM"], hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
           num_key_value_heads=2, head_dim=16, vocab_size=258, max_position_embeddings=512, eos_token_id=257)


def test_reasoning_parser_full_and_streaming():
    rp = ReasoningParser()
    assert rp.extract("<think>plan</think>answer") == ("plan", "answer")
    assert rp.extract("no tags") == (None, "no tags")
    assert ReasoningParser(True).extract("still thinking") == ("still thinking", None)
    text = "<think>abc</think>xyz"
    r = c = ""
    for i in range(1, len(text) + 1):
        dr, dc = rp.stream(text[: i - 1], text[:i])
        r, c = r + dr, c + dc
    assert (r, c) == ("abc", "xyz")


def test_tool_parsers():
    t = 'I will call.<tool_call>\n{"name": "get_weather", "arguments": {"city": "Paris"}}\n</tool_call>'
    content, calls = HermesToolParser().extract(t)
    assert content == "I will call." and calls[0].name == "get_weather" and json.loads(calls[0].arguments) == {"city": "Paris"}
    assert HermesToolParser().content_so_far("hello <tool_c") == "hello "
    q = "<tool_call>\n<function=add>\n<parameter=a>\n1\n</parameter>\n<parameter=b>\ntwo\n</parameter>\n</function>\n</tool_call>"
    content, calls = Qwen3CoderToolParser().extract(q)
    assert content is None and calls[0].name == "add" and json.loads(calls[0].arguments) == {"a": 1, "b": "two"}
    d = '<｜tool▁calls▁begin｜><｜tool▁call▁begin｜>function<｜tool▁sep｜>f\n```json\n{"x": 1}\n```<｜tool▁call▁end｜><｜tool▁calls▁end｜>'
    _, calls = DeepSeekV3ToolParser().extract(d)
    assert calls[0].name == "f" and json.loads(calls[0].arguments) == {"x": 1}
    assert HermesToolParser().extract("plain")[1] == []


def test_tagged_invoke_and_wrapped_pythonic_tool_parsers():
    from onecat_vllm.entrypoints.parsers import get_tool_parser
    c, calls = get_tool_parser("longcat").extract('hi <longcat_tool_call>{"name": "f", "arguments": {"a": 1}}</longcat_tool_call>')
    assert c == "hi" and calls[0].name == "f" and calls[0].arguments == '{"a": 1}'
    c, calls = get_tool_parser("minimax_m2").extract('ok\n<minimax:tool_call>\n<invoke name="get_weather">\n<parameter name="city">Paris</parameter>\n'
                                                     '<parameter name="days">3</parameter>\n</invoke>\n</minimax:tool_call>')
    assert c == "ok" and calls[0].name == "get_weather" and calls[0].arguments == '{"city": "Paris", "days": 3}'
    c, calls = get_tool_parser("lfm2").extract('<|tool_call_start|>[get_weather(location="Paris")]<|tool_call_end|>Checking.')
    assert c == "Checking." and calls[0].arguments == '{"location": "Paris"}'
    assert get_tool_parser("lfm2").extract("no call")[1] == [] and get_tool_parser("ernie45").extract('<tool_call>{"name": "g", "arguments": {}}</tool_call>')[1][0].name == "g"


def test_parser_manager_and_channel_reasoning():
    from onecat_vllm.entrypoints.parsers import ParserManager, get_reasoning_parser
    r, c, calls = ParserManager("qwen3", "hermes").parse('<think>plan</think>ok <tool_call>{"name": "f", "arguments": {"a": 1}}</tool_call>')
    assert r == "plan" and c == "ok" and calls[0].name == "f" and calls[0].arguments == '{"a": 1}'
    assert ParserManager(None, None).parse("x") == (None, "x", [])
    g = get_reasoning_parser("gptoss")
    assert g.extract("<|channel|>analysis<|message|>thinking<|end|><|start|>assistant<|channel|>final<|message|>Answer.") == ("thinking", "Answer.")
    assert g.stream("<|channel|>analysis<|message|>thin", "<|channel|>analysis<|message|>thinking<|en") == ("king", "")
    assert get_reasoning_parser("identity").extract("abc") == (None, "abc")
    g4 = get_reasoning_parser("gemma4")
    assert g4.extract("<|channel>thought\nlet me see<channel|>4.") == ("let me see", "4.") and g4.extract("plain") == (None, "plain")
    prev, deltas = "", []
    for cur in ("<|chan", "<|channel>tho", "<|channel>thought\nlet", "<|channel>thought\nlet me<channel|>An", "<|channel>thought\nlet me<channel|>Answer"):
        deltas.append(g4.stream(prev, cur))
        prev = cur
    assert "".join(d[0] for d in deltas) == "let me" and "".join(d[1] for d in deltas) == "Answer"
    assert get_reasoning_parser("seedoss").extract("<seed:think>a</seed:think>b") == ("a", "b")
    assert get_reasoning_parser("cohere_command").extract("<|START_THINKING|>a<|END_THINKING|>b") == ("a", "b")


@pytest.fixture(scope="module")
def client():
    from fastapi.testclient import TestClient
    from onecat_vllm.config import EngineArgs
    from onecat_vllm.engine.async_llm import AsyncLLM
    from onecat_vllm.entrypoints.openai.api_server import ServingState, build_app
    eng = AsyncLLM.from_engine_args(EngineArgs(hf_config=CFG, device="cpu", dtype="float32", max_model_len=256, tokenizer="byte", disable_log_stats=False))
    app = build_app(ServingState(eng, "tiny", "hermes", "qwen3", None))
    old = {k: os.environ.get(k) for k in ("ONECAT_SERVER_DEV_MODE", "ONECAT_ALLOW_RUNTIME_LORA_UPDATING")}
    os.environ["ONECAT_SERVER_DEV_MODE"] = os.environ["ONECAT_ALLOW_RUNTIME_LORA_UPDATING"] = "1"
    with TestClient(app) as c:
        yield c
    for k, v in old.items():
        os.environ.pop(k, None) if v is None else os.environ.__setitem__(k, v)
    eng.shutdown()


@pytest.mark.timeout(300)
def test_control_routes_are_closed_by_default_and_keyed(client, monkeypatch):
    """State-changing routes exist only in development mode; with an API key every route except probes and metrics needs it."""
    from onecat_vllm.entrypoints.openai.api_server import ServingState, build_app
    from fastapi.testclient import TestClient
    monkeypatch.delenv("ONECAT_SERVER_DEV_MODE")
    monkeypatch.delenv("ONECAT_ALLOW_RUNTIME_LORA_UPDATING")
    for path in ("/sleep", "/wake_up", "/pause", "/resume", "/reset_prefix_cache", "/start_profile", "/stop_profile"):
        assert client.post(path).status_code == 404, path
    assert client.post("/collective_rpc", json={"method": "shutdown"}).status_code == 404
    assert client.post("/v1/load_lora_adapter", json={"lora_name": "x", "lora_path": "/nowhere"}).status_code == 404
    monkeypatch.setenv("ONECAT_SERVER_DEV_MODE", "1")
    assert client.post("/collective_rpc", json={"method": "shutdown"}).status_code == 400          # not on the allow-list
    assert client.post("/collective_rpc", json={"method": "update_weights_ipc", "args": ["x"]}).status_code == 400
    assert client.post("/collective_rpc", json={"method": "check_health"}).json()["results"] == [True]
    keyed = build_app(ServingState(client.app.state.serving.engine, "tiny", "hermes", "qwen3", "sekret"))
    with TestClient(keyed) as kc:
        assert kc.get("/health").status_code == 200 and kc.get("/metrics").status_code == 200
        for method, path in (("post", "/pause"), ("post", "/tokenize"), ("get", "/v1/models"), ("post", "/collective_rpc"), ("post", "/sleep")):
            assert getattr(kc, method)(path).status_code == 401, path
        assert kc.get("/v1/models", headers={"authorization": "Bearer sekret"}).status_code == 200
        # (the engine's sockets live on the first client's event loop, so this second app is only asked for engine-free routes)
        assert kc.get("/is_sleeping", headers={"authorization": "Bearer sekret"}).json()["is_sleeping"] is False


@pytest.mark.timeout(300)
def test_server_routes(client):
    assert client.get("/health").status_code == 200
    assert client.get("/v1/models").json()["data"][0]["id"] == "tiny"
    assert client.get("/version").json()["version"]
    tk = client.post("/tokenize", json={"prompt": "hi"}).json()
    assert tk["count"] == 3 and client.post("/detokenize", json={"tokens": tk["tokens"]}).json()["prompt"] == "hi"
    r = client.post("/v1/completions", json={"prompt": "hello", "max_tokens": 5, "temperature": 0, "ignore_eos": True}).json()
    assert r["usage"]["completion_tokens"] == 5 and r["choices"][0]["finish_reason"] == "length"
    r2 = client.post("/v1/completions", json={"prompt": [72, 105], "max_tokens": 4, "temperature": 0, "ignore_eos": True, "n": 1, "logprobs": 2}).json()
    assert len(r2["choices"][0]["logprobs"]["token_logprobs"]) == 4
    bad = client.post("/v1/completions", json={"prompt": "x", "max_tokens": 0})
    assert bad.status_code == 400 and "error" in bad.json()
    c = client.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "hey"}], "max_tokens": 6, "temperature": 0, "ignore_eos": True}).json()
    assert c["choices"][0]["message"]["role"] == "assistant" and c["usage"]["completion_tokens"] == 6
    assert client.post("/reset_prefix_cache").status_code in (200, 409)
    m = client.get("/metrics").text
    assert "vllm:generation_tokens_total" in m and "vllm:time_to_first_token_seconds" in m
    for series in ("vllm:prompt_tokens_total", "vllm:request_prompt_tokens_bucket", "vllm:request_generation_tokens_bucket",
                   "vllm:request_time_per_output_token_seconds_bucket", "vllm:request_decode_time_seconds_bucket",
                   "vllm:iteration_tokens_total_bucket", 'finished_reason="length"'):
        assert series in m, series
    assert client.get("/server_info").json()["block_size"] == 16
    inv = client.post("/invocations", json={"prompt": "abc", "max_tokens": 3, "temperature": 0, "ignore_eos": True}).json()
    assert inv["usage"]["completion_tokens"] == 3
    inv = client.post("/invocations", json={"messages": [{"role": "user", "content": "hey"}], "max_tokens": 2, "temperature": 0, "ignore_eos": True}).json()
    assert inv["choices"][0]["message"]["role"] == "assistant"
    assert client.post("/invocations", json={"nothing": 1}).status_code == 400
    tr = client.post("/v1/completions", json={"prompt": "abcdefghij", "max_tokens": 1, "temperature": 0, "truncate_prompt_tokens": 4}).json()
    assert tr["usage"]["prompt_tokens"] == 4
    gc = client.post("/v1/completions", json={"prompt": "pick: ", "max_tokens": 8, "temperature": 0, "guided_choice": ["yes", "no"]}).json()
    assert gc["choices"][0]["text"] in ("yes", "no")
    assert client.post("/pause").json() == {"paused": True} and client.get("/is_paused").json()["is_paused"] is True
    assert client.post("/resume").json() == {"paused": False} and client.get("/is_paused").json()["is_paused"] is False
    assert client.post("/v1/completions", json={"prompt": "abc", "max_tokens": 2, "temperature": 0, "ignore_eos": True}).json()["usage"]["completion_tokens"] == 2
    n = client.post("/v1/messages/count_tokens", json={"system": "be brief", "messages": [{"role": "user", "content": "hello"}]}).json()["input_tokens"]
    assert n > len("hello")


@pytest.mark.timeout(300)
def test_server_streaming(client):
    with client.stream("POST", "/v1/completions", json={"prompt": "abc", "max_tokens": 6, "temperature": 0, "ignore_eos": True, "stream": True,
                                                        "stream_options": {"include_usage": True}}) as resp:
        lines = [l for l in resp.iter_lines() if l.startswith("data: ")]
    assert lines[-1] == "data: [DONE]"
    usage = json.loads(lines[-2][6:])["usage"]
    assert usage["completion_tokens"] == 6
    with client.stream("POST", "/v1/chat/completions", json={"messages": [{"role": "user", "content": "q"}], "max_tokens": 5, "temperature": 0,
                                                             "ignore_eos": True, "stream": True}) as resp:
        chunks = [json.loads(l[6:]) for l in resp.iter_lines() if l.startswith("data: ") and l != "data: [DONE]"]
    assert chunks[0]["choices"][0]["delta"]["role"] == "assistant"
    assert chunks[-1]["choices"][0]["finish_reason"] == "length"


@pytest.mark.timeout(300)
def test_pooling_routes(client):
    r = client.post("/v1/embeddings", json={"input": ["hello world", "hello world", "something else entirely"]}).json()
    e = [d["embedding"] for d in r["data"]]
    assert len(e) == 3 and len(e[0]) == 64 and r["usage"]["prompt_tokens"] > 0
    assert abs(sum(x * x for x in e[0]) - 1.0) < 1e-4
    assert max(abs(x - y) for x, y in zip(e[0], e[1])) < 1e-5
    assert max(abs(x - y) for x, y in zip(e[0], e[2])) > 1e-3
    r8 = client.post("/v1/embeddings", json={"input": "hello world", "dimensions": 8, "encoding_format": "base64"}).json()
    import base64
    assert len(base64.b64decode(r8["data"][0]["embedding"])) == 8 * 4
    p = client.post("/pooling", json={"input": "abc", "pooling_type": "mean"}).json()
    assert len(p["data"][0]["data"]) == 64
    s = client.post("/score", json={"text_1": "hello world", "text_2": ["hello world", "zzz"]}).json()
    assert abs(s["data"][0]["score"] - 1.0) < 1e-4 and s["data"][1]["score"] < 0.9999
    assert client.post("/v1/embeddings", json={"input": "x", "pooling_type": "bogus"}).status_code == 400
    rr = client.post("/v1/rerank", json={"query": "hello world", "documents": ["zzz qqq", "hello world", {"text": "hello"}], "top_n": 2}).json()
    assert len(rr["results"]) == 2 and rr["results"][0]["index"] == 1 and rr["results"][0]["relevance_score"] > 0.999
    assert rr["results"][0]["relevance_score"] >= rr["results"][1]["relevance_score"]
    assert client.post("/classify", json={"input": "x"}).status_code == 400   # a generative checkpoint has no score head


def test_more_tool_and_reasoning_parsers():
    from onecat_vllm.entrypoints.parsers import TOOL_PARSERS, get_reasoning_parser, get_tool_parser
    assert len(TOOL_PARSERS) >= 20
    one = lambda name, text: get_tool_parser(name).extract(text)
    c, calls = one("mistral", 'ok [TOOL_CALLS] [{"name": "f", "arguments": {"a": 1}}, {"name": "g", "arguments": {}}]')
    assert c == "ok" and [x.name for x in calls] == ["f", "g"] and json.loads(calls[0].arguments) == {"a": 1}
    c, calls = one("llama3_json", '<|python_tag|>{"name": "f", "parameters": {"x": "y"}}; {"name": "h", "parameters": {}}')
    assert c is None and [x.name for x in calls] == ["f", "h"] and json.loads(calls[0].arguments) == {"x": "y"}
    assert one("llama3_json", "just text")[1] == []
    c, calls = one("pythonic", '[get_weather(city="Paris", days=3), ping()]')
    assert [x.name for x in calls] == ["get_weather", "ping"] and json.loads(calls[0].arguments) == {"city": "Paris", "days": 3}
    assert one("pythonic", "[1, 2]")[1] == []
    k = 'pre<|tool_calls_section_begin|><|tool_call_begin|>functions.search:0<|tool_call_argument_begin|>{"q": "x"}<|tool_call_end|><|tool_calls_section_end|>'
    c, calls = one("kimi_k2", k)
    assert c == "pre" and calls[0].name == "search" and json.loads(calls[0].arguments) == {"q": "x"}
    g = "<tool_call>lookup\n<arg_key>id</arg_key>\n<arg_value>7</arg_value>\n<arg_key>s</arg_key>\n<arg_value>abc</arg_value>\n</tool_call>"
    c, calls = one("glm45", g)
    assert calls[0].name == "lookup" and json.loads(calls[0].arguments) == {"id": 7, "s": "abc"}
    c, calls = one("deepseek_v31", 'x<｜tool▁calls▁begin｜><｜tool▁call▁begin｜>f<｜tool▁sep｜>{"a": 2}<｜tool▁call▁end｜><｜tool▁calls▁end｜>')
    assert c == "x" and calls[0].name == "f" and json.loads(calls[0].arguments) == {"a": 2}
    c, calls = one("jamba", '<tool_calls>[{"name": "f", "arguments": {"a": 1}}]</tool_calls>')
    assert calls[0].name == "f"
    c, calls = one("internlm", 'hi<|action_start|><|plugin|>\n{"name": "f", "parameters": {"a": 1}}<|action_end|>')
    assert c == "hi" and json.loads(calls[0].arguments) == {"a": 1}
    c, calls = one("minimax", '<tool_calls>\n{"name": "a", "arguments": {}}\n{"name": "b", "arguments": {"z": 0}}\n</tool_calls>')
    assert [x.name for x in calls] == ["a", "b"]
    c, calls = one("phi4_mini_json", 'functools[{"name": "f", "arguments": {"q": 1}}]')
    assert calls[0].name == "f"
    assert get_reasoning_parser("mistral").extract("[THINK]plan[/THINK]done") == ("plan", "done")
    assert get_reasoning_parser("seed_oss").extract("<seed:think>a</seed:think>b") == ("a", "b")
    assert get_reasoning_parser("granite").extract("Here is my thought process: think. Here is my response: answer") == ("think.", "answer")
    assert get_reasoning_parser("granite").extract("plain") == (None, "plain")
    rp = get_reasoning_parser("mistral")
    text, r, cc = "[THINK]ab[/THINK]xy", "", ""
    for i in range(1, len(text) + 1):
        dr, dc = rp.stream(text[: i - 1], text[:i])
        r, cc = r + dr, cc + dc
    assert (r, cc) == ("ab", "xy")


@pytest.mark.timeout(300)
def test_responses_and_anthropic_messages_routes(client):
    r = client.post("/v1/responses", json={"input": "hello", "instructions": "be brief", "max_output_tokens": 6, "temperature": 0}).json()
    assert r["object"] == "response" and r["status"] == "completed" and r["usage"]["output_tokens"] <= 6
    assert isinstance(r["output_text"], str) and all(o["type"] in ("message", "reasoning", "function_call") for o in r["output"])
    r2 = client.post("/v1/responses", json={"input": [{"role": "user", "content": [{"type": "input_text", "text": "hi"}]}], "max_output_tokens": 4}).json()
    assert r2["usage"]["input_tokens"] > 0
    m = client.post("/v1/messages", json={"model": "tiny", "max_tokens": 5, "system": "s", "temperature": 0,
                                          "messages": [{"role": "user", "content": [{"type": "text", "text": "hello"}]}]}).json()
    assert m["type"] == "message" and m["role"] == "assistant" and m["stop_reason"] in ("end_turn", "max_tokens", "stop_sequence", "tool_use")
    assert m["usage"]["output_tokens"] <= 5
    kinds = []
    with client.stream("POST", "/v1/responses", json={"input": "x", "stream": True, "max_output_tokens": 3, "temperature": 0}) as resp:
        for line in resp.iter_lines():
            if line.startswith("event: "):
                kinds.append(line[7:])
    assert kinds[0] == "response.created" and kinds[-2:] == ["response.output_text.done", "response.completed"]
    kinds = []
    with client.stream("POST", "/v1/messages", json={"model": "tiny", "max_tokens": 4, "temperature": 0, "stream": True,
                                                     "messages": [{"role": "user", "content": "hello"}]}) as resp:
        for line in resp.iter_lines():
            if line.startswith("event: "):
                kinds.append(line[7:])
    assert kinds[0] == "message_start" and kinds[1] == "content_block_start" and kinds[-3:] == ["content_block_stop", "message_delta", "message_stop"]


@pytest.mark.timeout(300)
def test_serve_subprocess_health_completion_stream_and_shutdown(tmp_path):
    """The real thing: ``cli serve`` in its own process on a checkpoint directory, waited for on /health, driven over HTTP
    (completion, streamed chat, metrics) and stopped with SIGTERM (reference test model: tests/utils.py ``RemoteOpenAIServer``)."""
    import json
    import os
    import signal
    import socket
    import subprocess
    import sys
    import time
    import httpx
    import torch
    from onecat_vllm.config import ModelConfig
    from onecat_vllm.loader.weights import dummy_init, save_pretrained
    from onecat_vllm.models import build_model
    m = build_model(ModelConfig.from_hf_dict(CFG, dtype=torch.float32), "cpu")
    dummy_init(m, 0)
    save_pretrained(m, CFG, str(tmp_path))
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, PYTHONPATH=root + os.pathsep + os.environ.get("PYTHONPATH", ""))
    proc = subprocess.Popen([sys.executable, "-m", "onecat_vllm.entrypoints.cli", "serve", str(tmp_path), "--device", "cpu", "--dtype", "float32",
                             "--tokenizer", "byte", "--max-model-len", "256", "--port", str(port), "--served-model-name", "tiny"],
                            cwd=root, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    base = f"http://127.0.0.1:{port}"
    try:
        ok = False
        for _ in range(240):
            if proc.poll() is not None:
                break
            try:
                if httpx.get(base + "/health", timeout=1.0).status_code == 200:
                    ok = True
                    break
            except httpx.HTTPError:
                pass
            time.sleep(0.5)
        assert ok, "server did not become healthy:\n" + (proc.stdout.read().decode(errors="replace")[-3000:] if proc.poll() is not None else "")
        r = httpx.post(base + "/v1/completions", json={"model": "tiny", "prompt": "hello", "max_tokens": 5, "temperature": 0}, timeout=60).json()
        assert r["usage"]["completion_tokens"] == 5 and r["choices"][0]["finish_reason"] == "length"
        chunks = []
        with httpx.stream("POST", base + "/v1/chat/completions", timeout=60,
                          json={"model": "tiny", "messages": [{"role": "user", "content": "hi"}], "max_tokens": 4, "stream": True}) as resp:
            for line in resp.iter_lines():
                if line.startswith("data: ") and line != "data: [DONE]":
                    chunks.append(json.loads(line[6:]))
        assert chunks and chunks[-1]["choices"][0]["finish_reason"] in ("length", "stop")
        assert "onecat" in httpx.get(base + "/metrics", timeout=10).text or "vllm" in httpx.get(base + "/metrics", timeout=10).text
    finally:
        proc.send_signal(signal.SIGTERM)
        try:
            proc.wait(timeout=30)
        except subprocess.TimeoutExpired:
            proc.kill()
            proc.wait(timeout=10)
    assert proc.returncode is not None


@pytest.mark.timeout(300)
def test_cli_run_batch_bench_and_collect_env(tmp_path, capsys):
    """The offline commands: an OpenAI batch file through ``run-batch``, ``bench throughput / latency / startup`` and ``collect-env``."""
    import json
    import torch
    from onecat_vllm.config import ModelConfig
    from onecat_vllm.entrypoints.cli import COMMANDS
    from onecat_vllm.loader.weights import dummy_init, save_pretrained
    from onecat_vllm.models import build_model
    ck = tmp_path / "ck"
    m = build_model(ModelConfig.from_hf_dict(CFG, dtype=torch.float32), "cpu")
    dummy_init(m, 0)
    save_pretrained(m, CFG, str(ck))
    common = [str(ck), "--device", "cpu", "--dtype", "float32", "--tokenizer", "byte", "--max-model-len", "256"]
    inp, outp = tmp_path / "in.jsonl", tmp_path / "out.jsonl"
    inp.write_text("\n".join(json.dumps(r) for r in [
        {"custom_id": "a", "method": "POST", "url": "/v1/completions", "body": {"model": "m", "prompt": "hello", "max_tokens": 4, "temperature": 0}},
        {"custom_id": "b", "method": "POST", "url": "/v1/completions", "body": {"model": "m", "prompt": "world!", "max_tokens": 3, "temperature": 0}}]))
    COMMANDS["run-batch"](["-i", str(inp), "-o", str(outp), "--model", *common])
    rows = [json.loads(l) for l in outp.read_text().splitlines()]
    assert [r["custom_id"] for r in rows] == ["a", "b"] and rows[0]["response"]["body"]["usage"]["completion_tokens"] == 4
    capsys.readouterr()
    for mode, key in (("throughput", "output_tokens_per_s"), ("latency", "avg_latency_s"), ("startup", "engine_init_s")):
        COMMANDS["bench"]([mode, "--model", *common, "--input-len", "16", "--output-len", "4", "--num-prompts", "3", "--batch-size", "2",
                           "--num-iters", "1", "--num-iters-warmup", "0"])
        res = _last_json(capsys.readouterr().out)
        assert res[key] > 0, (mode, res)
    COMMANDS["collect-env"]([])
    assert "torch" in _last_json(capsys.readouterr().out)


def _last_json(text: str) -> dict:
    """The pretty-printed JSON object that ends the captured output (log lines may precede it)."""
    import json
    lines = text.splitlines()
    start = max(i for i, l in enumerate(lines) if l == "{")
    return json.loads("\n".join(lines[start:]))


def test_remaining_tool_call_formats():
    """One sample per output format of the model families added after the first thirty parser names."""
    from onecat_vllm.entrypoints.parsers import TOOL_PARSERS, get_tool_parser
    cases = {
        "apertus": ('I will check. <|tools_prefix|>[{"get_weather": {"city": "Paris"}}]<|tools_suffix|>', "get_weather", {"city": "Paris"}, "I will check."),
        "deepseek_v32": ('ok <｜DSML｜function_calls>\n<｜DSML｜invoke name="get_weather">\n<｜DSML｜parameter name="location" string="true">Hangzhou</｜DSML｜parameter>\n'
                         '<｜DSML｜parameter name="days" string="false">3</｜DSML｜parameter>\n</｜DSML｜invoke>\n</｜DSML｜function_calls>', "get_weather",
                         {"location": "Hangzhou", "days": 3}, "ok"),
        "deepseek_v4": ('<｜DSML｜tool_calls><｜DSML｜invoke name="f"><｜DSML｜parameter name="x" string="false">[1, 2]</｜DSML｜parameter></｜DSML｜invoke></｜DSML｜tool_calls>',
                        "f", {"x": [1, 2]}, None),
        "functiongemma": ('<start_function_call>call:set_timer{minutes:5,label:<escape>tea, green<escape>}<end_function_call>', "set_timer",
                          {"minutes": 5, "label": "tea, green"}, None),
        "gemma4": ('sure <|tool_call>call:lookup{q:<|"|>cats<|"|>,n:2}<tool_call|>', "lookup", {"q": "cats", "n": 2}, "sure"),
        "gigachat3": ('thinking<|message_sep|>function call<|role_sep|>\n{"name": "sum", "arguments": {"a": 1, "b": 2}}', "sum", {"a": 1, "b": 2}, "thinking"),
        "hy_v3": ('<tool_calls><tool_call>get_time<tool_sep><arg_key>tz</arg_key><arg_value>UTC</arg_value></tool_call></tool_calls>', "get_time", {"tz": "UTC"}, None),
        "minicpm5xml": ('<think>hm</think>Let me see <function name="search"><param name="q"><![CDATA[a<b]]></param><param name="k">3</param></function>', "search",
                        {"q": "a<b", "k": 3}, "Let me see"),
        "openai": ('<|channel|>analysis<|message|>need weather<|end|><|start|>assistant<|channel|>commentary to=functions.get_weather <|constrain|>json<|message|>'
                   '{"city": "Oslo"}<|call|>', "get_weather", {"city": "Oslo"}, None),
        "poolside_v1": ('<tool_call>run\n<arg_key>cmd</arg_key>\n<arg_value>ls</arg_value>\n</tool_call>', "run", {"cmd": "ls"}, None),
        "step3": ('x<｜tool_calls_begin｜><｜tool_call_begin｜>function<｜tool_sep｜><steptml:invoke name="add"><steptml:parameter name="a">1</steptml:parameter>'
                  '<steptml:parameter name="b">two</steptml:parameter></steptml:invoke><｜tool_call_end｜><｜tool_calls_end｜>', "add", {"a": 1, "b": "two"}, "x"),
        "step3p5": ('<tool_call>\n<function=f>\n<parameter=x>\n1\n</parameter>\n</function>\n</tool_call>', "f", {"x": 1}, None),
        "cohere_command": ('<|START_RESPONSE|>one moment<|END_RESPONSE|><|START_ACTION|>[{"tool_call_id": "0", "tool_name": "search", "parameters": {"q": "x"}}]<|END_ACTION|>',
                           "search", {"q": "x"}, "one moment"),
        "granite4": ('<tool_call>{"name": "f", "arguments": {"a": 1}}</tool_call>', "f", {"a": 1}, None),
    }
    for name, (text, fn, args, content) in cases.items():
        c, calls = get_tool_parser(name).extract(text)
        assert len(calls) == 1 and calls[0].name == fn and json.loads(calls[0].arguments) == args, (name, calls)
        assert c == content, (name, c)
        assert get_tool_parser(name).extract("plain answer") == ("plain answer", [])
    assert len(TOOL_PARSERS) >= 46


@pytest.mark.timeout(300)
def test_render_routes_return_the_prompt_the_engine_would_see(client):
    r = client.post("/v1/chat/completions/render", json={"model": "tiny", "messages": [{"role": "user", "content": "hi"}], "max_tokens": 5, "temperature": 0.3})
    assert r.status_code == 200, r.text
    body = r.json()
    assert body["prompt"].endswith("<|assistant|>") and "hi" in body["prompt"]
    assert body["token_ids"][0] == 256 and bytes(t for t in body["token_ids"] if t < 256).decode() == body["prompt"]
    assert body["sampling_params"]["max_tokens"] == 5 and abs(body["sampling_params"]["temperature"] - 0.3) < 1e-6
    r = client.post("/v1/completions/render", json={"model": "tiny", "prompt": ["ab", "c"], "max_tokens": 4})
    assert r.status_code == 200, r.text
    a, b = r.json()
    assert a["prompt"] == "ab" and a["token_ids"][-2:] == [97, 98] and b["token_ids"][-1] == 99
    r = client.post("/v1/completions/render", json={"model": "tiny", "prompt": [1, 2, 3], "max_tokens": 4})
    assert r.status_code == 200 and r.json()[0]["token_ids"] == [1, 2, 3] and r.json()[0]["prompt"] is None
    # the same messages through the generating route consume exactly the rendered prompt
    g = client.post("/v1/chat/completions", json={"model": "tiny", "messages": [{"role": "user", "content": "hi"}], "max_tokens": 2, "temperature": 0})
    assert g.status_code == 200 and g.json()["usage"]["prompt_tokens"] == len(body["token_ids"])


@pytest.mark.timeout(300)
def test_stored_responses_and_small_info_routes(client):
    r = client.post("/v1/responses", json={"model": "tiny", "input": "hi", "max_output_tokens": 3, "temperature": 0})
    assert r.status_code == 200, r.text
    rid = r.json()["id"]
    got = client.get(f"/v1/responses/{rid}")
    assert got.status_code == 200 and got.json() == r.json()
    assert client.post(f"/v1/responses/{rid}/cancel").json()["id"] == rid
    assert client.get("/v1/responses/resp_nope").status_code == 404
    r2 = client.post("/v1/responses", json={"model": "tiny", "input": "hi", "max_output_tokens": 3, "temperature": 0, "store": False})
    assert client.get(f"/v1/responses/{r2.json()['id']}").status_code == 404
    info = client.get("/tokenizer_info").json()
    assert info["tokenizer_class"] == "ByteTokenizer" and info["vocab_size"] == 258
    assert client.get("/get_world_size").json() == {"world_size": 1}
    assert client.post("/abort_requests", json={"request_ids": ["nothing-by-this-name"]}).status_code == 200
    assert client.post("/reset_mm_cache").json() == {"evicted": 0} and client.post("/reset_encoder_cache").status_code == 200


def test_encoder_cache_reset_evicts_only_unreferenced_entries():
    from types import SimpleNamespace
    from onecat_vllm.core.encoder_cache_manager import EncoderCacheManager
    from onecat_vllm.multimodal import MultiModalFeature
    m = EncoderCacheManager(10)
    f = lambda h, n: MultiModalFeature("image", h, 0, n, "embeds")
    a = SimpleNamespace(request_id="a", mm_features=[f("x", 4)])
    b = SimpleNamespace(request_id="b", mm_features=[f("y", 3)])
    for r in (a, b):
        assert m.can_allocate(r, 0, 100)
        m.allocate(r, 0)
    m.free(a)                                            # x is cached but nobody uses it; y is in use
    assert m.reset() == 1 and m.get_freed_mm_hashes() == ["x"]
    assert m.num_free_slots == 7 and m.num_freeable_slots == 7 and "y" in m.cached and "x" not in m.cached


@pytest.mark.timeout(300)
def test_weight_update_routes_load_a_checkpoint_in_place(client, tmp_path):
    import torch
    from safetensors.torch import save_file
    body = {"model": "tiny", "prompt": [5, 6, 7], "max_tokens": 6, "temperature": 0}
    before = client.post("/v1/completions", json=body).json()["choices"][0]["text"]
    save_file({"model.norm.weight": torch.linspace(-1.0, 2.0, 64)}, str(tmp_path / "model.safetensors"))
    assert client.post("/start_weight_update", json={}).status_code == 200
    assert client.get("/is_paused").json()["is_paused"] is True
    assert client.post("/update_weights", json={}).status_code == 400
    r = client.post("/update_weights", json={"update_info": {"path": str(tmp_path)}})
    assert r.status_code == 200 and r.json()["tensors"] == [1], r.text
    assert client.post("/finish_weight_update").status_code == 200
    assert client.get("/is_paused").json()["is_paused"] is False
    after = client.post("/v1/completions", json=body).json()["choices"][0]["text"]
    assert after != before
    assert client.post("/init_weight_transfer_engine", json={"init_info": {}}).status_code == 400
