"""The native (C++) front end: its tokenizer against Hugging Face `tokenizers` and the Python tekken tokenizer, and the HTTP server
end to end against the CPU engine it starts."""
import base64
import json
import os
import signal
import subprocess
import sys
import time

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TEXTS = ["hello world", "Hello,  world!!  ", " leading space", "tabs\tand\nnewlines\r\n\r\nend", "it's we're I'LL they'D don't", "12345 67 8.9 1,000,000",
         "héllo wörld ✓ — naïve café", "日本語のテキスト と spaces", "emoji 🙂🙃 mix", "a" * 50, "  \n  \n", "x=y+1;//c\n", "snake_case CamelCase kebab-case",
         "Ünïcödé ÀÉÎ õ", "3rd 1st ²³ ½", "trailing   ", " nbsp emspace", "<|special|> in text <|special|>"]

LLAMA3 = r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+"
QWEN2 = r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+"


def _binary():
    sys.path.insert(0, ROOT)
    from onecat_vllm.entrypoints.native_frontend import binary_path
    return binary_path()


def _native_encode(tok_path, texts):
    p = subprocess.run([_binary(), "--tokenizer", tok_path, "--tokenize-stdin"], input="".join(json.dumps(t) + "\n" for t in texts),
                       capture_output=True, text=True, timeout=60)
    assert p.returncode == 0, p.stderr
    return [json.loads(l) for l in p.stdout.splitlines()]


def _train(tmp_path, pattern):
    from tokenizers import Regex, Tokenizer, decoders, models, pre_tokenizers, trainers
    tok = Tokenizer(models.BPE())
    if pattern is None:
        tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=True)
    else:
        tok.pre_tokenizer = pre_tokenizers.Sequence([pre_tokenizers.Split(Regex(pattern), behavior="isolated", invert=False),
                                                     pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False)])
    tok.decoder = decoders.ByteLevel()
    corpus = TEXTS * 3 + ["the quick brown fox jumps over the lazy dog " * 4, "numbers 123 456 7890 and words words words", "über straße façade 東京 東京 東京"]
    tok.train_from_iterator(corpus, trainers.BpeTrainer(vocab_size=600, special_tokens=["<|special|>"], initial_alphabet=pre_tokenizers.ByteLevel.alphabet()))
    d = tmp_path / ("tok_" + str(abs(hash(pattern)) % 10000))
    d.mkdir()
    tok.save(str(d / "tokenizer.json"))
    return tok, str(d)


@pytest.mark.parametrize("pattern", [None, LLAMA3, QWEN2], ids=["gpt2", "llama3", "qwen2"])
def test_tokenizer_matches_hugging_face(tmp_path, pattern):
    hf, path = _train(tmp_path, pattern)
    got = _native_encode(path, TEXTS)
    for text, g in zip(TEXTS, got):
        want = hf.encode(text, add_special_tokens=False).ids
        assert g["ids"] == want, (text, g["pieces"], g["ids"], want)
        assert g["text"] == text


def test_tekken_matches_the_python_tokenizer(tmp_path):
    from onecat_vllm.engine.renderers import TekkenTokenizer
    toks = [bytes([i]) for i in range(256)] + [b"he", b"ll", b"hell", b"hello", b" w", b"or", b" wor", b"\xe6\x97", b"\xe6\x97\xa5"]
    special = ["<unk>", "<s>", "</s>", "[INST]", "[/INST]"]
    d = {"config": {"pattern": r"[^\r\n\p{L}\p{N}]?[\p{L}]+|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n/]*|\s*[\r\n]+|\s+(?!\S)|\s+",
                    "default_vocab_size": len(toks) + len(special), "default_num_special_tokens": len(special), "version": "v7"},
         "vocab": [{"rank": i, "token_bytes": base64.b64encode(b).decode()} for i, b in enumerate(toks)],
         "special_tokens": [{"rank": i, "token_str": s, "is_control": True} for i, s in enumerate(special)]}
    (tmp_path / "tekken.json").write_text(json.dumps(d))
    py = TekkenTokenizer(str(tmp_path / "tekken.json"))
    texts = [t for t in TEXTS if "<|special|>" not in t] + ["[INST]hello world[/INST]"]
    for text, g in zip(texts, _native_encode(str(tmp_path), texts)):
        assert g["ids"] == py.encode(text, add_special_tokens=False), (text, g["pieces"])


def test_unknown_split_pattern_refuses_text_but_decodes(tmp_path):
    hf, path = _train(tmp_path, LLAMA3)
    j = json.loads(open(os.path.join(path, "tokenizer.json")).read())
    j["pre_tokenizer"]["pretokenizers"][0]["pattern"]["Regex"] = r"\w+|\W+"
    open(os.path.join(path, "tokenizer.json"), "w").write(json.dumps(j))
    p = subprocess.run([_binary(), "--tokenizer", path, "--tokenize-stdin"], input='"abc"\n', capture_output=True, text=True, timeout=60)
    assert p.returncode != 0 and "unknown split pattern" in p.stderr


CFG = dict(architectures=["LlamaForCausalLM"], hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
           num_key_value_heads=2, head_dim=16, vocab_size=300, max_position_embeddings=256)


@pytest.mark.timeout(300)
def test_http_server_end_to_end_on_the_cpu_engine():
    import httpx
    from onecat_vllm import LLM, SamplingParams
    from onecat_vllm.entrypoints.native_frontend import command
    from onecat_vllm.executor.multiproc import _free_port
    llm = LLM(hf_config=CFG, device="cpu", dtype="float32", max_model_len=256)
    prompt_ids = [256] + list(b"hello")
    ref = llm.generate([{"prompt_token_ids": prompt_ids}], SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))[0].outputs[0].token_ids
    llm.shutdown()
    port = _free_port()
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    cmd = command(["--hf-config", json.dumps(CFG), "--device", "cpu", "--dtype", "float32", "--max-model-len", "256"], port=port,
                  tokenizer="byte", served_model_name="tiny", handshake_timeout=120)
    proc = subprocess.Popen(cmd, env=env, stderr=subprocess.PIPE, text=True)
    base = f"http://127.0.0.1:{port}"
    try:
        for _ in range(600):
            if proc.poll() is not None:
                raise AssertionError("front end exited: " + proc.stderr.read())
            try:
                if httpx.get(base + "/health", timeout=1).status_code == 200:
                    break
            except Exception:
                time.sleep(0.2)
        assert httpx.get(base + "/v1/models").json()["data"][0]["id"] == "tiny"
        assert httpx.post(base + "/tokenize", json={"prompt": "hi", "add_special_tokens": False}).json()["tokens"] == [104, 105]
        assert httpx.post(base + "/detokenize", json={"tokens": [104, 105]}).json()["prompt"] == "hi"
        body = {"prompt": "hello", "max_tokens": 8, "temperature": 0.0, "ignore_eos": True, "return_token_ids": True}
        r = httpx.post(base + "/v1/completions", json=body, timeout=60).json()
        assert r["choices"][0]["token_ids"] == ref and r["choices"][0]["finish_reason"] == "length"
        assert r["usage"] == {"prompt_tokens": 6, "completion_tokens": 8, "total_tokens": 14}
        r2 = httpx.post(base + "/v1/completions", json=dict(body, prompt=prompt_ids), timeout=60).json()
        assert r2["choices"][0]["token_ids"] == ref
        # streaming: server-sent events whose token ids add up to the same completion; two requests share one connection
        with httpx.Client(timeout=60) as cli:
            for _ in range(2):
                ids, done = [], False
                with cli.stream("POST", base + "/v1/completions", json=dict(body, stream=True)) as resp:
                    assert resp.headers["content-type"].startswith("text/event-stream")
                    for line in resp.iter_lines():
                        if line == "data: [DONE]":
                            done = True
                        elif line.startswith("data: "):
                            ids += json.loads(line[6:])["choices"][0]["token_ids"]
                assert done and ids == ref
        assert httpx.post(base + "/v1/completions", json={"max_tokens": 1}).status_code == 400
        assert httpx.post(base + "/v1/completions", content=b"{not json", headers={"content-type": "application/json"}).status_code == 400
        assert httpx.get(base + "/nope").status_code == 404
    finally:
        proc.send_signal(signal.SIGTERM)   # the exact process this test started; it stops its engine core itself
        try:
            proc.wait(timeout=30)
        except subprocess.TimeoutExpired:
            proc.kill()
    assert proc.returncode == 0
