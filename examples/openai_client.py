"""Start the OpenAI-compatible server and talk to it: a streamed chat completion and the render-only route.

    python examples/openai_client.py --device cpu
    python examples/openai_client.py --model /path/to/checkpoint
"""
import json
import os
import socket
import subprocess
import sys
import time
import urllib.request

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from _tiny import TINY, parse  # noqa: E402


def _open(url: str, body: dict):
    req = urllib.request.Request(url, data=json.dumps(body).encode(), headers={"Content-Type": "application/json"})
    return urllib.request.urlopen(req, timeout=120)


def post(url: str, body: dict) -> dict:
    return json.loads(_open(url, body).read())


def post_stream(url: str, body: dict):
    for line in _open(url, body):
        line = line.decode().strip()
        if line.startswith("data: ") and line != "data: [DONE]":
            yield json.loads(line[6:])


if __name__ == "__main__":
    args = parse(__doc__)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    cmd = [sys.executable, "-m", "onecat_vllm.entrypoints.cli", "serve", args.model or "dummy", "--device", args.device, "--port", str(port),
           "--served-model-name", "demo", "--max-model-len", "512"]
    if not args.model:
        cmd += ["--hf-config", json.dumps(TINY), "--tokenizer", "byte", "--dtype", "float32" if args.device == "cpu" else "bfloat16"]
    else:
        cmd += ["--tokenizer", args.model]
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    server = subprocess.Popen(cmd, cwd=ROOT, env=env, stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)
    base = f"http://127.0.0.1:{port}"
    try:
        for _ in range(600):
            try:
                if urllib.request.urlopen(base + "/health", timeout=1).status == 200:
                    break
            except OSError:
                time.sleep(0.5)
        msgs = [{"role": "user", "content": "Say hello."}]
        rendered = post(base + "/v1/chat/completions/render", {"model": "demo", "messages": msgs, "max_tokens": 16})
        print("prompt tokens:", len(rendered["token_ids"]))
        text = ""
        for chunk in post_stream(base + "/v1/chat/completions", {"model": "demo", "messages": msgs, "max_tokens": 16, "temperature": 0, "stream": True}):
            text += chunk["choices"][0]["delta"].get("content") or ""
        print("streamed:", repr(text))
    finally:
        server.terminate()
        server.wait(timeout=30)
