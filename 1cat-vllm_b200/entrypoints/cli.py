"""Command line: ``python -m onecat_vllm.entrypoints.cli {serve,chat,complete,bench,run-batch,collect-env}``
(reference: vllm/entrypoints/cli/main.py:17, serve.py:44, openai.py, run_batch.py, benchmark/)."""
from __future__ import annotations

import argparse
import json
import sys
import time


def _cmd_serve(argv):
    from onecat_vllm.entrypoints.openai.api_server import make_arg_parser, run_server
    run_server(make_arg_parser().parse_args(argv))


def _http(url: str, body=None, api_key=None, stream=False):
    import httpx
    headers = {"Authorization": f"Bearer {api_key}"} if api_key else {}
    if body is None:
        return httpx.get(url, headers=headers, timeout=600).json()
    if not stream:
        return httpx.post(url, json=body, headers=headers, timeout=600).json()
    return httpx.stream("POST", url, json=body, headers=headers, timeout=600)


def _cmd_complete(argv):
    p = argparse.ArgumentParser("complete")
    p.add_argument("--url", default="http://127.0.0.1:8000/v1")
    p.add_argument("--api-key", default=None)
    p.add_argument("--max-tokens", type=int, default=64)
    p.add_argument("prompt", nargs="?")
    a = p.parse_args(argv)
    model = _http(a.url + "/models", api_key=a.api_key)["data"][0]["id"]
    prompts = [a.prompt] if a.prompt else iter(lambda: input("> "), "")
    for pr in prompts:
        r = _http(a.url + "/completions", {"model": model, "prompt": pr, "max_tokens": a.max_tokens}, a.api_key)
        print(r["choices"][0]["text"])


def _cmd_chat(argv):
    p = argparse.ArgumentParser("chat")
    p.add_argument("--url", default="http://127.0.0.1:8000/v1")
    p.add_argument("--api-key", default=None)
    p.add_argument("--system-prompt", default=None)
    p.add_argument("message", nargs="?")
    a = p.parse_args(argv)
    model = _http(a.url + "/models", api_key=a.api_key)["data"][0]["id"]
    msgs = [{"role": "system", "content": a.system_prompt}] if a.system_prompt else []
    turns = [a.message] if a.message else iter(lambda: input("> "), "")
    for t in turns:
        msgs.append({"role": "user", "content": t})
        r = _http(a.url + "/chat/completions", {"model": model, "messages": msgs}, a.api_key)
        out = r["choices"][0]["message"]["content"]
        msgs.append({"role": "assistant", "content": out})
        print(out)


def _cmd_run_batch(argv):
    """OpenAI batch file format: one JSON request per line with ``custom_id``, ``url`` and ``body``."""
    p = argparse.ArgumentParser("run-batch")
    p.add_argument("-i", "--input-file", required=True)
    p.add_argument("-o", "--output-file", required=True)
    from onecat_vllm.config import EngineArgs
    EngineArgs.add_cli_args(p)
    a = p.parse_args(argv)
    from onecat_vllm import LLM
    from onecat_vllm.entrypoints.openai.protocol import ChatCompletionRequest, CompletionRequest
    ea = EngineArgs.from_cli_args(a)
    llm = LLM(**{k: v for k, v in ea.__dict__.items()})
    tok = llm.get_tokenizer()
    reqs = [json.loads(l) for l in open(a.input_file) if l.strip()]
    prompts, sps = [], []
    for r in reqs:
        if r["url"].endswith("/chat/completions"):
            b = ChatCompletionRequest(**r["body"])
            prompts.append(tok.apply_chat_template([m.model_dump(exclude_none=True) for m in b.messages], tokenize=False, add_generation_prompt=True))
        else:
            b = CompletionRequest(**r["body"])
            prompts.append(b.prompt)
        b.stream = False
        sps.append(b.to_sampling_params(ea.max_model_len or 4096))
    outs = llm.generate(prompts, sps)
    with open(a.output_file, "w") as f:
        for r, o in zip(reqs, outs):
            body = {"choices": [{"index": c.index, "text": c.text, "finish_reason": c.finish_reason} for c in o.outputs],
                    "usage": {"prompt_tokens": len(o.prompt_token_ids), "completion_tokens": sum(len(c.token_ids) for c in o.outputs)}}
            f.write(json.dumps({"id": "batch-" + r["custom_id"], "custom_id": r["custom_id"], "response": {"status_code": 200, "body": body}, "error": None}) + "\n")
    llm.shutdown()


def _cmd_collect_env(argv):
    import platform
    import torch
    info = {"python": sys.version.split()[0], "platform": platform.platform(), "torch": torch.__version__, "cuda": torch.version.cuda,
            "cuda_available": torch.cuda.is_available()}
    if torch.cuda.is_available():
        info["gpus"] = [torch.cuda.get_device_name(i) for i in range(torch.cuda.device_count())]
    from onecat_vllm.platforms import current_platform
    info["platform_summary"] = current_platform().describe()
    try:
        from onecat_vllm.ops import _C  # noqa: F401
        info["extension"] = "built"
    except ImportError as e:
        info["extension"] = f"missing ({e})"
    print(json.dumps(info, indent=1))


def _cmd_bench(argv):
    from onecat_vllm.entrypoints.bench import main as bench_main
    bench_main(argv)


def _cmd_serve_native(argv):
    """The C++ front end (HTTP server + tokenizer) in front of an engine-core process; see entrypoints/native_frontend.py."""
    from onecat_vllm.entrypoints.native_frontend import main as native_main
    native_main(argv)


COMMANDS = {"serve": _cmd_serve, "serve-native": _cmd_serve_native, "chat": _cmd_chat, "complete": _cmd_complete, "bench": _cmd_bench, "run-batch": _cmd_run_batch,
            "collect-env": _cmd_collect_env}


def main(argv=None) -> None:
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv or argv[0] not in COMMANDS:
        print("usage: onecat-vllm {" + ",".join(COMMANDS) + "} ...", file=sys.stderr)
        raise SystemExit(2)
    COMMANDS[argv[0]](argv[1:])


if __name__ == "__main__":
    main()
