"""OpenAI-compatible HTTP server (reference: vllm/entrypoints/openai/api_server.py:157 ``build_app``, :665 ``run_server``;
chat logic openai/chat_completion/serving.py; launcher + watchdog entrypoints/launcher.py:26,144).

Routes: ``/v1/chat/completions``, ``/v1/completions``, ``/v1/models``, ``/tokenize``, ``/detokenize``, ``/health``, ``/ping``,
``/version``, ``/metrics`` (Prometheus), ``/load``, ``/server_info``, ``/reset_prefix_cache``, ``/sleep``, ``/wake_up``,
``/is_sleeping``, ``/start_profile``, ``/stop_profile``, ``/collective_rpc``, ``/v1/embeddings``, ``/pooling``, ``/score``,
``/v1/responses``, ``/v1/messages`` (Anthropic), ``/v1/load_lora_adapter``, ``/v1/unload_lora_adapter``.
Streaming uses server-sent events."""
from __future__ import annotations

import argparse
import asyncio
import json
import os
import signal
from typing import AsyncGenerator, Optional

from fastapi import FastAPI, Request
from fastapi.responses import JSONResponse, Response, StreamingResponse

import onecat_vllm
from onecat_vllm import envs
from onecat_vllm.config import EngineArgs
from onecat_vllm.engine.async_llm import AsyncLLM
from onecat_vllm.engine.core import EngineDeadError
from onecat_vllm.entrypoints.openai.protocol import (ChatCompletionRequest, CompletionRequest, DetokenizeRequest, TokenizeRequest,
                                                      error_body, new_id, now)
from onecat_vllm.entrypoints.parsers import get_reasoning_parser, get_tool_parser
from onecat_vllm.logger import init_logger

log = init_logger(__name__)


class ServingState:
    def __init__(self, engine: AsyncLLM, model_name: str, tool_parser: Optional[str], reasoning_parser: Optional[str], api_key: Optional[str]):
        self.engine, self.model_name = engine, model_name
        self.tool_parser_name, self.reasoning_parser_name = tool_parser, reasoning_parser
        get_tool_parser(tool_parser), get_reasoning_parser(reasoning_parser)  # validate early
        self.api_key = api_key
        self.sleeping = False
        self.inflight = 0
        self.loras: dict = {}  # served adapter name -> LoRARequest
        self._next_lora_id = 1
        self.responses: dict = {}   # id -> finished Responses object (kept while ``store`` is true; the 1024 most recent)

    def keep_response(self, obj: dict) -> dict:
        self.responses[obj["id"]] = obj
        while len(self.responses) > 1024:
            self.responses.pop(next(iter(self.responses)))
        return obj

    def register_lora(self, name: str, path: str):
        from onecat_vllm.lora import LoRARequest
        if name in self.loras:
            return self.loras[name]
        self.loras[name] = LoRARequest(name, self._next_lora_id, path)
        self._next_lora_id += 1
        return self.loras[name]

    def lora_for(self, model: Optional[str]):
        """A request whose ``model`` names a registered adapter runs under it (reference: entrypoints/openai/models/serving.py)."""
        return self.loras.get(model) if model else None

    @property
    def max_model_len(self) -> int:
        return self.engine.cfg.model_config.max_model_len


def _sse(obj) -> str:
    return "data: " + (obj if isinstance(obj, str) else json.dumps(obj, ensure_ascii=False)) + "\n\n"


def _usage(n_prompt: int, n_out: int, cached: int = 0) -> dict:
    u = {"prompt_tokens": n_prompt, "completion_tokens": n_out, "total_tokens": n_prompt + n_out}
    if cached:
        u["prompt_tokens_details"] = {"cached_tokens": cached}
    return u


def _lp_chat(tok, logprobs, k: int) -> dict:
    content = []
    for d in logprobs or []:
        items = list(d.items())
        (tid, first) = items[0]
        tops = [{"token": v.decoded_token or str(t), "logprob": v.logprob, "bytes": list((v.decoded_token or "").encode())} for t, v in items[1:k + 1]]
        content.append({"token": first.decoded_token or str(tid), "logprob": first.logprob, "bytes": list((first.decoded_token or "").encode()),
                        "top_logprobs": tops})
    return {"content": content}


# worker methods that /collective_rpc may reach (development mode only); anything else, shutdown and weight loading from a
# pickled payload included, is refused
COLLECTIVE_RPC_METHODS = frozenset({"check_health", "list_loras", "get_kv_cache_specs", "save_sharded_state", "update_weights", "profile"})


def build_app(state: ServingState) -> FastAPI:
    app = FastAPI(title="onecat-vllm", version=onecat_vllm.__version__)
    app.state.serving = state

    # Routes that change or inspect engine state exist only in development mode, and loading adapters at run time needs its own
    # switch (reference: the dev-mode routers of entrypoints/serve/ are registered only under VLLM_SERVER_DEV_MODE, the LoRA
    # routes only under VLLM_ALLOW_RUNTIME_LORA_UPDATING). Without the switch they answer 404 as if they were not registered.
    dev_paths = {"/reset_prefix_cache", "/sleep", "/wake_up", "/is_sleeping", "/pause", "/resume", "/is_paused", "/collective_rpc",
                 "/start_profile", "/stop_profile", "/server_info", "/abort_requests", "/reset_mm_cache", "/reset_encoder_cache", "/get_world_size",
                 "/init_weight_transfer_engine", "/start_weight_update", "/update_weights", "/finish_weight_update"}
    lora_paths = {"/v1/load_lora_adapter", "/v1/unload_lora_adapter"}
    open_paths = {"/health", "/ping", "/version", "/metrics", "/load"}  # probes and scrapers carry no key

    @app.middleware("http")
    async def auth_and_load(request: Request, call_next):
        path = request.url.path
        if (path in dev_paths and not envs.ONECAT_SERVER_DEV_MODE) or (path in lora_paths and not envs.ONECAT_ALLOW_RUNTIME_LORA_UPDATING):
            return JSONResponse(error_body("Not Found", "NotFoundError", 404), status_code=404)
        if state.api_key and path not in open_paths and request.method != "OPTIONS":
            if request.headers.get("authorization") != f"Bearer {state.api_key}":
                return JSONResponse(error_body("invalid API key", "AuthenticationError", 401), status_code=401)
        state.inflight += 1
        try:
            return await call_next(request)
        finally:
            state.inflight -= 1

    @app.exception_handler(EngineDeadError)
    async def dead(_, exc):
        return JSONResponse(error_body(f"engine is dead: {exc}", "InternalServerError", 500), status_code=500)

    # ---- basic routes
    @app.get("/health")
    @app.get("/ping")
    async def health():
        try:
            await state.engine.check_health()
        except EngineDeadError:
            return Response(status_code=503)
        return Response(status_code=200)

    @app.get("/version")
    async def version():
        return {"version": onecat_vllm.__version__}

    @app.get("/v1/models")
    async def models():
        data = [{"id": state.model_name, "object": "model", "created": now(), "owned_by": "onecat-vllm", "max_model_len": state.max_model_len}]
        data += [{"id": n, "object": "model", "created": now(), "owned_by": "onecat-vllm", "parent": state.model_name, "root": r.lora_path}
                 for n, r in state.loras.items()]
        return {"object": "list", "data": data}

    @app.post("/v1/load_lora_adapter")
    async def load_lora(body: dict):
        try:
            req = state.register_lora(body["lora_name"], body["lora_path"])
            await state.engine.add_lora(req)
        except Exception as e:
            state.loras.pop(body.get("lora_name"), None)
            return JSONResponse(error_body(str(e)), status_code=400)
        return Response(content=f"Success: LoRA adapter '{req.lora_name}' added successfully.", status_code=200)

    @app.post("/v1/unload_lora_adapter")
    async def unload_lora(body: dict):
        req = state.loras.pop(body.get("lora_name"), None)
        if req is None:
            return JSONResponse(error_body(f"adapter {body.get('lora_name')!r} is not loaded", "NotFoundError", 404), status_code=404)
        await state.engine.remove_lora(req.lora_int_id)
        return Response(content=f"Success: LoRA adapter '{req.lora_name}' removed successfully.", status_code=200)

    @app.get("/metrics")
    async def metrics():
        import prometheus_client as pc
        return Response(pc.generate_latest(), media_type=pc.CONTENT_TYPE_LATEST)

    @app.get("/load")
    async def load():
        return {"server_load": state.inflight}

    @app.get("/server_info")
    async def server_info():
        c = state.engine.cfg
        return {"model": c.model_config.model, "architecture": c.model_config.architecture, "max_model_len": c.model_config.max_model_len,
                "tensor_parallel_size": c.parallel_config.tensor_parallel_size, "num_gpu_blocks": c.cache_config.num_gpu_blocks,
                "block_size": c.cache_config.block_size, "quantization": c.model_config.quant.method}

    @app.post("/tokenize")
    async def tokenize(req: TokenizeRequest):
        tok = state.engine.tokenizer
        if tok is None:
            return JSONResponse(error_body("the server has no tokenizer"), status_code=400)
        if req.messages is not None:
            text = tok.apply_chat_template([m.model_dump(exclude_none=True) for m in req.messages], tokenize=False, add_generation_prompt=True)
        else:
            text = req.prompt or ""
        ids = list(tok.encode(text, add_special_tokens=req.add_special_tokens))
        return {"tokens": ids, "count": len(ids), "max_model_len": state.max_model_len}

    @app.post("/detokenize")
    async def detokenize(req: DetokenizeRequest):
        tok = state.engine.tokenizer
        if tok is None:
            return JSONResponse(error_body("the server has no tokenizer"), status_code=400)
        return {"prompt": tok.decode(req.tokens)}

    @app.get("/tokenizer_info")
    async def tokenizer_info():
        tok = state.engine.tokenizer
        if tok is None:
            return JSONResponse(error_body("this server runs without a tokenizer"), status_code=400)
        return {"tokenizer_class": type(tok).__name__, "vocab_size": getattr(tok, "vocab_size", None), "bos_token_id": getattr(tok, "bos_token_id", None),
                "eos_token_id": getattr(tok, "eos_token_id", None), "chat_template": getattr(tok, "chat_template", None)}

    @app.get("/get_world_size")
    async def get_world_size(include_dp: bool = True):
        pc = state.engine.cfg.parallel_config
        return {"world_size": pc.world_size * (pc.data_parallel_size if include_dp else 1)}

    # ---- control routes
    @app.post("/abort_requests")
    async def abort_requests(body: dict):
        ids = [str(x) for x in body.get("request_ids", [])]
        for rid in ids:
            await state.engine.abort(rid)
        return {"aborted": ids}

    @app.post("/reset_mm_cache")
    @app.post("/reset_encoder_cache")
    async def reset_mm_cache():
        """Drops cached encoder outputs on every worker (reference: ``/reset_mm_cache``, ``/reset_encoder_cache``)."""
        return {"evicted": await state.engine.reset_mm_cache()}

    # ---- weight updates between rollouts (reference: entrypoints/serve/rlhf/api_router.py:113-170)
    @app.post("/init_weight_transfer_engine")
    async def init_weight_transfer_engine(body: dict):
        info = body.get("init_info")
        if not info or "init_method" not in info or "world_size" not in info:
            return JSONResponse(error_body("init_info needs init_method and world_size (and rank_offset, backend)"), status_code=400)
        await state.engine.collective_rpc("init_weight_transfer_offset", (info["init_method"], int(info.get("rank_offset", 1)), int(info["world_size"]),
                                                                         info.get("backend")))
        return {"message": "Weight transfer initialized"}

    @app.post("/start_weight_update")
    async def start_weight_update(body: Optional[dict] = None):
        await state.engine.pause_generation()
        state.updating_weights = True
        return {"message": "Weight update started"}

    @app.post("/update_weights")
    async def update_weights(body: dict):
        info = body.get("update_info")
        if not info:
            return JSONResponse(error_body("Missing 'update_info' in request body"), status_code=400)
        try:
            if "path" in info:       # a checkpoint directory every worker can read
                n = await state.engine.collective_rpc("update_weights_from_path", (info["path"],))
            elif "tensors" in info:  # names / dtypes / shapes of what the trainer (rank 0 of the transfer group) is broadcasting now
                n = await state.engine.collective_rpc("update_weights_broadcast", (info,))
            else:
                return JSONResponse(error_body("update_info needs 'path' or the broadcast description ('bucket_bytes', 'tensors')"), status_code=400)
        except Exception as e:
            return JSONResponse(error_body(f"weight update failed: {e}"), status_code=400)
        return {"message": "Weights updated", "tensors": n}

    @app.post("/finish_weight_update")
    async def finish_weight_update():
        await state.engine.reset_prefix_cache()      # cached KV belongs to the old weights
        await state.engine.resume_generation()
        state.updating_weights = False
        return {"message": "Weight update finished"}

    @app.post("/reset_prefix_cache")
    async def reset_prefix_cache():
        ok = await state.engine.reset_prefix_cache()
        return Response(status_code=200 if ok else 409)

    @app.post("/sleep")
    async def sleep(level: int = 1):
        await state.engine.sleep(level)
        state.sleeping = True
        return Response(status_code=200)

    @app.post("/pause")
    async def pause():
        """Requests stay queued with their KV until ``/resume`` (used around in-place weight updates)."""
        await state.engine.pause_generation()
        return {"paused": True}

    @app.post("/resume")
    async def resume():
        await state.engine.resume_generation()
        return {"paused": False}

    @app.get("/is_paused")
    async def is_paused():
        return {"is_paused": await state.engine.is_paused()}

    @app.post("/wake_up")
    async def wake_up():
        await state.engine.wake_up()
        state.sleeping = False
        return Response(status_code=200)

    @app.get("/is_sleeping")
    async def is_sleeping():
        return {"is_sleeping": state.sleeping}

    @app.post("/start_profile")
    async def start_profile():
        await state.engine.profile(True)
        return Response(status_code=200)

    @app.post("/stop_profile")
    async def stop_profile():
        await state.engine.profile(False)
        return Response(status_code=200)

    @app.post("/collective_rpc")
    async def collective_rpc(body: dict):
        if body.get("method") not in COLLECTIVE_RPC_METHODS:
            return JSONResponse(error_body(f"method {body.get('method')!r} is not callable through this route"), status_code=400)
        res = await state.engine.collective_rpc(body["method"], body.get("args", []), body.get("kwargs"))
        return {"results": res}

    # ---- pooling: embeddings, raw pooled states, similarity scores (reference: entrypoints/pooling/*/api_router.py)
    def _as_prompts(x):
        if isinstance(x, str) or (isinstance(x, list) and x and isinstance(x[0], int)):
            return [x]
        return list(x)

    async def _pool_many(prompts, pp, prefix: str):
        rid = new_id(prefix)
        prompts = [p if isinstance(p, str) else {"prompt_token_ids": p} for p in prompts]
        return await asyncio.gather(*[state.engine.encode(p, pp, f"{rid}-{i}") for i, p in enumerate(prompts)])

    @app.post("/v1/embeddings")
    async def embeddings(body: dict):
        from onecat_vllm.sampling_params import PoolingParams
        try:
            pp = PoolingParams(task="embed", normalize=body.get("normalize", True), dimensions=body.get("dimensions"),
                               pooling_type=body.get("pooling_type", "last"))
            outs = await _pool_many(_as_prompts(body["input"]), pp, "embd")
        except (ValueError, KeyError) as e:
            return JSONResponse(error_body(str(e)), status_code=400)
        fmt = body.get("encoding_format", "float")
        data = []
        for i, o in enumerate(outs):
            emb = o.outputs.data
            if fmt == "base64":
                import base64
                import struct
                emb = base64.b64encode(struct.pack(f"<{len(emb)}f", *emb)).decode()
            data.append({"index": i, "object": "embedding", "embedding": emb})
        n = sum(len(o.prompt_token_ids) for o in outs)
        return {"id": new_id("embd"), "object": "list", "created": now(), "model": body.get("model") or state.model_name, "data": data,
                "usage": {"prompt_tokens": n, "total_tokens": n}}

    @app.post("/pooling")
    async def pooling(body: dict):
        from onecat_vllm.sampling_params import PoolingParams
        try:
            pp = PoolingParams(task="encode", normalize=bool(body.get("normalize", False)), pooling_type=body.get("pooling_type", "last"))
            outs = await _pool_many(_as_prompts(body["input"]), pp, "pool")
        except (ValueError, KeyError) as e:
            return JSONResponse(error_body(str(e)), status_code=400)
        return {"id": new_id("pool"), "object": "list", "created": now(), "model": state.model_name,
                "data": [{"index": i, "object": "pooling", "data": o.outputs.data} for i, o in enumerate(outs)]}

    @app.post("/classify")
    async def classify(body: dict):
        from onecat_vllm.sampling_params import PoolingParams
        try:
            pp = PoolingParams(task="classify", normalize=False, use_activation=bool(body.get("use_activation", True)))
            outs = await _pool_many(_as_prompts(body["input"]), pp, "classify")
        except (ValueError, KeyError) as e:
            return JSONResponse(error_body(str(e)), status_code=400)
        data = [{"index": i, "label": str(max(range(len(o.outputs.data)), key=o.outputs.data.__getitem__)), "probs": o.outputs.data,
                 "num_classes": len(o.outputs.data)} for i, o in enumerate(outs)]
        n = sum(len(o.prompt_token_ids) for o in outs)
        return {"id": new_id("classify"), "object": "list", "created": now(), "model": state.model_name, "data": data,
                "usage": {"prompt_tokens": n, "total_tokens": n}}

    @app.post("/rerank")
    @app.post("/v1/rerank")
    @app.post("/v2/rerank")
    async def rerank(body: dict):
        """Documents ordered by similarity to the query (reference: entrypoints/pooling/score/ rerank routes, Jina / Cohere shape)."""
        from onecat_vllm.sampling_params import PoolingParams
        try:
            docs = [d if isinstance(d, str) else d.get("text", "") for d in body["documents"]]
            outs = await _pool_many([body["query"]] + docs, PoolingParams(task="embed", normalize=True), "rerank")
        except (ValueError, KeyError) as e:
            return JSONResponse(error_body(str(e)), status_code=400)
        qv = outs[0].outputs.data
        res = [{"index": i, "document": {"text": d}, "relevance_score": sum(x * y for x, y in zip(qv, o.outputs.data))}
               for i, (d, o) in enumerate(zip(docs, outs[1:]))]
        res.sort(key=lambda r: -r["relevance_score"])
        top_n = body.get("top_n") or len(res)
        n = sum(len(o.prompt_token_ids) for o in outs)
        return {"id": new_id("rerank"), "model": state.model_name, "usage": {"total_tokens": n}, "results": res[:top_n]}

    @app.post("/score")
    @app.post("/v1/score")
    async def score(body: dict):
        from onecat_vllm.sampling_params import PoolingParams
        try:
            a, b = _as_prompts(body["text_1"]), _as_prompts(body["text_2"])
            if len(a) == 1:
                a = a * len(b)
            if len(a) != len(b):
                raise ValueError("text_1 and text_2 must be 1:N or N:N")
            mc = state.engine.cfg.model_config
            if mc.num_labels == 1:   # cross-encoder: classify the concatenated pair
                tok = state.engine.tokenizer
                sep = getattr(tok, "sep_token_id", None)
                sep = mc.eos_token_id if sep is None else sep
                enc = lambda x, special=True: list(x) if not isinstance(x, str) else list(tok.encode(x, add_special_tokens=special))
                pairs = [enc(x) + ([sep] if sep is not None else []) + enc(y, False) for x, y in zip(a, b)]
                outs = await _pool_many(pairs, PoolingParams(task="classify", normalize=False), "score")
                return {"id": new_id("score"), "object": "list", "created": now(), "model": state.model_name,
                        "data": [{"index": i, "object": "score", "score": o.outputs.data[0]} for i, o in enumerate(outs)]}
            outs = await _pool_many(a + b, PoolingParams(task="embed", normalize=True), "score")
        except (ValueError, KeyError) as e:
            return JSONResponse(error_body(str(e)), status_code=400)
        ea, eb = outs[: len(a)], outs[len(a):]
        data = [{"index": i, "object": "score", "score": sum(x * y for x, y in zip(p.outputs.data, q.outputs.data))}
                for i, (p, q) in enumerate(zip(ea, eb))]
        return {"id": new_id("score"), "object": "list", "created": now(), "model": state.model_name, "data": data}

    # ---- Responses API and Anthropic Messages API: both are rewritten into a chat completion request and its result is
    # re-shaped (reference: entrypoints/openai/responses/serving.py; entrypoints/anthropic/serving_messages.py)
    def _as_chat(messages: list, body: dict, max_key: str) -> ChatCompletionRequest:
        keep = {k: body[k] for k in ("temperature", "top_p", "top_k", "seed", "stop", "model", "tools", "tool_choice") if body.get(k) is not None}
        if body.get("stop_sequences"):
            keep["stop"] = body["stop_sequences"]
        return ChatCompletionRequest(messages=messages, max_tokens=body.get(max_key), **keep)

    async def _run_chat(creq: ChatCompletionRequest, raw: Request):
        res = await chat(creq, raw)
        if isinstance(res, JSONResponse):
            return None, res
        return res, None

    def _text_of(content) -> str:
        if isinstance(content, str):
            return content
        return "".join(p.get("text", "") for p in content if isinstance(p, dict) and p.get("type") in ("text", "input_text", "output_text"))

    @app.post("/v1/responses")
    async def responses(body: dict, raw: Request):
        msgs = []
        if body.get("instructions"):
            msgs.append({"role": "system", "content": body["instructions"]})
        inp = body.get("input", "")
        if isinstance(inp, str):
            msgs.append({"role": "user", "content": inp})
        else:
            for it in inp:
                if it.get("type", "message") == "message":
                    msgs.append({"role": it.get("role", "user"), "content": _text_of(it.get("content", ""))})
        try:
            creq = _as_chat(msgs, body, "max_output_tokens")
        except Exception as e:
            return JSONResponse(error_body(str(e)), status_code=400)
        if body.get("stream"):
            # the chat stream re-shaped into Responses events: created, output_text deltas, output_text done, completed
            creq.stream = True
            sres = await chat(creq, raw)
            if isinstance(sres, JSONResponse):
                return sres

            async def gen():
                rid, seq, parts = new_id("resp"), 0, []

                def ev(kind: str, data: dict) -> str:
                    nonlocal seq
                    seq += 1
                    return f"event: {kind}\ndata: {json.dumps(dict(data, type=kind, sequence_number=seq))}\n\n"
                head = {"id": rid, "object": "response", "created_at": now(), "model": state.model_name, "status": "in_progress", "output": []}
                yield ev("response.created", {"response": head})
                async for chunk in sres.body_iterator:
                    text = chunk.decode() if isinstance(chunk, (bytes, bytearray)) else chunk
                    for line in text.split("\n"):
                        if not line.startswith("data: ") or line.strip() == "data: [DONE]":
                            continue
                        for ch in json.loads(line[6:]).get("choices", []):
                            piece = (ch.get("delta") or {}).get("content")
                            if piece:
                                parts.append(piece)
                                yield ev("response.output_text.delta", {"output_index": 0, "content_index": 0, "delta": piece})
                full = "".join(parts)
                yield ev("response.output_text.done", {"output_index": 0, "content_index": 0, "text": full})
                done = dict(head, status="completed", output_text=full,
                            output=[{"type": "message", "id": new_id("msg"), "role": "assistant", "status": "completed",
                                     "content": [{"type": "output_text", "text": full, "annotations": []}]}])
                yield ev("response.completed", {"response": done})
            return StreamingResponse(gen(), media_type="text/event-stream")
        res, err = await _run_chat(creq, raw)
        if err is not None:
            return err
        ch = res["choices"][0]
        out = []
        if ch["message"].get("reasoning_content"):
            out.append({"type": "reasoning", "id": new_id("rs"), "summary": [], "content": [{"type": "reasoning_text", "text": ch["message"]["reasoning_content"]}]})
        for tc in ch["message"].get("tool_calls") or []:
            out.append({"type": "function_call", "id": new_id("fc"), "call_id": tc["id"], "name": tc["function"]["name"],
                        "arguments": tc["function"]["arguments"], "status": "completed"})
        if ch["message"].get("content"):
            out.append({"type": "message", "id": new_id("msg"), "role": "assistant", "status": "completed",
                        "content": [{"type": "output_text", "text": ch["message"]["content"], "annotations": []}]})
        u = res["usage"]
        obj = {"id": new_id("resp"), "object": "response", "created_at": now(), "model": res["model"], "status": "completed",
               "incomplete_details": {"reason": "max_output_tokens"} if ch["finish_reason"] == "length" else None, "output": out,
               "output_text": ch["message"].get("content") or "",
               "usage": {"input_tokens": u["prompt_tokens"], "output_tokens": u["completion_tokens"], "total_tokens": u["total_tokens"]}}
        return state.keep_response(obj) if body.get("store", True) else obj

    @app.get("/v1/responses/{response_id}")
    async def get_response(response_id: str):
        """A finished response kept by ``store`` (reference: entrypoints/openai/responses ``retrieve_responses``)."""
        obj = state.responses.get(response_id)
        if obj is None:
            return JSONResponse(error_body(f"response {response_id} not found", "NotFoundError", 404), status_code=404)
        return obj

    @app.post("/v1/responses/{response_id}/cancel")
    async def cancel_response(response_id: str):
        """Responses run to completion inside their request here, so only a stored, finished one can be named: it is returned as it is
        (cancelling a finished response is a no-op in the reference too)."""
        obj = state.responses.get(response_id)
        if obj is None:
            return JSONResponse(error_body(f"response {response_id} not found", "NotFoundError", 404), status_code=404)
        return obj

    @app.post("/v1/messages")
    async def anthropic_messages(body: dict, raw: Request):
        msgs = []
        if body.get("system"):
            msgs.append({"role": "system", "content": _text_of(body["system"])})
        for m in body.get("messages", []):
            msgs.append({"role": m["role"], "content": _text_of(m.get("content", ""))})
        tools = [{"type": "function", "function": {"name": t["name"], "description": t.get("description", ""), "parameters": t.get("input_schema", {})}}
                 for t in body.get("tools") or []]
        b2 = dict(body)
        b2["tools"] = tools or None
        b2.pop("tool_choice", None)
        try:
            creq = _as_chat(msgs, b2, "max_tokens")
        except Exception as e:
            return JSONResponse({"type": "error", "error": {"type": "invalid_request_error", "message": str(e)}}, status_code=400)
        if body.get("stream"):
            # the chat stream re-shaped into Messages events: message_start, one text block of deltas, message_delta, message_stop
            creq.stream = True
            sres = await chat(creq, raw)
            if isinstance(sres, JSONResponse):
                return sres

            def ev(kind: str, data: dict) -> str:
                return f"event: {kind}\ndata: {json.dumps(data)}\n\n"

            async def gen():
                mid, n_out, stop = new_id("msg"), 0, "end_turn"
                yield ev("message_start", {"type": "message_start", "message": {"id": mid, "type": "message", "role": "assistant", "model": state.model_name,
                                                                               "content": [], "stop_reason": None, "usage": {"input_tokens": 0, "output_tokens": 0}}})
                yield ev("content_block_start", {"type": "content_block_start", "index": 0, "content_block": {"type": "text", "text": ""}})
                async for chunk in sres.body_iterator:
                    text = chunk.decode() if isinstance(chunk, (bytes, bytearray)) else chunk
                    for line in text.split("\n"):
                        if not line.startswith("data: ") or line.strip() == "data: [DONE]":
                            continue
                        d = json.loads(line[6:])
                        for ch in d.get("choices", []):
                            piece = (ch.get("delta") or {}).get("content")
                            if piece:
                                n_out += 1
                                yield ev("content_block_delta", {"type": "content_block_delta", "index": 0, "delta": {"type": "text_delta", "text": piece}})
                            if ch.get("finish_reason"):
                                stop = {"stop": "end_turn", "length": "max_tokens", "tool_calls": "tool_use"}.get(ch["finish_reason"], "end_turn")
                yield ev("content_block_stop", {"type": "content_block_stop", "index": 0})
                yield ev("message_delta", {"type": "message_delta", "delta": {"stop_reason": stop, "stop_sequence": None}, "usage": {"output_tokens": n_out}})
                yield ev("message_stop", {"type": "message_stop"})
            return StreamingResponse(gen(), media_type="text/event-stream")
        res, err = await _run_chat(creq, raw)
        if err is not None:
            return err
        ch = res["choices"][0]
        content = []
        if ch["message"].get("content"):
            content.append({"type": "text", "text": ch["message"]["content"]})
        for tc in ch["message"].get("tool_calls") or []:
            content.append({"type": "tool_use", "id": tc["id"], "name": tc["function"]["name"], "input": json.loads(tc["function"]["arguments"] or "{}")})
        stop = {"stop": "end_turn", "length": "max_tokens", "tool_calls": "tool_use"}.get(ch["finish_reason"], "end_turn")
        if ch.get("stop_reason") is not None and isinstance(ch["stop_reason"], str):
            stop = "stop_sequence"
        u = res["usage"]
        return {"id": new_id("msg"), "type": "message", "role": "assistant", "model": res["model"], "content": content, "stop_reason": stop,
                "stop_sequence": ch.get("stop_reason") if stop == "stop_sequence" else None,
                "usage": {"input_tokens": u["prompt_tokens"], "output_tokens": u["completion_tokens"]}}

    @app.post("/v1/messages/count_tokens")
    async def anthropic_count_tokens(body: dict):
        """Prompt length of a Messages request after the chat template (reference: entrypoints/anthropic count_tokens route)."""
        tok = state.engine.tokenizer
        if tok is None:
            return JSONResponse(error_body("the server has no tokenizer"), status_code=400)
        msgs = [{"role": "system", "content": _text_of(body["system"])}] if body.get("system") else []
        msgs += [{"role": m["role"], "content": _text_of(m.get("content", ""))} for m in body.get("messages", [])]
        text = tok.apply_chat_template(msgs, tokenize=False, add_generation_prompt=True)
        return {"input_tokens": len(tok.encode(text, add_special_tokens=False))}

    @app.post("/invocations")
    async def invocations(body: dict, raw: Request):
        """Single entry point that dispatches on the shape of the body (reference: the SageMaker-style ``/invocations`` route)."""
        if "messages" in body:
            return await chat(ChatCompletionRequest(**body), raw)
        if "prompt" in body:
            return await completions(CompletionRequest(**body), raw)
        if "input" in body:
            return await embeddings(body)
        return JSONResponse(error_body("the body must carry messages, prompt or input"), status_code=400)

    # ---- completions
    @app.post("/v1/completions")
    async def completions(req: CompletionRequest, raw: Request):
        prompts = req.prompt
        if isinstance(prompts, str) or (prompts and isinstance(prompts[0], int)):
            prompts = [prompts]
        rid = new_id("cmpl")
        try:
            sp = req.to_sampling_params(state.max_model_len, logprobs=req.logprobs)
            gens = []
            for i, p in enumerate(prompts):
                sp_i = sp.clone()
                gens.append(state.engine.generate(p, sp_i, f"{rid}-{i}", priority=req.priority, lora_request=state.lora_for(req.model)))
        except ValueError as e:
            return JSONResponse(error_body(str(e)), status_code=400)
        model = req.model or state.model_name

        if req.stream:
            async def stream() -> AsyncGenerator[str, None]:
                n_prompt = n_out = 0
                try:
                    for i, g in enumerate(gens):
                        async for out in g:
                            n_prompt = len(out.prompt_token_ids)
                            for c in out.outputs:
                                n_out += len(c.token_ids)
                                yield _sse({"id": rid, "object": "text_completion", "created": now(), "model": model,
                                            "choices": [{"index": i * req.n + c.index, "text": c.text, "logprobs": None,
                                                         "finish_reason": c.finish_reason, "stop_reason": c.stop_reason}]})
                    if req.stream_options and req.stream_options.get("include_usage"):
                        yield _sse({"id": rid, "object": "text_completion", "created": now(), "model": model, "choices": [],
                                    "usage": _usage(n_prompt, n_out)})
                    yield _sse("[DONE]")
                except EngineDeadError as e:
                    yield _sse(error_body(str(e), "InternalServerError", 500))
            return StreamingResponse(stream(), media_type="text/event-stream")

        choices, n_prompt, n_out = [], 0, 0
        try:
            for i, g in enumerate(gens):
                final = None
                async for out in g:
                    final = out
                    if await raw.is_disconnected():
                        await state.engine.abort(f"{rid}-{i}")
                        return Response(status_code=499)
                n_prompt += len(final.prompt_token_ids)
                for c in final.outputs:
                    n_out += len(c.token_ids)
                    text = ((final.prompt or "") + c.text) if req.echo else c.text
                    lp = None
                    if req.logprobs is not None and c.logprobs:
                        lp = {"tokens": [next(iter(d.values())).decoded_token for d in c.logprobs],
                              "token_logprobs": [next(iter(d.values())).logprob for d in c.logprobs],
                              "top_logprobs": [{(v.decoded_token or str(t)): v.logprob for t, v in d.items()} for d in c.logprobs]}
                    choices.append({"index": i * req.n + c.index, "text": text, "logprobs": lp, "finish_reason": c.finish_reason,
                                    "stop_reason": c.stop_reason, "token_ids": c.token_ids if state.engine.tokenizer is None else None})
        except ValueError as e:
            return JSONResponse(error_body(str(e)), status_code=400)
        return {"id": rid, "object": "text_completion", "created": now(), "model": model, "choices": choices, "usage": _usage(n_prompt, n_out)}

    # ---- rendering only: what the engine would be asked to generate from, without generating
    # (reference: entrypoints/serve/render/api_router.py ``/v1/chat/completions/render``, ``/v1/completions/render``)
    def _rendered(prompt, sp) -> dict:
        tok = state.engine.tokenizer
        ids = list(prompt) if isinstance(prompt, (list, tuple)) else (tok.encode(prompt) if tok is not None else None)
        if ids is None:
            raise ValueError("text prompts need a tokenizer")
        return {"token_ids": ids, "prompt": prompt if isinstance(prompt, str) else None,
                "sampling_params": {"max_tokens": sp.max_tokens, "temperature": sp.temperature, "top_p": sp.top_p, "top_k": sp.top_k,
                                    "stop": sp.stop, "seed": sp.seed, "n": sp.n}}

    @app.post("/v1/chat/completions/render")
    async def render_chat_completion(req: ChatCompletionRequest):
        tok = state.engine.tokenizer
        if tok is None:
            return JSONResponse(error_body("chat completions need a tokenizer with a chat template"), status_code=400)
        kw = dict(req.chat_template_kwargs or {})
        if req.tools and req.tool_choice != "none":
            kw["tools"] = req.tools
        try:
            from onecat_vllm.engine.renderers import render_chat
            tools = kw.pop("tools", None)
            prompt = render_chat(tok, [m.model_dump(exclude_none=True) for m in req.messages], architecture=state.engine.cfg.model_config.architecture,
                                 tools=tools, add_generation_prompt=req.add_generation_prompt, **kw)
            if req.max_completion_tokens is not None and req.max_tokens is None:
                req.max_tokens = req.max_completion_tokens
            return _rendered(prompt, req.to_sampling_params(state.max_model_len))
        except Exception as e:
            return JSONResponse(error_body(f"rendering failed: {e}"), status_code=400)

    @app.post("/v1/completions/render")
    async def render_completion(req: CompletionRequest):
        try:
            sp = req.to_sampling_params(state.max_model_len)
            p = req.prompt
            many = isinstance(p, list) and p and isinstance(p[0], (str, list))
            return [_rendered(x, sp) for x in (p if many else [p])]
        except Exception as e:
            return JSONResponse(error_body(f"rendering failed: {e}"), status_code=400)

    # ---- chat completions
    @app.post("/v1/chat/completions")
    async def chat(req: ChatCompletionRequest, raw: Request):
        tok = state.engine.tokenizer
        if tok is None:
            return JSONResponse(error_body("chat completions need a tokenizer with a chat template"), status_code=400)
        msgs = [m.model_dump(exclude_none=True) for m in req.messages]
        kw = dict(req.chat_template_kwargs or {})
        if req.tools and req.tool_choice != "none":
            kw["tools"] = req.tools
        try:
            from onecat_vllm.engine.renderers import render_chat
            tools = kw.pop("tools", None)
            prompt = render_chat(tok, msgs, architecture=state.engine.cfg.model_config.architecture, tools=tools,
                                 add_generation_prompt=req.add_generation_prompt, **kw)
        except Exception as e:
            return JSONResponse(error_body(f"chat template failed: {e}"), status_code=400)
        if req.max_completion_tokens is not None and req.max_tokens is None:
            req.max_tokens = req.max_completion_tokens
        k = (req.top_logprobs or 0) if req.logprobs else None
        rid = new_id("chatcmpl")
        try:
            sp = req.to_sampling_params(state.max_model_len, logprobs=k)
            gen = state.engine.generate(prompt, sp, rid, priority=req.priority, lora_request=state.lora_for(req.model))
        except ValueError as e:
            return JSONResponse(error_body(str(e)), status_code=400)
        model = req.model or state.model_name
        rp = get_reasoning_parser(state.reasoning_parser_name)
        tp = get_tool_parser(state.tool_parser_name) if (req.tools and req.tool_choice != "none") else None

        if req.stream:
            async def stream() -> AsyncGenerator[str, None]:
                def chunk(index, delta, finish=None):
                    return _sse({"id": rid, "object": "chat.completion.chunk", "created": now(), "model": model,
                                 "choices": [{"index": index, "delta": delta, "logprobs": None, "finish_reason": finish}]})
                acc: dict = {}
                sent: dict = {}
                n_prompt = n_out = 0
                try:
                    for i in range(req.n):
                        yield chunk(i, {"role": "assistant", "content": ""})
                    async for out in gen:
                        n_prompt = len(out.prompt_token_ids)
                        for c in out.outputs:
                            n_out += len(c.token_ids)
                            prev = acc.get(c.index, "")
                            cur = prev + c.text
                            acc[c.index] = cur
                            delta: dict = {}
                            if rp is not None:
                                r_d, c_d = rp.stream(prev, cur)
                                visible_prev, visible_cur = rp._split_partial(prev)[1], rp._split_partial(cur)[1]
                            else:
                                r_d, visible_prev, visible_cur = "", prev, cur
                            if r_d:
                                delta["reasoning_content"] = r_d
                            if tp is not None:
                                shown = tp.content_so_far(visible_cur)
                                already = sent.get(c.index, 0)
                                if len(shown) > already:
                                    delta["content"] = shown[already:]
                                    sent[c.index] = len(shown)
                            else:
                                if len(visible_cur) > len(visible_prev):
                                    delta["content"] = visible_cur[len(visible_prev):]
                            finish = c.finish_reason
                            if finish is not None and tp is not None:
                                _, calls = tp.extract(rp.extract(cur)[1] or "" if rp else cur)
                                if calls:
                                    delta["tool_calls"] = [tc.to_openai(j) for j, tc in enumerate(calls)]
                                    finish = "tool_calls"
                            if delta or finish is not None:
                                yield chunk(c.index, delta, finish)
                    if req.stream_options and req.stream_options.get("include_usage"):
                        yield _sse({"id": rid, "object": "chat.completion.chunk", "created": now(), "model": model, "choices": [],
                                    "usage": _usage(n_prompt, n_out)})
                    yield _sse("[DONE]")
                except EngineDeadError as e:
                    yield _sse(error_body(str(e), "InternalServerError", 500))
            return StreamingResponse(stream(), media_type="text/event-stream")

        final = None
        outs_by_index: dict = {}
        async for out in gen:
            final = out
            for c in out.outputs:
                outs_by_index[c.index] = c
        choices, n_out = [], 0
        for idx in sorted(outs_by_index):
            c = outs_by_index[idx]
            n_out += len(c.token_ids)
            reasoning, content = (rp.extract(c.text) if rp is not None else (None, c.text))
            msg: dict = {"role": "assistant", "content": content}
            finish = c.finish_reason
            if reasoning is not None:
                msg["reasoning_content"] = reasoning
            if tp is not None and content:
                content2, calls = tp.extract(content)
                if calls:
                    msg["content"], msg["tool_calls"], finish = content2, [tc.to_openai() for tc in calls], "tool_calls"
            choices.append({"index": idx, "message": msg, "logprobs": _lp_chat(tok, c.logprobs, k or 0) if req.logprobs else None,
                            "finish_reason": finish, "stop_reason": c.stop_reason})
        return {"id": rid, "object": "chat.completion", "created": now(), "model": model, "choices": choices,
                "usage": _usage(len(final.prompt_token_ids), n_out, final.num_cached_tokens)}

    return app


async def _watchdog(state: ServingState, server) -> None:
    """Stop serving when the engine has died (reference: launcher.py:144-166)."""
    while True:
        await asyncio.sleep(2.0)
        if not state.engine.is_running:
            log.error("engine died: shutting the server down")
            server.should_exit = True
            return


def make_arg_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser("onecat-vllm serve")
    p.add_argument("model_tag", nargs="?", default=None)
    p.add_argument("--host", default="127.0.0.1")
    p.add_argument("--port", type=int, default=8000)
    p.add_argument("--grpc-port", type=int, default=None, help="also serve the msgpack-over-gRPC endpoint (entrypoints/grpc_server.py) on this port")
    p.add_argument("--served-model-name", default=None)
    p.add_argument("--api-key", default=envs.ONECAT_API_KEY)
    p.add_argument("--tool-call-parser", default=None)
    p.add_argument("--reasoning-parser", default=None)
    p.add_argument("--enable-auto-tool-choice", action="store_true")
    p.add_argument("--lora-modules", nargs="*", default=[], help="adapters to serve, as name=path")
    EngineArgs.add_cli_args(p)
    return p


def run_server(args: argparse.Namespace) -> None:
    import uvicorn
    if args.model_tag:
        args.model = args.model_tag
    ea = EngineArgs.from_cli_args(args)
    ea.disable_log_stats = False
    if ea.tokenizer is None and os.path.isdir(ea.model):
        ea.tokenizer = ea.model
    engine = AsyncLLM.from_engine_args(ea)
    state = ServingState(engine, args.served_model_name or ea.model, args.tool_call_parser, args.reasoning_parser, args.api_key)
    for item in getattr(args, "lora_modules", []) or []:
        name, _, path = item.partition("=")
        state.register_lora(name, path)
    app = build_app(state)
    config = uvicorn.Config(app, host=args.host, port=args.port, log_level="warning")
    server = uvicorn.Server(config)

    async def main():
        wd = asyncio.create_task(_watchdog(state, server))
        grpc_server = None
        if getattr(args, "grpc_port", None):
            from onecat_vllm.entrypoints.grpc_server import serve_grpc
            grpc_server, bound = await serve_grpc(engine, args.host, args.grpc_port)   # same engine, same event loop
            log.info(f"gRPC endpoint on {args.host}:{bound}")
        try:
            await server.serve()
        finally:
            wd.cancel()
            if grpc_server is not None:
                await grpc_server.stop(1.0)
            engine.shutdown()

    asyncio.run(main())


if __name__ == "__main__":
    run_server(make_arg_parser().parse_args())
