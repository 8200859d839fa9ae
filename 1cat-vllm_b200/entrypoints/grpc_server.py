"""gRPC endpoint over the async engine: streaming generation for callers that keep one HTTP/2 connection and many requests on it
(routers, other languages' clients). The service is ``onecat.Engine`` with four methods; messages are msgpack maps, so no generated
stubs are needed on either side (any gRPC client can call the methods with its own msgpack codec):

  Generate  (unary request → stream)   request  {"request_id"?, "prompt"? | "prompt_token_ids"?, "sampling_params"?: {...}, "priority"?}
                                       response {"request_id", "text", "token_ids", "finished", "finish_reason", "num_prompt_tokens",
                                                 "num_cached_tokens"}   (deltas; the last one has finished = true)
  Abort     (unary)                    {"request_id"} → {"aborted": bool}
  Tokenize  (unary)                    {"text", "add_special_tokens"?} → {"token_ids"}
  Health    (unary)                    {} → {"ok": true, "unfinished": n}

A cancelled Generate call aborts its request in the engine. ``serve_grpc`` is what ``cli serve --grpc-port`` runs next to the HTTP
server. (reference: rust/src/server gRPC front end and vllm/entrypoints/grpc_server.py: the same engine-facing operations)"""
from __future__ import annotations

import itertools
from typing import Optional

import grpc
import msgpack

from onecat_vllm.sampling_params import RequestOutputKind, SamplingParams

SERVICE = "onecat.Engine"
_pack = lambda o: msgpack.packb(o, use_bin_type=True)
_unpack = lambda b: msgpack.unpackb(b, raw=False) if b else {}


class EngineService:
    def __init__(self, engine):
        self.engine = engine
        self._ids = itertools.count()

    async def Generate(self, req: dict, context):
        rid = str(req.get("request_id") or f"grpc-{next(self._ids)}")
        spd = dict(req.get("sampling_params") or {})
        try:
            sp = SamplingParams(**spd)
        except (TypeError, ValueError) as e:
            await context.abort(grpc.StatusCode.INVALID_ARGUMENT, f"bad sampling_params: {e}")
        sp.output_kind = RequestOutputKind.DELTA
        if "prompt_token_ids" in req:
            prompt = {"prompt_token_ids": list(req["prompt_token_ids"])}
        elif "prompt" in req:
            prompt = req["prompt"]
        else:
            await context.abort(grpc.StatusCode.INVALID_ARGUMENT, "need prompt or prompt_token_ids")
        try:
            async for out in self.engine.generate(prompt, sp, rid, priority=int(req.get("priority", 0))):
                o = out.outputs[0]
                yield {"request_id": rid, "text": o.text, "token_ids": list(o.token_ids), "finished": bool(out.finished),
                       "finish_reason": o.finish_reason, "num_prompt_tokens": len(out.prompt_token_ids or []),
                       "num_cached_tokens": out.num_cached_tokens}
        except ValueError as e:
            await context.abort(grpc.StatusCode.INVALID_ARGUMENT, str(e))

    async def Abort(self, req: dict, context):
        rid = str(req.get("request_id", ""))
        known = rid in getattr(self.engine.output_processor, "states", {})
        if known:
            await self.engine.abort(rid)
        return {"aborted": known}

    async def Tokenize(self, req: dict, context):
        tok = self.engine.tokenizer
        if tok is None:
            await context.abort(grpc.StatusCode.FAILED_PRECONDITION, "the engine has no tokenizer")
        return {"token_ids": list(tok.encode(req.get("text", ""), add_special_tokens=bool(req.get("add_special_tokens", True))))}

    async def Health(self, req: dict, context):
        return {"ok": True, "unfinished": len(getattr(self.engine.output_processor, "states", {}))}


def _handlers(svc: EngineService):
    unary = lambda f: grpc.unary_unary_rpc_method_handler(f, request_deserializer=_unpack, response_serializer=_pack)
    return grpc.method_handlers_generic_handler(SERVICE, {
        "Generate": grpc.unary_stream_rpc_method_handler(svc.Generate, request_deserializer=_unpack, response_serializer=_pack),
        "Abort": unary(svc.Abort), "Tokenize": unary(svc.Tokenize), "Health": unary(svc.Health)})


async def serve_grpc(engine, host: str = "127.0.0.1", port: int = 50051):
    """Starts the server and returns ``(server, bound_port)``; the caller awaits ``server.wait_for_termination()`` or stops it."""
    server = grpc.aio.server()
    server.add_generic_rpc_handlers((_handlers(EngineService(engine)),))
    bound = server.add_insecure_port(f"{host}:{port}")
    await server.start()
    return server, bound


class EngineClient:
    """Async client for the service above (what a router or a test uses)."""

    def __init__(self, target: str):
        self.channel = grpc.aio.insecure_channel(target)
        m = lambda name, kind: getattr(self.channel, kind)(f"/{SERVICE}/{name}", request_serializer=_pack, response_deserializer=_unpack)
        self._generate = m("Generate", "unary_stream")
        self._abort, self._tokenize, self._health = m("Abort", "unary_unary"), m("Tokenize", "unary_unary"), m("Health", "unary_unary")

    def generate(self, **req):
        return self._generate(req)

    async def abort(self, request_id: str) -> dict:
        return await self._abort({"request_id": request_id})

    async def tokenize(self, text: str, add_special_tokens: bool = True) -> dict:
        return await self._tokenize({"text": text, "add_special_tokens": add_special_tokens})

    async def health(self) -> dict:
        return await self._health({})

    async def close(self) -> None:
        await self.channel.close()
