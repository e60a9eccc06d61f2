"""Anthropic Messages dialect (reference: crates/apiserve/src/anthropic.rs:30-33 routes; request:
``max_tokens`` required, ``system`` string or text blocks, ``stop_sequences``, tools rejected;
response ``{id:"msg_…", type:"message", role, content:[{type:"text",text}], model, stop_reason,
usage:{input_tokens, output_tokens}}``; SSE events message_start, content_block_start,
content_block_delta(text_delta), content_block_stop, message_delta, message_stop;
``count_tokens`` is the chars/4 heuristic)."""
from __future__ import annotations

import json
import uuid
from typing import Any, Dict, List

from aiohttp import web

from .bridge import Accounting, Job, read_outcome
from .errors import ApiError, from_exception
from .executor import Executor
from .openai import read_json

_STOP = {"stop": "end_turn", "length": "max_tokens", "stop_sequence": "stop_sequence", "tool_calls": "end_turn"}


def _blocks_text(c) -> str:
    if isinstance(c, str):
        return c
    if isinstance(c, list):
        out = []
        for b in c:
            if not isinstance(b, dict):
                raise ApiError("invalid_request", "content blocks must be objects")
            if b.get("type") == "text":
                out.append(b.get("text", ""))
            elif b.get("type") in ("image", "document", "tool_use", "tool_result"):
                raise ApiError("invalid_request", f"content block type '{b.get('type')}' is not supported")
        return "".join(out)
    raise ApiError("invalid_request", "content must be a string or an array of blocks")


def parse_messages_request(body: Dict[str, Any]) -> Dict[str, Any]:
    if not isinstance(body, dict):
        raise ApiError("invalid_request", "request body must be a JSON object")
    model = body.get("model")
    if not isinstance(model, str) or not model:
        raise ApiError("invalid_request", "'model' is required")
    mt = body.get("max_tokens")
    if not isinstance(mt, int) or isinstance(mt, bool) or mt < 1:
        raise ApiError("invalid_request", "'max_tokens' is required and must be a positive integer")
    msgs = body.get("messages")
    if not isinstance(msgs, list) or not msgs:
        raise ApiError("invalid_request", "'messages' must be a non-empty array")
    if body.get("tools"):
        raise ApiError("invalid_request", "tools are not supported on this endpoint")
    flat: List[Dict[str, str]] = []
    for m in msgs:
        if not isinstance(m, dict) or m.get("role") not in ("user", "assistant"):
            raise ApiError("invalid_request", "each message needs role 'user' or 'assistant'")
        flat.append({"role": m["role"], "content": _blocks_text(m.get("content"))})
    params: Dict[str, Any] = {"messages": json.dumps(flat), "max_new": mt,
                              "temp": float(body.get("temperature", 1.0)), "top_p": float(body.get("top_p", 1.0)),
                              "top_k": int(body.get("top_k", 40)), "seed": 0}
    if body.get("system") is not None:
        params["system"] = _blocks_text(body["system"])
    ss = body.get("stop_sequences")
    if ss is not None:
        if not isinstance(ss, list) or not all(isinstance(s, str) for s in ss):
            raise ApiError("invalid_request", "'stop_sequences' must be an array of strings")
        params["stop"] = json.dumps(ss)
    th = body.get("thinking")
    if isinstance(th, dict):
        params["enable_thinking"] = th.get("type") == "enabled"
    return {"model": model, "stream": bool(body.get("stream", False)), "params": params}


class AnthropicSurface:
    def __init__(self, ex: Executor):
        self.ex = ex
        self.acct = Accounting()

    def routes(self, app: web.Application):
        app.router.add_post("/v1/messages", self.messages)
        app.router.add_post("/v1/messages/count_tokens", self.count_tokens)
        app.router.add_get("/v1/models", self.models)

    async def models(self, req):
        data = [{"type": "model", "id": k, "display_name": k, "created_at": "2026-01-01T00:00:00Z"}
                for k in self.ex.models()]
        return web.json_response({"data": data, "has_more": False, "first_id": data[0]["id"] if data else None,
                                  "last_id": data[-1]["id"] if data else None})

    async def count_tokens(self, req):
        body = await read_json(req)
        if not isinstance(body, dict) or not isinstance(body.get("messages"), list):
            raise ApiError("invalid_request", "'messages' must be an array")
        chars = sum(len(_blocks_text(m.get("content"))) for m in body["messages"] if isinstance(m, dict))
        if body.get("system") is not None:
            chars += len(_blocks_text(body["system"]))
        return web.json_response({"input_tokens": max(1, (chars + 3) // 4)})

    async def messages(self, req):
        pr = parse_messages_request(await read_json(req))
        model = pr["model"]
        m = self.ex.get(model)
        if m is None:
            raise ApiError("model_not_found", f"model: {model}")
        if not m.manifest().is_chat():
            raise ApiError("invalid_request", f"model '{model}' is not a chat model")
        mid = "msg_" + uuid.uuid4().hex[:24]
        job = Job(self.ex, model, "generate", pr["params"])
        if not pr["stream"]:
            try:
                async for _ in job.events():
                    pass
                r = read_outcome(await job.result())
            except BaseException as e:
                job.abort()
                self.acct.add(None)
                if type(e).__name__ == "CancelledError":
                    raise
                raise from_exception(e)
            self.acct.add(r)
            return web.json_response({
                "id": mid, "type": "message", "role": "assistant", "content": [{"type": "text", "text": r.text}],
                "model": model, "stop_reason": _STOP.get(r.finish_reason, "end_turn"), "stop_sequence": None,
                "usage": {"input_tokens": r.prompt_tokens, "output_tokens": r.completion_tokens}})
        resp = web.StreamResponse(status=200, headers={"Content-Type": "text/event-stream", "Cache-Control": "no-cache"})
        await resp.prepare(req)

        async def send(event, obj):
            await resp.write(f"event: {event}\ndata: {json.dumps(obj, separators=(',', ':'))}\n\n".encode())
        try:
            await send("message_start", {"type": "message_start", "message": {
                "id": mid, "type": "message", "role": "assistant", "content": [], "model": model,
                "stop_reason": None, "stop_sequence": None, "usage": {"input_tokens": 0, "output_tokens": 0}}})
            await send("content_block_start", {"type": "content_block_start", "index": 0,
                                               "content_block": {"type": "text", "text": ""}})
            async for p in job.events():
                if p.kind == "token":
                    await send("content_block_delta", {"type": "content_block_delta", "index": 0,
                                                       "delta": {"type": "text_delta", "text": p.text}})
            r = read_outcome(await job.result())
            await send("content_block_stop", {"type": "content_block_stop", "index": 0})
            await send("message_delta", {"type": "message_delta",
                                         "delta": {"stop_reason": _STOP.get(r.finish_reason, "end_turn"), "stop_sequence": None},
                                         "usage": {"input_tokens": r.prompt_tokens, "output_tokens": r.completion_tokens}})
            await send("message_stop", {"type": "message_stop"})
            self.acct.add(r)
        except (ConnectionResetError, ConnectionError):
            job.abort()
            self.acct.add(None)
            return resp
        except BaseException as e:
            job.abort()
            self.acct.add(None)
            if type(e).__name__ == "CancelledError":
                raise
            await send("error", from_exception(e).body("anthropic"))
        await resp.write_eof()
        return resp
