"""OpenAI-compatible dialect (reference: crates/apiserve/src/openai.rs — routes :32-40, request
parsing :293-369 and :376-460, non-stream response :574-606, streamed deltas :652-676 and
:993-1108; crates/apiserve/src/models.rs:26-92 model listing).  OpenRouter reuses these handlers
with ``native=True`` (extra ``top_k``/``seed`` pass-through and ``context_length`` in listings)."""
from __future__ import annotations

import json
import uuid
from typing import Any, Dict, List, Optional

from aiohttp import web

from .bridge import Accounting, ChatResult, Job, read_outcome
from .errors import ApiError, from_exception
from .executor import Executor

CREATED = 1767225600
MAX_TOOLS, MAX_TOOLS_BYTES, MAX_TOOL_NAME = 128, 256 * 1024, 64


def _content_text(c) -> str:
    if c is None:
        return ""
    if isinstance(c, str):
        return c
    if isinstance(c, list):
        return "".join(p.get("text", "") for p in c if isinstance(p, dict) and p.get("type", "text") == "text")
    raise ApiError("invalid_request", "message content must be a string or an array of content parts")


def parse_chat_request(body: Dict[str, Any], native: bool = False) -> Dict[str, Any]:
    """Validated request -> ``{"model", "stream", "include_usage", "params"}``; ``params`` is the
    ``generate`` action's parameter map."""
    if not isinstance(body, dict):
        raise ApiError("invalid_request", "request body must be a JSON object")
    model = body.get("model")
    if not isinstance(model, str) or not model:
        raise ApiError("invalid_request", "'model' is required")
    msgs = body.get("messages")
    if not isinstance(msgs, list) or not msgs:
        raise ApiError("invalid_request", "'messages' must be a non-empty array")
    n = body.get("n", 1)
    if n not in (None, 1):
        raise ApiError("invalid_request", "only n=1 is supported")
    flat: List[Dict[str, str]] = []
    for m in msgs:
        if not isinstance(m, dict) or "role" not in m:
            raise ApiError("invalid_request", "each message needs a 'role'")
        role = m["role"]
        role = "system" if role in ("system", "developer") else role if role in ("assistant", "tool") else "user"
        text = _content_text(m.get("content"))
        if role == "assistant" and m.get("tool_calls"):
            for tc in m["tool_calls"]:
                fn = tc.get("function", {})
                text += f'\n<tool_call>\n{{"name": "{fn.get("name", "")}", "arguments": {fn.get("arguments", "{}")}}}\n</tool_call>'
        flat.append({"role": role, "content": text})
    max_new = body.get("max_completion_tokens", body.get("max_tokens"))
    if max_new is None:
        max_new = 1024
    if not isinstance(max_new, int) or isinstance(max_new, bool) or max_new < 1:
        raise ApiError("invalid_request", "'max_tokens' must be a positive integer")

    def num(name, default, lo=None, hi=None):
        v = body.get(name, default)
        if v is None:
            v = default
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ApiError("invalid_request", f"'{name}' must be a number")
        if lo is not None and v < lo or hi is not None and v > hi:
            raise ApiError("invalid_request", f"'{name}' is out of range")
        return v
    params: Dict[str, Any] = {
        "messages": json.dumps(flat), "max_new": max_new,
        "temp": float(num("temperature", 1.0, 0.0, 2.0)), "top_p": float(num("top_p", 1.0, 0.0, 1.0)),
        "top_k": int(num("top_k", 40, 0)), "seed": int(num("seed", 0)),
    }
    stop = body.get("stop")
    if stop is not None:
        if isinstance(stop, str):
            stop = [stop]
        if not isinstance(stop, list) or not all(isinstance(s, str) for s in stop):
            raise ApiError("invalid_request", "'stop' must be a string or an array of strings")
        params["stop"] = json.dumps(stop)
    tools = body.get("tools")
    if tools is not None:
        if not isinstance(tools, list) or len(tools) > MAX_TOOLS:
            raise ApiError("invalid_request", f"'tools' must be an array of at most {MAX_TOOLS} entries")
        raw = json.dumps(tools)
        if len(raw) > MAX_TOOLS_BYTES:
            raise ApiError("invalid_request", "'tools' is too large")
        for t in tools:
            name = (t.get("function") or {}).get("name") if isinstance(t, dict) else None
            if not isinstance(name, str) or not name or len(name) > MAX_TOOL_NAME:
                raise ApiError("invalid_request", "each tool needs a function name of at most 64 characters")
        if tools:
            params["tools"] = raw
    tc = body.get("tool_choice")
    if tc is not None:
        if isinstance(tc, str):
            if tc not in ("auto", "none", "required"):
                raise ApiError("invalid_request", "'tool_choice' must be auto, none, required or a function object")
            params["tool_choice"] = tc
        elif isinstance(tc, dict) and isinstance((tc.get("function") or {}).get("name"), str):
            params["tool_choice"] = json.dumps(tc)
        else:
            raise ApiError("invalid_request", "'tool_choice' must be auto, none, required or a function object")
    ctk = body.get("chat_template_kwargs")
    if isinstance(ctk, dict) and isinstance(ctk.get("enable_thinking"), bool):
        params["enable_thinking"] = ctk["enable_thinking"]
    so = body.get("stream_options") or {}
    return {"model": model, "stream": bool(body.get("stream", False)),
            "include_usage": bool(so.get("include_usage", False)), "params": params}


def _usage(r: ChatResult) -> Dict[str, int]:
    return {"prompt_tokens": r.prompt_tokens, "completion_tokens": r.completion_tokens,
            "total_tokens": r.prompt_tokens + r.completion_tokens}


def _finish(reason: str) -> str:
    return {"stop_sequence": "stop"}.get(reason, reason if reason in ("stop", "length", "tool_calls") else "stop")


def _tool_calls_json(calls) -> List[Dict]:
    return [{"id": c.get("id") or f"call_{i}", "type": "function",
             "function": {"name": c["name"], "arguments": c["arguments"] if isinstance(c["arguments"], str)
                          else json.dumps(c["arguments"])}} for i, c in enumerate(calls)]


def chat_response(rid: str, model: str, r: ChatResult) -> Dict:
    msg: Dict[str, Any] = {"role": "assistant", "content": r.text if (r.text or not r.tool_calls) else None,
                           "refusal": None}
    if r.reasoning_content:
        msg["reasoning_content"] = r.reasoning_content
    if r.tool_calls:
        msg["tool_calls"] = _tool_calls_json(r.tool_calls)
    return {"id": rid, "object": "chat.completion", "created": CREATED, "model": model,
            "choices": [{"index": 0, "message": msg, "finish_reason": _finish(r.finish_reason), "logprobs": None}],
            "usage": _usage(r)}


class OpenAiSurface:
    def __init__(self, ex: Executor, native: bool = False, owned_by: str = "brain"):
        self.ex, self.native, self.owned_by = ex, native, owned_by
        self.acct = Accounting()

    def routes(self, app: web.Application):
        for pre in ("", "/v1"):
            app.router.add_post(pre + "/chat/completions", self.chat)
            app.router.add_post(pre + "/embeddings", self.embeddings)
            app.router.add_post(pre + "/images/generations", self.images)
            app.router.add_get(pre + "/models", self.models)
            app.router.add_get(pre + "/models/{id:.+}", self.model)

    # ---- models
    def _model_obj(self, mid: str, m) -> Dict:
        o = {"id": mid, "object": "model", "created": CREATED, "owned_by": self.owned_by}
        ctx = m.context_length()
        if ctx:
            o["context_length"] = ctx
        return o

    async def models(self, req):
        return web.json_response({"object": "list", "data": [self._model_obj(k, m) for k, m in self.ex.models().items()]})

    async def model(self, req):
        mid = req.match_info["id"]
        m = self.ex.get(mid)
        if m is None:
            raise ApiError("model_not_found", f"The model '{mid}' does not exist.")
        return web.json_response(self._model_obj(mid, m))

    # ---- chat
    async def chat(self, req: web.Request):
        body = await read_json(req)
        pr = parse_chat_request(body, self.native)
        model = pr["model"]
        m = self.ex.get(model)
        if m is None:
            raise ApiError("model_not_found", f"The model '{model}' does not exist.")
        if not m.manifest().is_chat():
            raise ApiError("invalid_request", f"The model '{model}' is not a chat model.")
        rid = "chatcmpl-" + uuid.uuid4().hex
        job = Job(self.ex, model, "generate", pr["params"])
        if not pr["stream"]:
            try:
                async for _ in job.events():
                    pass
                r = read_outcome(await job.result())
            except BaseException as e:
                job.abort()
                self.acct.add(None)
                if isinstance(e, (KeyboardInterrupt, SystemExit)) or type(e).__name__ == "CancelledError":
                    raise
                raise from_exception(e)
            self.acct.add(r)
            return web.json_response(chat_response(rid, model, r))
        return await self._stream(req, rid, model, job, pr["include_usage"])

    async def _stream(self, req, rid, model, job: Job, include_usage: bool):
        resp = web.StreamResponse(status=200, headers={"Content-Type": "text/event-stream",
                                                       "Cache-Control": "no-cache", "X-Accel-Buffering": "no"})
        await resp.prepare(req)

        async def send(obj):
            await resp.write(b"data: " + json.dumps(obj, separators=(",", ":")).encode() + b"\n\n")

        def chunk(delta, finish=None):
            return {"id": rid, "object": "chat.completion.chunk", "created": CREATED, "model": model,
                    "choices": [{"index": 0, "delta": delta, "finish_reason": finish, "logprobs": None}]}
        announced = False
        streamed_calls = False

        async def announce():
            nonlocal announced
            if not announced:
                announced = True
                await send(chunk({"role": "assistant", "content": ""}))
        try:
            async for p in job.events():
                if p.kind == "token":
                    await announce()
                    await send(chunk({"content": p.text}))
                elif p.kind == "reasoning":
                    await announce()
                    await send(chunk({"reasoning_content": p.text}))
                elif p.kind == "tool_call_start":
                    streamed_calls = True
                    await announce()
                    await send(chunk({"tool_calls": [{"index": p.data["index"], "id": p.data["id"], "type": "function",
                                                      "function": {"name": p.data["name"], "arguments": ""}}]}))
                elif p.kind == "tool_call_args":
                    await send(chunk({"tool_calls": [{"index": p.data["index"], "function": {"arguments": p.text}}]}))
            r = read_outcome(await job.result())
            await announce()
            if r.tool_calls and not streamed_calls:      # calls parsed from the finished text
                await send(chunk({"tool_calls": [dict(tc, index=i) for i, tc in
                                                 enumerate(_tool_calls_json(r.tool_calls))]}))
            await send(chunk({}, _finish(r.finish_reason)))
            if include_usage:
                await send({"id": rid, "object": "chat.completion.chunk", "created": CREATED, "model": model,
                            "choices": [], "usage": _usage(r)})
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
            err = from_exception(e)
            await resp.write(b"event: error\ndata: " + json.dumps(err.body("openai")).encode() + b"\n\n")
        await resp.write(b"data: [DONE]\n\n")
        await resp.write_eof()
        return resp

    # ---- embeddings / images
    async def embeddings(self, req):
        body = await read_json(req)
        model = body.get("model")
        m = self.ex.get(model) if isinstance(model, str) else None
        if not isinstance(model, str) or not model:
            raise ApiError("invalid_request", "'model' is required")
        if m is None:
            raise ApiError("model_not_found", f"The model '{model}' does not exist.")
        if m.manifest().action("embed") is None:
            raise ApiError("invalid_request", f"The model '{model}' does not produce embeddings.")
        inp = body.get("input")
        inputs = [inp] if isinstance(inp, str) else inp
        if not isinstance(inputs, list) or not inputs or not all(isinstance(s, str) for s in inputs):
            raise ApiError("invalid_request", "'input' must be a string or an array of strings")
        data, toks = [], 0
        for i, text in enumerate(inputs):
            job = Job(self.ex, model, "embed", {"text": text})
            try:
                async for _ in job.events():
                    pass
                out = await job.result()
            except BaseException as e:
                job.abort()
                if type(e).__name__ == "CancelledError":
                    raise
                raise from_exception(e)
            data.append({"object": "embedding", "index": i, "embedding": out.outputs["mean"]})
            toks += int(out.outputs.get("tokens", 0))
        return web.json_response({"object": "list", "data": data, "model": model,
                                  "usage": {"prompt_tokens": toks, "total_tokens": toks}})

    async def images(self, req):
        body = await read_json(req)
        model = body.get("model") if isinstance(body, dict) else None
        if isinstance(model, str) and self.ex.get(model) is None:
            raise ApiError("model_not_found", f"The model '{model}' does not exist.")
        raise ApiError("not_implemented", "no image generation model is served by this build")


async def read_json(req: web.Request):
    raw = await req.read()
    try:
        return json.loads(raw.decode("utf-8"))
    except (ValueError, UnicodeDecodeError):
        raise ApiError("invalid_request", "request body is not valid JSON")
