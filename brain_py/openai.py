"""OpenAI-dialect HTTP transport (reference: brain-py/brain_py/openai.py): ``run``/``subscribe`` for
``generate`` map to ``/v1/chat/completions`` (SSE when subscribing), ``embed`` to ``/v1/embeddings``;
``manifests`` is synthesised from ``/v1/models``.  Standard library only."""
from __future__ import annotations

import json
import urllib.error
import urllib.request
from typing import Any, Dict, Iterator, List, Optional

from .base import BrainBase, BrainError, Outcome


def _normalize(url: str) -> str:
    url = url.rstrip("/")
    return url if url.endswith("/v1") else url + "/v1"


class BrainOpenAI(BrainBase):
    def __init__(self, base_url: str = "http://127.0.0.1:8788", api_key: str = "", timeout: float = 600.0):
        self.base = _normalize(base_url)
        self.api_key = api_key
        self.timeout = timeout

    def _headers(self) -> Dict[str, str]:
        h = {"Content-Type": "application/json"}
        if self.api_key:
            h["Authorization"] = f"Bearer {self.api_key}"
        return h

    def _open(self, path: str, body: Optional[dict], timeout: float):
        data = json.dumps(body).encode() if body is not None else None
        req = urllib.request.Request(self.base + path, data=data, headers=self._headers(),
                                     method="POST" if body is not None else "GET")
        try:
            return urllib.request.urlopen(req, timeout=timeout)
        except urllib.error.HTTPError as e:
            raw = e.read().decode("utf-8", errors="replace")
            try:
                err = json.loads(raw)["error"]
                raise BrainError(err.get("message", raw), name=err.get("code"), status=e.code) from None
            except (ValueError, KeyError, TypeError):
                raise BrainError(raw or str(e), status=e.code) from None
        except urllib.error.URLError as e:
            raise BrainError(f"cannot reach {self.base}: {e.reason}") from None

    def manifests(self) -> List[dict]:
        with self._open("/models", None, 30.0) as r:
            data = json.load(r)["data"]
        return [{"model": m["id"], "summary": "", "max_context_tokens": m.get("context_length"),
                 "actions": [{"name": "generate", "streaming": True}, {"name": "embed", "streaming": False}]}
                for m in data]

    @staticmethod
    def _chat_body(model: str, params: dict, stream: bool) -> dict:
        p = dict(params)
        if "messages" in p:
            msgs = json.loads(p.pop("messages")) if isinstance(p["messages"], str) else p.pop("messages")
        else:
            msgs = [{"role": "user", "content": p.pop("prompt", "")}]
        if p.get("system"):
            msgs = [{"role": "system", "content": p.pop("system")}] + msgs
        body: Dict[str, Any] = {"model": model, "messages": msgs, "stream": stream}
        for src, dst in (("max_new", "max_tokens"), ("temp", "temperature"), ("top_p", "top_p"), ("top_k", "top_k"),
                         ("seed", "seed")):
            if src in p:
                body[dst] = p[src]
        if p.get("stop"):
            body["stop"] = json.loads(p["stop"]) if isinstance(p["stop"], str) else p["stop"]
        if p.get("tools"):
            body["tools"] = json.loads(p["tools"]) if isinstance(p["tools"], str) else p["tools"]
        if "enable_thinking" in p:
            body["chat_template_kwargs"] = {"enable_thinking": bool(p["enable_thinking"])}
        if stream:
            body["stream_options"] = {"include_usage": True}
        return body

    def run(self, model, action, params=None, *, blobs=None, timeout: Optional[float] = None) -> Outcome:
        params = params or {}
        timeout = timeout or self.timeout
        if action == "embed":
            with self._open("/embeddings", {"model": model, "input": params.get("text", "")}, timeout) as r:
                d = json.load(r)
            return Outcome({"mean": d["data"][0]["embedding"], "tokens": d["usage"]["prompt_tokens"]})
        if action != "generate":
            raise BrainError(f"the OpenAI transport has no mapping for action {action!r}")
        with self._open("/chat/completions", self._chat_body(model, params, False), timeout) as r:
            d = json.load(r)
        ch = d["choices"][0]
        msg = ch["message"]
        out = {"prompt_tokens": d["usage"]["prompt_tokens"], "completion_tokens": d["usage"]["completion_tokens"],
               "finish_reason": ch["finish_reason"]}
        if msg.get("reasoning_content"):
            out["reasoning_content"] = msg["reasoning_content"]
        if msg.get("tool_calls"):
            out["tool_calls"] = json.dumps([{"id": t["id"], "name": t["function"]["name"],
                                             "arguments": t["function"]["arguments"]} for t in msg["tool_calls"]])
        return Outcome(out, {"text": {"media": "text", "data": (msg.get("content") or "").encode(), "meta": {}}})

    def subscribe(self, model, action, params=None, *, blobs=None, timeout: Optional[float] = None) -> Iterator[dict]:
        if action != "generate":
            yield {"type": "result", "outcome": self.run(model, action, params, timeout=timeout)}
            return
        text: List[str] = []
        finish, usage = "stop", {}
        event = None
        with self._open("/chat/completions", self._chat_body(model, params or {}, True), timeout or self.timeout) as r:
            for raw in r:
                line = raw.decode("utf-8").rstrip("\n")
                if line.startswith("event:"):
                    event = line[6:].strip()
                    continue
                if not line.startswith("data:"):
                    continue
                payload = line[5:].strip()
                if payload == "[DONE]":
                    break
                obj = json.loads(payload)
                if event == "error" or "error" in obj:
                    err = obj.get("error", {})
                    raise BrainError(err.get("message", "error"), name=err.get("code"))
                if obj.get("usage"):
                    usage = obj["usage"]
                for ch in obj.get("choices", []):
                    d = ch.get("delta", {})
                    if d.get("content"):
                        text.append(d["content"])
                        yield {"type": "token", "text": d["content"]}
                    elif any(k in d for k in ("reasoning_content", "tool_calls")):
                        yield {"type": "event", "data": d}
                    if ch.get("finish_reason"):
                        finish = ch["finish_reason"]
        out = {"prompt_tokens": usage.get("prompt_tokens", 0), "completion_tokens": usage.get("completion_tokens", 0),
               "finish_reason": finish}
        yield {"type": "result", "outcome": Outcome(out, {"text": {"media": "text", "data": "".join(text).encode(),
                                                                    "meta": {}}})}
