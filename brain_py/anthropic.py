"""Anthropic-dialect HTTP transport (reference: brain-py/brain_py/anthropic.py): ``generate`` maps to
``POST /v1/messages`` (``x-api-key``), streaming through the Messages SSE event set."""
from __future__ import annotations

import json
import urllib.error
import urllib.request
from typing import Dict, Iterator, List, Optional, Tuple

from .base import BrainBase, BrainError, Outcome

_FINISH = {"end_turn": "stop", "max_tokens": "length", "stop_sequence": "stop_sequence"}


class BrainAnthropic(BrainBase):
    def __init__(self, base_url: str = "http://127.0.0.1:8787", api_key: str = "", timeout: float = 600.0):
        self.base = base_url.rstrip("/")
        if self.base.endswith("/v1"):
            self.base = self.base[:-3]
        self.api_key = api_key
        self.timeout = timeout

    def _headers(self) -> Dict[str, str]:
        return {"Content-Type": "application/json", "x-api-key": self.api_key, "anthropic-version": "2023-06-01"}

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
                raise BrainError(err.get("message", raw), name=err.get("type"), status=e.code) from None
            except (ValueError, KeyError, TypeError):
                raise BrainError(raw or str(e), status=e.code) from None
        except urllib.error.URLError as e:
            raise BrainError(f"cannot reach {self.base}: {e.reason}") from None

    def manifests(self) -> List[dict]:
        with self._open("/v1/models", None, 30.0) as r:
            data = json.load(r)["data"]
        return [{"model": m["id"], "summary": "", "actions": [{"name": "generate", "streaming": True}]} for m in data]

    @staticmethod
    def _build(model: str, params: dict, stream: bool) -> dict:
        p = dict(params)
        if "messages" in p:
            msgs = json.loads(p["messages"]) if isinstance(p["messages"], str) else p["messages"]
        else:
            msgs = [{"role": "user", "content": p.get("prompt", "")}]
        system = p.get("system")
        keep = []
        for m in msgs:
            if m.get("role") == "system":
                system = (system + "\n" if system else "") + (m.get("content") or "")
            else:
                keep.append({"role": m["role"], "content": m.get("content") or ""})
        body = {"model": model, "messages": keep, "max_tokens": int(p.get("max_new", 1024)), "stream": stream}
        if system:
            body["system"] = system
        if "temp" in p:
            body["temperature"] = p["temp"]
        if "top_p" in p:
            body["top_p"] = p["top_p"]
        if "top_k" in p:
            body["top_k"] = p["top_k"]
        if p.get("stop"):
            body["stop_sequences"] = json.loads(p["stop"]) if isinstance(p["stop"], str) else p["stop"]
        return body

    def count_tokens(self, messages, system: Optional[str] = None) -> int:
        body = {"model": "any", "messages": messages}
        if system:
            body["system"] = system
        with self._open("/v1/messages/count_tokens", body, 30.0) as r:
            return int(json.load(r)["input_tokens"])

    def run(self, model, action, params=None, *, blobs=None, timeout: Optional[float] = None) -> Outcome:
        if action != "generate":
            raise BrainError(f"the Anthropic transport has no mapping for action {action!r}")
        with self._open("/v1/messages", self._build(model, params or {}, False), timeout or self.timeout) as r:
            d = json.load(r)
        text = "".join(b.get("text", "") for b in d["content"] if b.get("type") == "text")
        out = {"prompt_tokens": d["usage"]["input_tokens"], "completion_tokens": d["usage"]["output_tokens"],
               "finish_reason": _FINISH.get(d.get("stop_reason"), "stop")}
        return Outcome(out, {"text": {"media": "text", "data": text.encode(), "meta": {}}})

    def subscribe(self, model, action, params=None, *, blobs=None, timeout: Optional[float] = None) -> Iterator[dict]:
        if action != "generate":
            raise BrainError(f"the Anthropic transport has no mapping for action {action!r}")
        text: List[str] = []
        usage, finish, event = {}, "stop", None
        with self._open("/v1/messages", self._build(model, params or {}, True), timeout or self.timeout) as r:
            for raw in r:
                line = raw.decode("utf-8").rstrip("\n")
                if line.startswith("event:"):
                    event = line[6:].strip()
                    continue
                if not line.startswith("data:"):
                    continue
                obj = json.loads(line[5:].strip())
                if event == "error":
                    err = obj.get("error", {})
                    raise BrainError(err.get("message", "error"), name=err.get("type"))
                if event == "content_block_delta":
                    piece = obj.get("delta", {}).get("text", "")
                    if piece:
                        text.append(piece)
                        yield {"type": "token", "text": piece}
                elif event == "message_delta":
                    usage = obj.get("usage", usage)
                    finish = _FINISH.get(obj.get("delta", {}).get("stop_reason"), "stop")
                elif event == "message_stop":
                    break
        out = {"prompt_tokens": usage.get("input_tokens", 0), "completion_tokens": usage.get("output_tokens", 0),
               "finish_reason": finish}
        yield {"type": "result", "outcome": Outcome(out, {"text": {"media": "text", "data": "".join(text).encode(),
                                                                    "meta": {}}})}
