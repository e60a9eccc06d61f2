"""Shared client model (reference: brain-py/brain_py/base.py — ``Outcome`` :92-136, ``BrainError``
:59-90, ``EXIT_SKIP = 77`` and ``skip`` :44-56, ``BrainBase`` convenience wrappers :147-300)."""
from __future__ import annotations

import base64
import json
import sys
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Iterator, List, NoReturn, Optional

EXIT_SKIP = 77


def skip(reason: str) -> NoReturn:
    """Print ``SKIP: <reason>`` to stderr and exit with the skip status examples use."""
    print(f"SKIP: {reason}", file=sys.stderr)
    sys.exit(EXIT_SKIP)


class BrainError(RuntimeError):
    def __init__(self, message: str, *, name: Optional[str] = None, status: Optional[int] = None):
        super().__init__(message)
        self.message, self.name, self.status = message, name, status

    def __str__(self) -> str:
        return f"{self.name}: {self.message}" if self.name else self.message


@dataclass
class Outcome:
    outputs: Dict[str, Any] = field(default_factory=dict)
    blobs: Dict[str, Dict[str, Any]] = field(default_factory=dict)     # name -> {media, data(bytes), meta}

    def get(self, key: str, default: Any = None) -> Any:
        return self.outputs.get(key, default)

    def text(self, name: str = "text") -> str:
        b = self.blobs.get(name)
        return b["data"].decode("utf-8", errors="replace") if b else ""

    def bytes(self, name: str) -> bytes:
        return self.blobs[name]["data"]

    @staticmethod
    def from_wire(outputs: Dict[str, Any], blobs: List[Dict[str, Any]]) -> "Outcome":
        return Outcome(dict(outputs or {}), {
            b["name"]: {"media": b.get("media"), "data": base64.b64decode(b.get("b64", "")), "meta": b.get("meta") or {}}
            for b in blobs or []})


def flatten_messages(messages: Any) -> str:
    return messages if isinstance(messages, str) else json.dumps(messages)


class BrainBase:
    """Transports implement ``manifests``, ``run`` and ``subscribe``; the wrappers are shared."""

    def manifests(self) -> List[dict]:  # pragma: no cover - abstract
        raise NotImplementedError

    def run(self, model: str, action: str, params: Optional[dict] = None, *, blobs: Optional[dict] = None,
            timeout: float = 600.0) -> Outcome:  # pragma: no cover - abstract
        raise NotImplementedError

    def subscribe(self, model: str, action: str, params: Optional[dict] = None, *, blobs: Optional[dict] = None,
                  timeout: float = 600.0) -> Iterator[dict]:  # pragma: no cover - abstract
        raise NotImplementedError

    def close(self) -> None:
        pass

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    # ---- discovery
    def models(self) -> List[str]:
        return [m["model"] for m in self.manifests()]

    def actions(self, model: str) -> List[str]:
        for m in self.manifests():
            if m["model"] == model:
                return [a["name"] for a in m["actions"]]
        raise BrainError(f"unknown model {model!r}")

    def model_for(self, action: str) -> str:
        for m in self.manifests():
            if any(a["name"] == action for a in m["actions"]):
                return m["model"]
        raise BrainError(f"no served model offers action {action!r}")

    def _pick(self, action: str, model: Optional[str]) -> str:
        return model or self.model_for(action)

    # ---- wrappers
    def generate(self, prompt: Optional[str] = None, *, messages: Any = None, model: Optional[str] = None,
                 max_new: Optional[int] = None, temp: Optional[float] = None, top_k: Optional[int] = None,
                 top_p: Optional[float] = None, seed: Optional[int] = None, system: Optional[str] = None,
                 stop: Optional[List[str]] = None, on_token: Optional[Callable[[str], None]] = None,
                 timeout: float = 600.0, **extra) -> Outcome:
        params: Dict[str, Any] = dict(extra)
        if messages is not None:
            params["messages"] = flatten_messages(messages)
        elif prompt is not None:
            params["prompt"] = prompt
        else:
            raise ValueError("generate needs prompt= or messages=")
        for k, v in (("max_new", max_new), ("temp", temp), ("top_k", top_k), ("top_p", top_p), ("seed", seed),
                     ("system", system)):
            if v is not None:
                params[k] = v
        if stop:
            params["stop"] = json.dumps(list(stop))
        m = self._pick("generate", model)
        if on_token is None:
            return self.run(m, "generate", params, timeout=timeout)
        result: Optional[Outcome] = None
        for ev in self.subscribe(m, "generate", params, timeout=timeout):
            if ev["type"] == "token":
                on_token(ev["text"])
            elif ev["type"] == "result":
                result = ev["outcome"]
        if result is None:
            raise BrainError("stream ended without a result")
        return result

    def chat(self, text: str, *, model: Optional[str] = None, **kw) -> str:
        return self.generate(messages=[{"role": "user", "content": text}], model=model, **kw).text()

    def embed(self, text: str, *, model: Optional[str] = None, timeout: float = 120.0) -> List[float]:
        out = self.run(self._pick("embed", model), "embed", {"text": text}, timeout=timeout)
        return list(out.get("mean") or [])

    def text2image(self, prompt: str, *, model: Optional[str] = None, timeout: float = 600.0, **params) -> bytes:
        """Image bytes from the first model that provides ``text2image`` (none of the models this
        server build ships does: the call then raises ``BrainError`` naming the missing action)."""
        out = self.run(self._pick("text2image", model), "text2image", dict(params, prompt=prompt), timeout=timeout)
        return out.bytes("image")
