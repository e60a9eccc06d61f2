"""Capability manifests and typed invocations (reference: crates/capability/src/lib.rs:206-214,
304-310 manifest/action/param shapes; :218-262 ``ActionSpec::validate`` — unknown parameters are
rejected, types checked, defaults filled; ``last_user_text`` picks the prompt a chat action sees)."""
from __future__ import annotations

import base64
import json
import threading
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional

_TYPES = {"str": str, "int": int, "float": (int, float), "bool": bool}


class ValidationError(ValueError):
    pass


@dataclass
class ParamSpec:
    name: str
    type: str
    summary: str = ""
    default: Any = None
    required: bool = False

    def to_json(self):
        v = {"name": self.name, "type": self.type, "summary": self.summary, "required": self.required}
        if self.default is not None:
            v["default"] = self.default
        return v


@dataclass
class BlobSpec:
    name: str
    media: str
    summary: str = ""
    required: bool = False

    def to_json(self):
        return {"name": self.name, "media": self.media, "summary": self.summary, "required": self.required}


@dataclass
class ActionSpec:
    name: str
    summary: str = ""
    streaming: bool = False
    params: List[ParamSpec] = field(default_factory=list)
    inputs: List[BlobSpec] = field(default_factory=list)
    outputs: List[BlobSpec] = field(default_factory=list)

    def validate(self, params: Dict[str, Any], blobs: Optional[Dict[str, "Blob"]] = None) -> Dict[str, Any]:
        known = {p.name: p for p in self.params}
        out: Dict[str, Any] = {}
        for k, v in params.items():
            spec = known.get(k)
            if spec is None:
                raise ValidationError(f"action '{self.name}': unknown parameter '{k}'")
            if v is None:
                continue
            if spec.type == "float" and isinstance(v, bool) or spec.type == "int" and isinstance(v, bool):
                raise ValidationError(f"parameter '{k}' must be {spec.type}")
            if spec.type == "int" and isinstance(v, float) and v.is_integer():
                v = int(v)
            if not isinstance(v, _TYPES[spec.type]):
                raise ValidationError(f"parameter '{k}' must be {spec.type}")
            out[k] = float(v) if spec.type == "float" else v
        for p in self.params:
            if p.name not in out:
                if p.required:
                    raise ValidationError(f"action '{self.name}': missing required parameter '{p.name}'")
                if p.default is not None:
                    out[p.name] = p.default
        have = blobs or {}
        names = {b.name for b in self.inputs}
        for k in have:
            if k not in names:
                raise ValidationError(f"action '{self.name}': unknown input blob '{k}'")
        for b in self.inputs:
            if b.required and b.name not in have:
                raise ValidationError(f"action '{self.name}': missing required input blob '{b.name}'")
        return out

    def to_json(self):
        return {"name": self.name, "summary": self.summary, "streaming": self.streaming,
                "params": [p.to_json() for p in self.params], "inputs": [b.to_json() for b in self.inputs],
                "outputs": [b.to_json() for b in self.outputs]}


@dataclass
class Manifest:
    model: str
    summary: str
    actions: List[ActionSpec]
    max_context_tokens: Optional[int] = None

    def action(self, name: str) -> Optional[ActionSpec]:
        return next((a for a in self.actions if a.name == name), None)

    def is_chat(self) -> bool:
        a = self.action("generate")
        return a is not None and a.streaming and any(p.name in ("messages", "prompt") for p in a.params)

    def to_json(self):
        v = {"model": self.model, "summary": self.summary, "actions": [a.to_json() for a in self.actions]}
        if self.max_context_tokens is not None:
            v["max_context_tokens"] = self.max_context_tokens
        return v


@dataclass
class Blob:
    media: str
    data: bytes
    meta: Dict[str, Any] = field(default_factory=dict)

    def to_json(self, name: str):
        return {"name": name, "media": self.media, "b64": base64.b64encode(self.data).decode("ascii"),
                "meta": self.meta}

    @staticmethod
    def from_json(d) -> "Blob":
        return Blob(d.get("media", "bytes"), base64.b64decode(d.get("b64", "")), d.get("meta") or {})


class CancelToken:
    def __init__(self):
        self._ev = threading.Event()
        self._hooks: List[Callable[[], None]] = []

    def cancel(self):
        self._ev.set()
        for h in list(self._hooks):
            try:
                h()
            except Exception:
                pass

    def is_cancelled(self) -> bool:
        return self._ev.is_set()

    def on_cancel(self, fn: Callable[[], None]):
        self._hooks.append(fn)
        if self._ev.is_set():
            fn()


@dataclass
class Invocation:
    params: Dict[str, Any]
    blobs: Dict[str, Blob] = field(default_factory=dict)
    cancel: CancelToken = field(default_factory=CancelToken)


@dataclass
class Outcome:
    outputs: Dict[str, Any] = field(default_factory=dict)
    blobs: Dict[str, Blob] = field(default_factory=dict)

    def text(self) -> str:
        b = self.blobs.get("text")
        return b.data.decode("utf-8", errors="replace") if b else ""


@dataclass
class Progress:
    """A streamed step: ``kind`` is token | reasoning | tool_call_start | tool_call_args |
    tool_call_end | step."""
    kind: str
    step: int = 0
    total: int = 0
    text: str = ""
    data: Dict[str, Any] = field(default_factory=dict)


class ActionError(RuntimeError):
    """A failure whose message is safe to show to the client (validation, capacity)."""

    def __init__(self, message: str, kind: str = "invalid_request"):
        super().__init__(message)
        self.kind = kind


def last_user_text(params: Dict[str, Any]) -> str:
    msgs = params.get("messages")
    if msgs:
        try:
            arr = json.loads(msgs) if isinstance(msgs, str) else msgs
            for m in reversed(arr):
                if m.get("role") == "user":
                    c = m.get("content")
                    if isinstance(c, list):
                        return " ".join(p.get("text", "") for p in c if isinstance(p, dict))
                    return c or ""
        except (ValueError, AttributeError):
            pass
    return params.get("prompt") or ""


def generate_spec(summary: str) -> ActionSpec:
    """The chat action contract shared by every language model (reference:
    crates/cli/src/resident_llm.rs:41-66)."""
    P = ParamSpec
    return ActionSpec("generate", summary, True, [
        P("prompt", "str", "a raw prompt (alternative to messages)"),
        P("messages", "str", "chat messages as a JSON array string"),
        P("system", "str", "system prompt"),
        P("chat", "bool", "apply the chat template", True),
        P("max_new", "int", "max new tokens", 128),
        P("temp", "float", "sampling temperature", 0.8),
        P("top_k", "int", "top-k", 40),
        P("top_p", "float", "nucleus sampling p", 1.0),
        P("seed", "int", "sampling seed", 0),
        P("stop", "str", "stop sequences as a JSON array string"),
        P("tools", "str", "tool definitions as a JSON array string"),
        P("tool_choice", "str", "tool_choice directive"),
        P("enable_thinking", "bool", "let the model think before answering", True),
        P("ignore_eos", "bool", "keep generating past the end-of-turn token (benchmarks)", False),
    ], [], [BlobSpec("text", "text", "the generated text")])


def all_manifests() -> List[Manifest]:
    from .resident import registry_from_env
    return [m.manifest() for m in registry_from_env(load=False).values()]
