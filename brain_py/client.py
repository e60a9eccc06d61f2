"""JSONL-over-stdio transport (reference: brain-py/brain_py/client.py — spawn ``brain serve
--stdio``, a reader thread demultiplexes replies on ``req_id``, terminal events are
``action_result | error | cancelled | manifest_result``)."""
from __future__ import annotations

import base64
import itertools
import json
import os
import queue
import subprocess
import sys
import threading
from typing import Any, Dict, Iterator, List, Optional

from .base import BrainBase, BrainError, Outcome

_TERMINAL = ("action_result", "error", "cancelled", "manifest_result")


def _find_brain(explicit: Optional[str]) -> List[str]:
    if explicit:
        return [explicit]
    env = os.environ.get("BRAIN_BIN")
    if env:
        return [env]
    here = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "brain")
    if os.path.exists(here):
        return [sys.executable, here]
    return [sys.executable, "-m", "brain_b200.cli"]


def _wire_blobs(blobs: Optional[dict]) -> List[dict]:
    out = []
    for name, b in (blobs or {}).items():
        if isinstance(b, (bytes, bytearray)):
            b = {"media": "bytes", "data": bytes(b)}
        out.append({"name": name, "media": b.get("media", "bytes"),
                    "b64": base64.b64encode(b["data"]).decode("ascii"), "meta": b.get("meta") or {}})
    return out


class BrainStdio(BrainBase):
    def __init__(self, brain_bin: Optional[str] = None, *, env: Optional[Dict[str, str]] = None,
                 args: Optional[List[str]] = None, device: Optional[str] = None, ready_timeout: float = 300.0):
        cmd = _find_brain(brain_bin) + ["serve", "--stdio"] + list(args or [])
        if device:
            cmd += ["--device", device]
        full_env = dict(os.environ)
        full_env.update(env or {})
        self.proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, stderr=subprocess.PIPE,
                                     text=True, bufsize=1, env=full_env)
        self._ids = itertools.count(1)
        self._pending: Dict[str, "queue.Queue[dict]"] = {}
        self._lock = threading.Lock()
        self._ready = threading.Event()
        self._dead: Optional[str] = None
        self.stderr_tail: List[str] = []
        threading.Thread(target=self._reader, daemon=True).start()
        threading.Thread(target=self._drain_stderr, daemon=True).start()
        if not self._ready.wait(ready_timeout):
            self.close()
            raise BrainError("brain serve --stdio did not become ready: " + " | ".join(self.stderr_tail[-5:]))

    # ---- plumbing
    def _reader(self):
        try:
            for line in self.proc.stdout:
                line = line.strip()
                if not line:
                    continue
                try:
                    ev = json.loads(line)
                except ValueError:
                    continue
                if ev.get("event") == "ready":
                    self._ready.set()
                    continue
                q = self._pending.get(ev.get("req_id"))
                if q is not None:
                    q.put(ev)
        finally:
            self._dead = "server closed the stream"
            self._ready.set()
            for q in list(self._pending.values()):
                q.put({"event": "error", "message": self._dead})

    def _drain_stderr(self):
        for line in self.proc.stderr:
            self.stderr_tail.append(line.rstrip())
            del self.stderr_tail[:-50]

    def _send(self, obj: dict):
        if self._dead or self.proc.poll() is not None:
            raise BrainError("brain serve is not running")
        with self._lock:
            self.proc.stdin.write(json.dumps(obj, separators=(",", ":")) + "\n")
            self.proc.stdin.flush()

    def _open(self) -> str:
        rid = f"r{next(self._ids)}"
        self._pending[rid] = queue.Queue()
        return rid

    def _events(self, rid: str, timeout: float) -> Iterator[dict]:
        q = self._pending[rid]
        try:
            while True:
                try:
                    ev = q.get(timeout=timeout)
                except queue.Empty:
                    self._send({"event": "cancel", "req_id": rid})
                    raise BrainError(f"timed out after {timeout:.0f} s")
                yield ev
                if ev.get("event") in _TERMINAL:
                    return
        finally:
            self._pending.pop(rid, None)

    # ---- API
    def manifests(self, timeout: float = 30.0) -> List[dict]:
        rid = self._open()
        self._send({"event": "manifest_request", "req_id": rid})
        for ev in self._events(rid, timeout):
            if ev["event"] == "manifest_result":
                return ev["manifests"]
            if ev["event"] == "error":
                raise BrainError(ev.get("message", "error"))
        raise BrainError("no manifest_result")

    def subscribe(self, model, action, params=None, *, blobs=None, timeout: float = 600.0) -> Iterator[dict]:
        rid = self._open()
        self._send({"event": "action_request", "req_id": rid, "model": model, "action": action,
                    "params": params or {}, "blobs": _wire_blobs(blobs)})
        for ev in self._events(rid, timeout):
            kind = ev["event"]
            if kind == "action_progress":
                msg = ev.get("message")
                if isinstance(msg, str):
                    yield {"type": "token", "text": msg, "step": ev.get("step"), "total": ev.get("total")}
                else:
                    yield {"type": "event", "data": msg}
            elif kind == "action_result":
                yield {"type": "result", "outcome": Outcome.from_wire(ev.get("outputs"), ev.get("blobs"))}
            elif kind == "cancelled":
                raise BrainError("cancelled", name="cancelled")
            elif kind == "error":
                raise BrainError(ev.get("message", "error"))

    def run(self, model, action, params=None, *, blobs=None, timeout: float = 600.0) -> Outcome:
        for ev in self.subscribe(model, action, params, blobs=blobs, timeout=timeout):
            if ev["type"] == "result":
                return ev["outcome"]
        raise BrainError("stream ended without a result")

    def converse(self, text: str, timeout: float = 120.0) -> str:
        """The ``user_text`` verb: streamed ``brain_text_chunk`` pieces joined."""
        rid = self._open()
        self._send({"event": "user_text", "req_id": rid, "text": text})
        parts: List[str] = []
        for ev in self._events(rid, timeout):
            if ev["event"] == "brain_text_chunk":
                parts.append(ev.get("text", ""))
            elif ev["event"] == "error":
                raise BrainError(ev.get("message", "error"))
        return "".join(parts)

    def close(self):
        try:
            if self.proc.poll() is None:
                self.proc.stdin.close()
                self.proc.wait(timeout=10)
        except Exception:
            try:
                self.proc.kill()
            except Exception:
                pass


BrainClient = BrainStdio
