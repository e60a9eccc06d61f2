"""Bridge between the async HTTP handlers and the blocking executor lanes (reference:
crates/apiserve/src/bridge.rs — ``read_outcome`` :73-112 pulls ``text``, token counts,
``finish_reason``, ``reasoning_content`` and ``tool_calls`` out of an action result; ``CancelGuard``
cancels the job when the client goes away; :250-285 per-request token accounting)."""
from __future__ import annotations

import asyncio
import json
import threading
from dataclasses import dataclass, field
from typing import Any, AsyncIterator, Dict, List, Optional, Tuple

from .capability import CancelToken, Invocation, Outcome, Progress
from .executor import Executor


@dataclass
class ChatResult:
    text: str
    prompt_tokens: int
    completion_tokens: int
    finish_reason: str
    reasoning_content: Optional[str] = None
    tool_calls: List[Dict[str, Any]] = field(default_factory=list)


def read_outcome(out: Outcome) -> ChatResult:
    o = out.outputs
    calls = []
    if o.get("tool_calls"):
        try:
            calls = json.loads(o["tool_calls"])
        except ValueError:
            calls = []
    return ChatResult(out.text(), int(o.get("prompt_tokens", 0)), int(o.get("completion_tokens", 0)),
                      str(o.get("finish_reason") or "stop"), o.get("reasoning_content"), calls)


class Accounting:
    """Cumulative per-surface token accounting."""

    def __init__(self):
        self.lock = threading.Lock()
        self.requests = 0
        self.prompt_tokens = 0
        self.completion_tokens = 0
        self.errors = 0

    def add(self, r: Optional[ChatResult]):
        with self.lock:
            self.requests += 1
            if r is None:
                self.errors += 1
            else:
                self.prompt_tokens += r.prompt_tokens
                self.completion_tokens += r.completion_tokens

    def snapshot(self) -> Dict[str, int]:
        with self.lock:
            return {"requests": self.requests, "prompt_tokens": self.prompt_tokens,
                    "completion_tokens": self.completion_tokens, "errors": self.errors}


_END = object()


class Job:
    """One in-flight action: ``events()`` yields Progress items then ends; ``result()`` returns
    the Outcome or raises.  Dropping the job (client disconnect) cancels it."""

    def __init__(self, ex: Executor, model_id: str, action: str, params: Dict[str, Any], blobs=None):
        self.loop = asyncio.get_running_loop()
        self.q: asyncio.Queue = asyncio.Queue()
        self.cancel = CancelToken()
        inv = Invocation(params, blobs or {}, self.cancel)

        def progress(p: Progress):
            self.loop.call_soon_threadsafe(self.q.put_nowait, p)

        self.fut = ex.submit(model_id, action, inv, progress)
        self.fut.add_done_callback(lambda f: self.loop.call_soon_threadsafe(self.q.put_nowait, _END))

    async def events(self) -> AsyncIterator[Progress]:
        while True:
            item = await self.q.get()
            if item is _END:
                return
            yield item

    async def result(self) -> Outcome:
        return await asyncio.wrap_future(self.fut)

    def abort(self):
        self.cancel.cancel()
