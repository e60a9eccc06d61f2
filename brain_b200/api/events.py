"""JSONL event protocol: one JSON object per line with ``"event"`` and an optional ``"req_id"``
echo (reference: crates/events/src/lib.rs:144-175 framing, :190-283 event set).

Client -> server: ``manifest_request``, ``action_request{model,action,params,blobs}``,
``user_text{text}``, ``cancel``.  Server -> client: ``ready``, ``manifest_result``,
``action_progress{step,total,message}``, ``action_result{outputs,blobs}``,
``brain_text_chunk{text,seq,done}``, ``error{message}``, ``log{message}``, ``cancelled``."""
from __future__ import annotations

import json
from typing import Any, Dict, Optional

CLIENT_EVENTS = ("manifest_request", "action_request", "user_text", "cancel")
SERVER_EVENTS = ("ready", "manifest_result", "action_progress", "action_result", "brain_text_chunk",
                 "error", "log", "cancelled")
TERMINAL = ("action_result", "error", "cancelled", "manifest_result")


def encode(event: str, req_id: Optional[str] = None, **fields) -> str:
    obj: Dict[str, Any] = {"event": event}
    if req_id is not None:
        obj["req_id"] = req_id
    obj.update(fields)
    return json.dumps(obj, separators=(",", ":"), ensure_ascii=False)


def decode(line: str) -> Dict[str, Any]:
    obj = json.loads(line)
    if not isinstance(obj, dict) or not isinstance(obj.get("event"), str):
        raise ValueError("not an event object")
    return obj
