"""Error bodies per dialect (reference: crates/apiserve/src/error.rs:14-180).  Internal failure text
is never shown to a client: anything that is not a deliberate, client-safe message becomes a
generic ``server_error`` (crates/apiserve/src/bridge.rs:151-156)."""
from __future__ import annotations

import re
from dataclasses import dataclass
from typing import Dict, Optional, Tuple

_TABLE = {
    # code: (http status, openai type, anthropic type)
    "invalid_api_key": (401, "invalid_request_error", "authentication_error"),
    "model_not_found": (404, "invalid_request_error", "not_found_error"),
    "not_found": (404, "invalid_request_error", "not_found_error"),
    "invalid_request": (400, "invalid_request_error", "invalid_request_error"),
    "context_length_exceeded": (400, "invalid_request_error", "invalid_request_error"),
    "payload_too_large": (413, "invalid_request_error", "request_too_large"),
    "not_implemented": (501, "invalid_request_error", "invalid_request_error"),
    "rate_limit_exceeded": (429, "rate_limit_error", "rate_limit_error"),
    "server_error": (503, "server_error", "overloaded_error"),
    "internal_error": (500, "server_error", "api_error"),
}

_CAPACITY_RE = re.compile(r"needs (\d+) tokens, engine capacity is (\d+)")


@dataclass
class ApiError(Exception):
    code: str
    message: str
    retry_after: Optional[int] = None

    @property
    def status(self) -> int:
        return _TABLE[self.code][0]

    def headers(self) -> Dict[str, str]:
        return {"Retry-After": str(self.retry_after)} if self.retry_after is not None else {}

    def body(self, dialect: str) -> Dict:
        _, otype, atype = _TABLE[self.code]
        if dialect == "anthropic":
            return {"type": "error", "error": {"type": atype, "message": self.message}}
        code = "server_error" if self.code == "internal_error" else self.code
        return {"error": {"message": self.message, "type": otype, "param": None, "code": code}}


def from_exception(e: BaseException) -> ApiError:
    """Map executor / model failures onto the public error vocabulary."""
    from .capability import ActionError, ValidationError
    from .executor import Busy
    if isinstance(e, ApiError):
        return e
    if isinstance(e, Busy):
        if e.shed:
            return ApiError("server_error", "The server is overloaded; retry shortly.", 1)
        return ApiError("rate_limit_exceeded", "The model is busy; retry shortly.", 1)
    if isinstance(e, ValidationError):
        return ApiError("invalid_request", str(e))
    if isinstance(e, ActionError):
        m = _CAPACITY_RE.search(str(e))
        if m or e.kind == "context_length_exceeded":
            msg = (f"This model's maximum context length is {m.group(2)} tokens; the request needs "
                   f"{m.group(1)}." if m else str(e))
            return ApiError("context_length_exceeded", msg)
        if e.kind == "not_implemented":
            return ApiError("not_implemented", str(e))
        if e.kind == "rate_limit_exceeded":     # the scheduler's admission policy turned it away
            return ApiError("rate_limit_exceeded", "The model is busy; retry shortly.", 1)
        if e.kind == "cancelled":
            return ApiError("invalid_request", "request cancelled")
        return ApiError("invalid_request", str(e))
    if isinstance(e, KeyError):
        return ApiError("model_not_found", f"The model {e.args[0]!r} does not exist.")
    return ApiError("internal_error", "The server had an error while processing the request.")
