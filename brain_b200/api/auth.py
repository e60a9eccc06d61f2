"""API keys (reference: crates/apiserve/src/surface.rs:60-113 — a fresh ``sk-brain-<32 hex>`` key
per surface, printed as ``APIKEY <provider> <key>`` and optionally written as a mode-0600 JSON map;
crates/apiserve/src/auth.rs:14-45 — bearer / x-api-key extraction with a constant-time compare)."""
from __future__ import annotations

import hmac
import json
import os
import secrets
from typing import Dict, Mapping, Optional


def new_key() -> str:
    return "sk-brain-" + secrets.token_hex(16)


def write_keys(path: str, keys: Dict[str, str]) -> None:
    tmp = path + ".tmp"
    fd = os.open(tmp, os.O_WRONLY | os.O_CREAT | os.O_TRUNC, 0o600)
    with os.fdopen(fd, "w") as f:
        json.dump(keys, f)
    os.chmod(tmp, 0o600)
    os.replace(tmp, path)


def presented_key(headers: Mapping[str, str], scheme: str) -> Optional[str]:
    """``scheme='bearer'``: ``Authorization: Bearer <key>``; ``'x-api-key'``: that header (a bearer
    token is accepted as a fallback, as SDKs differ)."""
    auth = headers.get("Authorization") or headers.get("authorization")
    bearer = auth[7:].strip() if auth and auth[:7].lower() == "bearer " else None
    if scheme == "x-api-key":
        return headers.get("x-api-key") or headers.get("X-Api-Key") or bearer
    return bearer


def check(headers: Mapping[str, str], scheme: str, expected: str) -> bool:
    got = presented_key(headers, scheme)
    if got is None:
        return False
    return hmac.compare_digest(got.encode("utf-8"), expected.encode("utf-8"))
