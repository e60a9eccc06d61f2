"""brain_py: Python client for a running ``brain serve`` (reference: brain-py/brain_py/__init__.py —
one high-level capability API over interchangeable transports).

Transports: ``jsonl`` (spawns ``brain serve --stdio`` and correlates by ``req_id``), ``openai`` and
``anthropic`` (HTTP).  The reference's default D-Bus transport is not offered: there is no D-Bus
service in this framework.

    from brain_py import Brain
    with Brain(transport="jsonl", env={"BRAIN_MOCK": "1"}) as brain:
        print(brain.models())
        print(brain.generate(prompt="hello", model="brain/mock").text())
"""
from typing import Any

from .anthropic import BrainAnthropic
from .base import EXIT_SKIP, BrainBase, BrainError, Outcome, skip
from .client import BrainStdio
from .openai import BrainOpenAI


def Brain(transport: str = "jsonl", **kwargs: Any) -> BrainBase:
    t = transport.lower()
    if t in ("jsonl", "stdio", "stdout"):
        return BrainStdio(**kwargs)
    if t == "openai":
        return BrainOpenAI(**kwargs)
    if t == "anthropic":
        return BrainAnthropic(**kwargs)
    if t in ("dbus", "d-bus", "bus"):
        raise BrainError("the D-Bus transport is not available in this build; use 'jsonl', 'openai' or 'anthropic'")
    raise ValueError(f"unknown transport {transport!r}; use 'jsonl', 'openai' or 'anthropic'")


__all__ = ["Brain", "BrainStdio", "BrainOpenAI", "BrainAnthropic", "BrainBase", "BrainError", "Outcome",
           "EXIT_SKIP", "skip"]
