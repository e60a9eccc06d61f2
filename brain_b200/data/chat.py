"""Chat / SFT dataset preparation (reference: crates/data/src/chat.rs — ``ChatExample::encode``
masks the prompt and supervises ``assistant + <|im_end|>\\n``, an end-of-text token separates
examples; ``prepare_chat`` writes train/val token files plus the supervision mask)."""
from __future__ import annotations

import json
import re
from dataclasses import dataclass
from pathlib import Path
from typing import Dict, Iterable, List, Optional, Tuple

import numpy as np

from . import binio

ENDOFTEXT = 151643


@dataclass
class ChatExample:
    user: str
    assistant: str
    system: Optional[str] = None

    def messages(self) -> List[Tuple[str, str]]:
        m = [("system", self.system)] if self.system else []
        m.append(("user", self.user))
        return m

    def encode(self, tok) -> Tuple[List[int], List[int]]:
        prompt = tok.encode(tok.apply_chat_template(self.messages(), True))
        resp = tok.encode(f"{self.assistant}<|im_end|>\n")
        eot = tok.special.get("<|endoftext|>", ENDOFTEXT) if hasattr(tok, "special") else ENDOFTEXT
        return prompt + resp + [eot], [0] * len(prompt) + [1] * len(resp) + [0]


def encode_split(examples: Iterable[ChatExample], tok) -> Tuple[np.ndarray, np.ndarray]:
    ids: List[int] = []
    mask: List[int] = []
    for ex in examples:
        i, m = ex.encode(tok)
        ids += i
        mask += m
    return np.asarray(ids, dtype=np.uint32), np.asarray(mask, dtype=np.uint8)


def prepare_chat(train: List[ChatExample], val: List[ChatExample], tok, vocab: int, out_dir) -> None:
    tr, trm = encode_split(train, tok)
    va, _ = encode_split(val, tok)
    binio.write_dataset(out_dir, tr, va, vocab, None, mask=trm)


def load_jsonl(path) -> List[Dict]:
    out = []
    with open(path, encoding="utf-8") as f:
        for line in f:
            line = line.strip()
            if line:
                out.append(json.loads(line))
    return out


def examples_from_records(records: List[Dict]) -> List[ChatExample]:
    """Accepts ``{"messages":[...]}`` (last assistant turn supervised) or ``{"prompt","response"}``
    / ``{"user","assistant"[,"system"]}`` records."""
    out = []
    for r in records:
        if "messages" in r:
            msgs = r["messages"]
            sys_ = next((m["content"] for m in msgs if m["role"] == "system"), None)
            users = [m["content"] for m in msgs if m["role"] == "user"]
            asst = [m.get("content") or "" for m in msgs if m["role"] == "assistant"]
            if users and asst:
                out.append(ChatExample(users[-1], asst[-1], sys_))
        elif "prompt" in r:
            out.append(ChatExample(r["prompt"], r.get("response", r.get("completion", "")), r.get("system")))
        elif "user" in r:
            out.append(ChatExample(r["user"], r.get("assistant", ""), r.get("system")))
    return out


_TOOL_RE = re.compile(r"<tool_call>\s*(\{.*?\})\s*</tool_call>", re.S)
_THINK_RE = re.compile(r"<think>(.*?)</think>\s*", re.S)


def split_reasoning(text: str) -> Tuple[Optional[str], str]:
    """(reasoning, visible) — the content of a leading ``<think>`` block and the remainder."""
    m = _THINK_RE.search(text)
    if m:
        return m.group(1).strip() or None, (text[:m.start()] + text[m.end():]).strip()
    if "</think>" in text:      # the template opened the block for us
        r, rest = text.split("</think>", 1)
        return r.strip() or None, rest.strip()
    return None, text


class ReasoningStream:
    """Streaming counterpart of :func:`split_reasoning`: text pieces go in, (kind, text) pairs come
    out with kind ``"reasoning"`` inside a ``<think>`` block and ``"token"`` outside; the markers
    themselves are dropped.  A piece that ends in what may be the start of a marker is held until
    the next piece decides it."""

    OPEN, CLOSE = "<think>", "</think>"

    def __init__(self):
        self.inside = False
        self.held = ""

    def feed(self, piece: str) -> List[Tuple[str, str]]:
        out: List[Tuple[str, str]] = []
        text = self.held + piece
        self.held = ""
        while text:
            marker = self.CLOSE if self.inside else self.OPEN
            k = text.find(marker)
            if k < 0:
                # keep a possible marker prefix at the end for the next piece
                hold = next((n for n in range(min(len(marker) - 1, len(text)), 0, -1)
                             if text.endswith(marker[:n])), 0)
                if len(text) > hold:
                    out.append(("reasoning" if self.inside else "token", text[:len(text) - hold]))
                self.held = text[len(text) - hold:] if hold else ""
                break
            if k:
                out.append(("reasoning" if self.inside else "token", text[:k]))
            self.inside = not self.inside
            text = text[k + len(marker):]
        return out

    def flush(self) -> List[Tuple[str, str]]:
        held, self.held = self.held, ""
        return [("reasoning" if self.inside else "token", held)] if held else []


def parse_tool_calls(text: str) -> Tuple[List[Dict], str]:
    """All ``<tool_call>{json}</tool_call>`` blocks as ``{"name","arguments"}`` plus the text with
    the blocks removed."""
    calls = []
    for m in _TOOL_RE.finditer(text):
        try:
            obj = json.loads(m.group(1))
        except json.JSONDecodeError:
            continue
        if isinstance(obj, dict) and "name" in obj:
            calls.append({"name": obj["name"], "arguments": obj.get("arguments", {})})
    return calls, _TOOL_RE.sub("", text).strip()
