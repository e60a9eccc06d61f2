"""Take-and-remove argument grammar shared by every model command (reference:
crates/cli/src/args.rs:14-99).  Each command pulls exactly the flags it knows; ``finish`` reports
whatever is left so unknown flags surface instead of being silently dropped."""
from __future__ import annotations

import sys
from typing import List, Optional

_VERB_ALIASES = {"gen": "infer", "sample": "infer", "generate": "infer", "fine-tune": "finetune"}


def canon_verb(v: Optional[str]) -> Optional[str]:
    return _VERB_ALIASES.get(v, v) if v is not None else None


class Args:
    def __init__(self, toks: List[str]):
        self.toks = list(toks)
        self.used = [False] * len(self.toks)

    def take_str(self, name: str) -> Optional[str]:
        for i, t in enumerate(self.toks):
            if not self.used[i] and t == name:
                self.used[i] = True
                if i + 1 < len(self.toks):
                    self.used[i + 1] = True
                    return self.toks[i + 1]
                print(f"{name} requires a value", file=sys.stderr)
                raise SystemExit(2)
        return None

    def take_all(self, name: str) -> List[str]:
        out = []
        while True:
            v = self.take_str(name)
            if v is None:
                return out
            out.append(v)

    def str_or(self, name: str, default: str) -> str:
        v = self.take_str(name)
        return default if v is None else v

    def _num(self, name, default, conv):
        v = self.take_str(name)
        if v is None:
            return default
        try:
            return conv(v)
        except ValueError:
            return default

    def int_or(self, name: str, default: int) -> int:
        return self._num(name, default, int)

    def float_or(self, name: str, default: float) -> float:
        return self._num(name, default, float)

    def opt_int(self, name: str) -> Optional[int]:
        return self._num(name, None, int)

    def char_opt(self, name: str) -> Optional[str]:
        v = self.take_str(name)
        return v[0] if v else None

    def take_flag(self, name: str) -> bool:
        for i, t in enumerate(self.toks):
            if not self.used[i] and t == name:
                self.used[i] = True
                return True
        return False

    def positional(self) -> Optional[str]:
        for i, t in enumerate(self.toks):
            if not self.used[i] and not t.startswith("--"):
                self.used[i] = True
                return t
        return None

    def leftover(self) -> List[str]:
        return [t for t, u in zip(self.toks, self.used) if not u]

    def finish(self) -> None:
        extra = self.leftover()
        if extra:
            print(f"ignoring unrecognised args: {extra}", file=sys.stderr)
