"""Command resolution (reference: crates/cli/src/resolve.rs:143-192): the first token that names a
known architecture selects its handler and everything else becomes that handler's argv, so
``brain train qwen3 data/`` and ``brain qwen3 train data/`` are the same command.  ``import <FILE>``
and ``quantize <SRC>`` are the two file-first exceptions."""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

from .. import arch as archs


@dataclass
class Resolved:
    kind: str                  # 'arch' | 'import' | 'quantize' | 'unknown' | 'empty'
    arch: Optional[str] = None
    rest: Optional[List[str]] = None
    word: Optional[str] = None


def resolve(argv: List[str]) -> Resolved:
    if not argv:
        return Resolved("empty")
    first = argv[0]
    a = archs.by_id(first)
    if a is not None:
        return Resolved("arch", a.id, list(argv[1:]))
    if len(argv) > 1:
        b = archs.by_id(argv[1])
        if b is not None:
            return Resolved("arch", b.id, [first] + list(argv[2:]))
    if first == "import":
        return Resolved("import", rest=list(argv[1:]))
    if first == "quantize":
        return Resolved("quantize", rest=list(argv[1:]))
    return Resolved("unknown", word=first)
