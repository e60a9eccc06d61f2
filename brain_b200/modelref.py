"""Fully-qualified model references ``<vendor>/<repo>[-<QUANT>][:<owner>:<name>:<tag>]``
(reference: crates/modelref/src/lib.rs:100-260 grammar and checks, :345-440 the closed quant set,
crates/modelref/src/alias.rs legacy short names).

* Case is exact: the reference must equal the upstream URL byte for byte.
* ``QUANT`` is one of a closed, upper-case set; ``BF16``/``F16``/``F32``/``FP8`` are dtypes of the
  base repository and stay part of the repo name.  Two quant suffixes are an error.
* ``brain``, ``local`` and ``test`` are reserved vendors that never lead to a fetch.
* ``.`` / ``..`` segments are refused: vendor, repo and the adapter components become path
  components of the model store."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

QUANTS = ("Q4_0", "Q4_1", "Q5_0", "Q5_1", "Q8_0", "Q2_K", "Q3_K_S", "Q3_K_M", "Q3_K_L", "Q4_K_S", "Q4_K_M",
          "Q5_K_S", "Q5_K_M", "Q6_K", "Q8_K")
RESERVED_VENDORS = ("brain", "local", "test")

#: legacy short names accepted at the two places that resolve a client-supplied name
ALIASES = {"mock": "brain/mock", "qwen": "brain/qwen3", "gpt": "brain/gpt2", "gpt2": "brain/gpt2",
           "toymoe": "brain/toymoe"}


class RefError(ValueError):
    def __init__(self, kind: str, text: str):
        super().__init__(f"{kind}: {text!r}")
        self.kind = kind


@dataclass(frozen=True, order=True)
class AdapterRef:
    owner: str
    name: str
    tag: str


def _strip_quant(rest: str) -> Optional[Tuple[str, str]]:
    for q in QUANTS:
        suf = "-" + q
        if rest.endswith(suf) and len(rest) > len(suf):
            return rest[:-len(suf)], q
    return None


@dataclass(frozen=True, order=True)
class ModelRef:
    vendor: str
    repo: str
    quant: Optional[str] = None
    adapter: Optional[AdapterRef] = None

    @staticmethod
    def parse(s: str) -> "ModelRef":
        if not s or "/" not in s:
            raise RefError("NoVendor", s)
        vendor, rest = s.split("/", 1)
        if not vendor or not rest:
            raise RefError("EmptySegment", s)
        if "/" in rest:
            raise RefError("TooManySegments", s)
        if any(c.isspace() for c in s):
            raise RefError("BadChar", s)
        adapter = None
        if ":" in rest:
            rest, tail = rest.split(":", 1)
            segs = tail.split(":")
            if len(segs) != 3 or not all(segs):
                raise RefError("BadAdapter", s)
            if any(x in (".", "..") for x in segs):
                raise RefError("PathTraversal", s)
            adapter = AdapterRef(*segs)
        if not rest:
            raise RefError("EmptySegment", s)
        quant = None
        st = _strip_quant(rest)
        if st is not None:
            rest, quant = st
            if _strip_quant(rest) is not None:
                raise RefError("TwoQuants", s)
        if vendor in (".", "..") or rest in (".", ".."):
            raise RefError("PathTraversal", s)
        return ModelRef(vendor, rest, quant, adapter)

    def __str__(self) -> str:
        s = f"{self.vendor}/{self.repo}"
        if self.quant:
            s += "-" + self.quant
        if self.adapter:
            s += f":{self.adapter.owner}:{self.adapter.name}:{self.adapter.tag}"
        return s

    def base(self) -> "ModelRef":
        return ModelRef(self.vendor, self.repo)

    def without_adapter(self) -> "ModelRef":
        return ModelRef(self.vendor, self.repo, self.quant)

    def with_adapter(self, owner: str, name: str, tag: str = "latest") -> "ModelRef":
        return ModelRef(self.vendor, self.repo, self.quant, AdapterRef(owner, name, tag))

    def is_reserved(self) -> bool:
        return self.vendor in RESERVED_VENDORS


def canonical(name: str) -> str:
    """A client-supplied model name -> canonical id (legacy short names map through ``ALIASES``;
    anything else is returned unchanged for the normal not-found path to judge)."""
    return ALIASES.get(name, name)
