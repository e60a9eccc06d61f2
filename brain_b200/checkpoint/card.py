"""Model card carried in the checkpoint metadata (``brain.card``), field-for-field the reference's
``ModelCard`` / ``Adapter`` (crates/checkpoint/src/st.rs:53-109); ``None`` fields are omitted."""
from __future__ import annotations

import json
from dataclasses import dataclass, field, fields
from typing import Any, Dict, List, Optional

CARD_KEY = "brain.card"
CONFIG_KEY = "brain.config"


@dataclass
class Adapter:
    kind: str = "lora"
    rank: Optional[int] = None
    base: Optional[str] = None
    alpha: Optional[float] = None
    targets: Optional[List[str]] = None
    dataset_id: Optional[str] = None

    def to_json(self):
        return {k: v for k, v in self.__dict__.items() if v is not None}


@dataclass
class ModelCard:
    id: str = "brain/model"
    family: str = "qwen"
    schema_version: int = 1
    display_name: Optional[str] = None
    architecture: Optional[str] = None
    variant_of: Optional[str] = None
    adapter: Optional[Adapter] = None
    capabilities: List[str] = field(default_factory=list)
    modalities: Optional[Dict[str, List[str]]] = None
    context_length: Optional[int] = None
    param_count: Optional[int] = None
    license: Optional[str] = None
    created: Optional[int] = None
    owned_by: Optional[str] = None
    tokenizer: Optional[str] = None
    quant: Optional[str] = None
    embedding_dim: Optional[int] = None
    default_params: Optional[Any] = None
    vendor: Optional[str] = None
    repo: Optional[str] = None
    revision: Optional[str] = None
    source_repo: Optional[str] = None

    def to_json(self) -> dict:
        out = {"schema_version": self.schema_version, "id": self.id}
        for f in fields(self):
            if f.name in ("schema_version", "id"):
                continue
            v = getattr(self, f.name)
            if f.name == "capabilities":
                out[f.name] = list(v)
            elif v is None:
                continue
            elif f.name == "adapter":
                out[f.name] = v.to_json()
            else:
                out[f.name] = v
        return out

    @staticmethod
    def from_json(d: dict) -> "ModelCard":
        known = {f.name for f in fields(ModelCard)}
        kw = {k: v for k, v in d.items() if k in known}
        if isinstance(kw.get("adapter"), dict):
            ak = {f.name for f in fields(Adapter)}
            kw["adapter"] = Adapter(**{k: v for k, v in kw["adapter"].items() if k in ak})
        return ModelCard(**kw)

    def to_metadata(self) -> Dict[str, str]:
        """``brain.card`` is the source of truth; well-known scalars are mirrored as flat keys."""
        m = {CARD_KEY: json.dumps(self.to_json(), separators=(",", ":")), "id": self.id,
             "family": self.family}
        for k in ("architecture", "license", "vendor", "repo"):
            v = getattr(self, k)
            if v is not None:
                m[k] = v
        for k in ("param_count", "context_length"):
            v = getattr(self, k)
            if v is not None:
                m[k] = str(v)
        return m

    @staticmethod
    def from_metadata(meta: Dict[str, str]) -> Optional["ModelCard"]:
        raw = meta.get(CARD_KEY)
        if not raw:
            return None
        try:
            return ModelCard.from_json(json.loads(raw))
        except Exception:
            return None
