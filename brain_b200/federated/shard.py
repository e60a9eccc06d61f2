"""Expert-shard layout with a SHA-256 manifest (reference: crates/federated/src/shard.rs:30-40
``expert_id`` name rule, :40-80 manifest ``{base_config_sha256, experts, files}``, :87-173 split,
:175-191 verify, :193-227 merge, :229-300 assemble with overlays replacing the base's experts).

Directory: ``shared.safetensors`` (every non-expert tensor, carries the config/card metadata),
``experts/expert_<E>.safetensors`` (all layers' tensors of expert E), ``manifest.json``."""
from __future__ import annotations

import hashlib
import json
import os
from dataclasses import dataclass, field
from pathlib import Path
from typing import Dict, Iterable, List, Optional, Sequence

from ..checkpoint import st

SHARED = "shared.safetensors"


def expert_id(name: str) -> Optional[int]:
    """``blocks.<L>.moe.experts.<E>.…`` -> E; None for shared tensors."""
    parts = name.split(".")
    if len(parts) >= 6 and parts[0] == "blocks" and parts[2] == "moe" and parts[3] == "experts" and parts[4].isdigit():
        return int(parts[4])
    return None


def config_hash(config: dict) -> str:
    return hashlib.sha256(json.dumps(config, separators=(",", ":")).encode()).hexdigest()


def file_hash(path) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for chunk in iter(lambda: f.read(1 << 22), b""):
            h.update(chunk)
    return h.hexdigest()


@dataclass
class Manifest:
    base_config_sha256: str
    experts: List[int] = field(default_factory=list)
    files: Dict[str, str] = field(default_factory=dict)

    def to_json(self) -> str:
        return json.dumps({"base_config_sha256": self.base_config_sha256, "experts": self.experts,
                           "files": dict(sorted(self.files.items()))})

    @staticmethod
    def from_json(s: str) -> "Manifest":
        v = json.loads(s)
        if not isinstance(v.get("base_config_sha256"), str) or not isinstance(v.get("experts"), list):
            raise ValueError("manifest: missing base_config_sha256 / experts")
        return Manifest(v["base_config_sha256"], [int(e) for e in v["experts"]], dict(v.get("files") or {}))

    @staticmethod
    def load(d) -> "Manifest":
        return Manifest.from_json((Path(d) / "manifest.json").read_text())


def _expert_file(e: int) -> str:
    return f"experts/expert_{e}.safetensors"


def split_filtered(base_weights: str, out_dir, keep: Optional[Sequence[int]] = None) -> Manifest:
    """Write the shared file (only for a full split) and the kept expert shards, one tensor in
    memory at a time."""
    out = Path(out_dir)
    (out / "experts").mkdir(parents=True, exist_ok=True)
    with st.WeightReader(base_weights) as r:
        config = r.config() or {}
        meta = dict(r.metadata)
        shared, experts = [], {}
        for n in r.names():
            e = expert_id(n)
            if e is None:
                shared.append(n)
            elif keep is None or e in keep:
                experts.setdefault(e, []).append(n)
        m = Manifest(config_hash(config), sorted(experts))

        def write(rel: str, names: List[str], metadata: Dict[str, str]):
            w = st.StWriter(str(out / rel), [(n, r.shape(n)) for n in names], metadata)
            try:
                for n in names:
                    w.write(n, r.read(n))
            except BaseException:
                w.close(abort=True)
                raise
            w.close()
            m.files[rel] = file_hash(out / rel)
        if keep is None:
            write(SHARED, shared, meta)
        for e, names in sorted(experts.items()):
            write(_expert_file(e), names, {"expert": str(e), "base_config_sha256": m.base_config_sha256})
    (out / "manifest.json").write_text(m.to_json())
    return m


def split(base_weights: str, out_dir) -> Manifest:
    return split_filtered(base_weights, out_dir, None)


def verify(d) -> Manifest:
    d = Path(d)
    m = Manifest.load(d)
    for rel, want in m.files.items():
        p = d / rel
        if not p.exists():
            raise IOError(f"{d}: missing {rel}")
        got = file_hash(p)
        if got != want:
            raise IOError(f"{d}: {rel} hash mismatch (manifest {want[:16]}…, file {got[:16]}…)")
    for e in m.experts:
        if _expert_file(e) not in m.files:
            raise IOError(f"{d}: expert {e} is listed but has no shard file")
    if SHARED in m.files:
        with st.WeightReader(str(d / SHARED)) as r:
            if config_hash(r.config() or {}) != m.base_config_sha256:
                raise IOError(f"{d}: shared file's config does not match base_config_sha256")
    return m


def _write_full(shared_path: str, expert_paths: Dict[int, str], out_weights: str) -> None:
    """Canonical order = the model's ``param_list`` order, recovered from the config."""
    from ..models import build_from_config
    with st.WeightReader(shared_path) as sh:
        config = sh.config()
        meta = dict(sh.metadata)
        readers = {e: st.WeightReader(p) for e, p in expert_paths.items()}
        try:
            have = {n: sh for n in sh.names()}
            for r in readers.values():
                for n in r.names():
                    have[n] = r
            model = build_from_config(config)
            order = [n for n in model.reference_state() if n in have]
            missing = [n for n in model.reference_state() if n not in have]
            if missing:
                raise IOError(f"cannot assemble: {len(missing)} tensors missing (first: {missing[0]})")
            w = st.StWriter(out_weights, [(n, have[n].shape(n)) for n in order], meta)
            try:
                for n in order:
                    w.write(n, have[n].read(n))
            except BaseException:
                w.close(abort=True)
                raise
            w.close()
        finally:
            for r in readers.values():
                r.close()


def merge_to_full(d, out_weights: str) -> None:
    d = Path(d)
    m = verify(d)
    if SHARED not in m.files:
        raise IOError(f"{d}: an overlay directory has no shared part; use assemble with a base directory")
    _write_full(str(d / SHARED), {e: str(d / _expert_file(e)) for e in m.experts}, out_weights)


def assemble(base_dir, overlays: Iterable, out_weights: str) -> None:
    """Base directory plus overlay directories (later overlays win); every overlay must have been
    split from a checkpoint with the same config."""
    base_dir = Path(base_dir)
    bm = verify(base_dir)
    if SHARED not in bm.files:
        raise IOError(f"{base_dir}: base directory has no shared part")
    experts = {e: str(base_dir / _expert_file(e)) for e in bm.experts}
    for ov in overlays:
        ov = Path(ov)
        om = verify(ov)
        if om.base_config_sha256 != bm.base_config_sha256:
            raise IOError(f"{ov}: overlay was made for a different base config")
        for e in om.experts:
            experts[e] = str(ov / _expert_file(e))
    _write_full(str(base_dir / SHARED), experts, out_weights)
