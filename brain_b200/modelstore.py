"""On-disk model store ``<root>/<vendor>/<repo>/…`` (reference: crates/modelstore/src/lib.rs:100-330 —
root resolution, file names, ``local`` / ``scan``).  Nothing is fetched: a reference that is not on
disk is simply not found.

    <root>/<vendor>/<repo>/model.brain.safetensors                       base weights (brain format)
    <root>/<vendor>/<repo>/tokenizer.json
    <root>/<vendor>/<repo>/kv_calib.json                                 optional int8-KV ceilings
    <root>/<vendor>/<repo>/adapters/<owner>/<name>/<tag>/adapter.brain.safetensors
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import List, Optional

from .modelref import AdapterRef, ModelRef

BASE_WEIGHTS_FILE = "model.brain.safetensors"
TOKENIZER_FILE = "tokenizer.json"
ADAPTERS_DIR = "adapters"
ADAPTER_WEIGHTS_FILE = "adapter.brain.safetensors"


def default_root(flag: Optional[str] = None) -> Optional[str]:
    """``--models-dir`` flag, else BRAIN_MODELS_DIR, else $XDG_DATA_HOME/brain/models, else
    $HOME/.local/share/brain/models; None when none of them is set."""
    if flag:
        return flag
    if os.environ.get("BRAIN_MODELS_DIR"):
        return os.environ["BRAIN_MODELS_DIR"]
    if os.environ.get("XDG_DATA_HOME"):
        return os.path.join(os.environ["XDG_DATA_HOME"], "brain", "models")
    if os.environ.get("HOME"):
        return os.path.join(os.environ["HOME"], ".local", "share", "brain", "models")
    return None


@dataclass
class LocalModel:
    reference: ModelRef
    dir: str
    weights: str
    tokenizer: Optional[str]
    adapter: Optional[str] = None
    card: Optional[object] = None


class Store:
    def __init__(self, root: str):
        self.root = root

    def repo_dir(self, ref: ModelRef) -> str:
        return os.path.join(self.root, ref.vendor, ref.repo)

    def adapter_weights_path(self, ref: ModelRef) -> Optional[str]:
        a = ref.adapter
        if a is None:
            return None
        return os.path.join(self.repo_dir(ref), ADAPTERS_DIR, a.owner, a.name, a.tag, ADAPTER_WEIGHTS_FILE)

    def _card(self, path: str):
        try:
            from .checkpoint.st import WeightReader
            with WeightReader(path) as r:    # header only: no tensor is read
                return r.card()
        except Exception:   # noqa: BLE001 - an unreadable file is "not found", not an error
            return None

    def local(self, ref: ModelRef) -> Optional[LocalModel]:
        """The files of ``ref`` on disk, or None (missing base, missing adapter, or a quantised
        variant: GGUF files are not read by this build)."""
        if ref.quant is not None:
            return None
        d = self.repo_dir(ref)
        weights = os.path.join(d, BASE_WEIGHTS_FILE)
        if not os.path.isfile(weights):
            return None
        tok = os.path.join(d, TOKENIZER_FILE)
        tok = tok if os.path.isfile(tok) else None
        if ref.adapter is not None:
            ap = self.adapter_weights_path(ref)
            if not os.path.isfile(ap):
                return None
            return LocalModel(ref, d, weights, tok, ap, self._card(ap))
        return LocalModel(ref, d, weights, tok, None, self._card(weights))

    def scan(self) -> List[LocalModel]:
        """Every servable model on disk: one entry per base repo with weights, one per adapter."""
        out: List[LocalModel] = []
        if not os.path.isdir(self.root):
            return out
        for vendor in sorted(os.listdir(self.root)):
            vdir = os.path.join(self.root, vendor)
            if not os.path.isdir(vdir):
                continue
            for repo in sorted(os.listdir(vdir)):
                rdir = os.path.join(vdir, repo)
                if not os.path.isdir(rdir):
                    continue
                base = ModelRef(vendor, repo)
                m = self.local(base)
                if m is None:
                    continue
                out.append(m)
                adir = os.path.join(rdir, ADAPTERS_DIR)
                if not os.path.isdir(adir):
                    continue
                for owner in sorted(os.listdir(adir)):
                    for name in sorted(os.listdir(os.path.join(adir, owner))):
                        for tag in sorted(os.listdir(os.path.join(adir, owner, name))):
                            r = ModelRef(vendor, repo, None, AdapterRef(owner, name, tag))
                            am = self.local(r)
                            if am is not None:
                                out.append(am)
        return out

    def install(self, ref: ModelRef, weights: str, tokenizer: Optional[str] = None) -> LocalModel:
        """Place a brain-format checkpoint (and its tokenizer) into the store under ``ref``
        (hard link when possible, else copy)."""
        import shutil
        d = self.repo_dir(ref)
        os.makedirs(d, exist_ok=True)
        for src, name in ((weights, BASE_WEIGHTS_FILE), (tokenizer, TOKENIZER_FILE)):
            if not src:
                continue
            dst = os.path.join(d, name)
            if os.path.abspath(src) == os.path.abspath(dst):
                continue
            if os.path.exists(dst):
                os.remove(dst)
            try:
                os.link(src, dst)
            except OSError:
                shutil.copyfile(src, dst)
        return self.local(ref.base())
