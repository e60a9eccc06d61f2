"""Model reference grammar and the on-disk store (crates/modelref/src/lib.rs tests: quant suffix
set, dtype tokens stay in the repo name, two quants, traversal; crates/modelstore layout)."""
import os

import pytest
import torch

from brain_b200.modelref import ModelRef, RefError, canonical
from brain_b200.modelstore import Store, default_root


def test_parse_and_roundtrip():
    r = ModelRef.parse("Qwen/Qwen3-0.6B")
    assert (r.vendor, r.repo, r.quant, r.adapter) == ("Qwen", "Qwen3-0.6B", None, None)
    r = ModelRef.parse("Qwen/Qwen3-0.6B-Q4_K_M")
    assert r.repo == "Qwen3-0.6B" and r.quant == "Q4_K_M" and str(r) == "Qwen/Qwen3-0.6B-Q4_K_M"
    r = ModelRef.parse("nvidia/NVIDIA-Nemotron-3-Nano-30B-A3B-BF16-Q8_0")
    assert r.repo == "NVIDIA-Nemotron-3-Nano-30B-A3B-BF16" and r.quant == "Q8_0"
    assert ModelRef.parse("x/y-q8_0").quant is None            # lower case is part of the name
    assert ModelRef.parse("x/y-BF16").quant is None            # a dtype, not a quantisation
    r = ModelRef.parse("Qwen/Qwen3-0.6B-Q8_0:me:calc:v1")
    assert r.quant == "Q8_0" and (r.adapter.owner, r.adapter.name, r.adapter.tag) == ("me", "calc", "v1")
    assert ModelRef.parse(str(r)) == r and r.without_adapter() == ModelRef("Qwen", "Qwen3-0.6B", "Q8_0")
    assert ModelRef.parse("brain/mock").is_reserved() and not ModelRef.parse("Qwen/x").is_reserved()


@pytest.mark.parametrize("text,kind", [
    ("", "NoVendor"), ("qwen", "NoVendor"), ("/x", "EmptySegment"), ("x/", "EmptySegment"),
    ("a/b/c", "TooManySegments"), ("a/b c", "BadChar"), ("a/b-Q8_0-Q4_0", "TwoQuants"),
    ("../x", "PathTraversal"), ("x/..", "PathTraversal"), ("a/b:o:n", "BadAdapter"), ("a/b:o::t", "BadAdapter"),
    ("a/b:..:n:t", "PathTraversal"), ("a/:o:n:t", "EmptySegment"),
])
def test_parse_errors(text, kind):
    with pytest.raises(RefError) as e:
        ModelRef.parse(text)
    assert e.value.kind == kind


def test_aliases():
    assert canonical("mock") == "brain/mock" and canonical("qwen") == "brain/qwen3"
    assert canonical("Qwen/Qwen3-0.6B") == "Qwen/Qwen3-0.6B" and canonical("nope") == "nope"


def test_default_root_precedence(monkeypatch, tmp_path):
    for k in ("BRAIN_MODELS_DIR", "XDG_DATA_HOME", "HOME"):
        monkeypatch.delenv(k, raising=False)
    assert default_root() is None
    monkeypatch.setenv("HOME", "/h")
    assert default_root() == "/h/.local/share/brain/models"
    monkeypatch.setenv("XDG_DATA_HOME", "/x")
    assert default_root() == "/x/brain/models"
    monkeypatch.setenv("BRAIN_MODELS_DIR", "/m")
    assert default_root() == "/m" and default_root("/flag") == "/flag"


def test_store_install_local_scan_and_serve(tmp_path, monkeypatch):
    from brain_b200.checkpoint import st
    from brain_b200.models.config import LoraCfg, QwenConfig
    from brain_b200.models.lora import attach_lora, save_adapter
    from brain_b200.models.qwen3 import Qwen3
    cfg = QwenConfig(vocab=264, block_size=64, n_layers=1, d_model=32, n_heads=4, n_kv_heads=2, head_dim=8, d_ff=64)
    m = Qwen3(cfg).init_weights(1)
    w = str(tmp_path / "w.safetensors")
    st.save_model(w, m)
    store = Store(str(tmp_path / "models"))
    ref = ModelRef.parse("local/tiny")
    assert store.local(ref) is None and store.scan() == []
    lm = store.install(ref, w)
    assert lm.weights.endswith("local/tiny/model.brain.safetensors") and lm.tokenizer is None
    assert lm.card is not None and lm.card.family == "qwen"
    assert store.local(ModelRef.parse("local/tiny-Q8_0")) is None       # GGUF variants are not read
    aref = ref.with_adapter("me", "calc", "v1")
    assert store.adapter_weights_path(aref).endswith("local/tiny/adapters/me/calc/v1/adapter.brain.safetensors")
    assert store.local(aref) is None
    attach_lora(m, LoraCfg(rank=2, alpha=4.0))
    with torch.no_grad():
        for n, p in m.named_parameters():
            if "lora_b" in n:
                p.normal_(0, 0.05)
    os.makedirs(os.path.dirname(store.adapter_weights_path(aref)))
    save_adapter(store.adapter_weights_path(aref), m, base_id="local/tiny")
    assert store.local(aref).adapter == store.adapter_weights_path(aref)
    assert [str(x.reference) for x in store.scan()] == ["local/tiny", "local/tiny:me:calc:v1"]

    # the serving registry resolves BRAIN_MODEL through the store (and refuses what is not on disk)
    from brain_b200.api.resident import resolve_env_model
    monkeypatch.delenv("BRAIN_QWEN_WEIGHTS", raising=False)
    monkeypatch.setenv("BRAIN_MODELS_DIR", store.root)
    monkeypatch.setenv("BRAIN_MODEL", "local/tiny:me:calc:v1")
    wts, tok, adapter, sid = resolve_env_model()
    assert wts == lm.weights and adapter == store.adapter_weights_path(aref) and sid == "local/tiny:me:calc:v1"
    monkeypatch.setenv("BRAIN_MODEL", "Qwen/Qwen3-0.6B")
    with pytest.raises(FileNotFoundError):
        resolve_env_model()
