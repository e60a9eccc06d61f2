"""GGUF container and codecs: block decoders against the ``gguf`` library (including k-quant blocks
built from random bytes), the two encoders bit for bit, reader/writer against the library's reader,
a tiny Qwen3 through export -> import (same logits), any-container quantisation with its stated
reasons, and the ``.pt`` source."""
import numpy as np
import pytest
import torch

from brain_b200.checkpoint import convert, gguf as G, st
from brain_b200.models.config import QwenConfig
from brain_b200.models.qwen3 import Qwen3

lib = pytest.importorskip("gguf")


@pytest.mark.parametrize("name", ["Q8_0", "Q4_0", "Q4_1", "Q5_0", "Q5_1", "Q4_K", "Q5_K", "Q6_K", "F16", "BF16"])
def test_block_decoders_match_the_library(name):
    rng = np.random.default_rng(hash(name) & 0xFFFF)
    qt = getattr(lib.GGMLQuantizationType, name)
    _, be, bb = G.TYPES[G.TYPE_BY_NAME[name]]
    nb = 24
    raw = rng.integers(0, 256, (nb, bb), dtype=np.uint8)
    # every fp16 field of a block must be a finite number: overwrite them with valid halves
    halves = {"Q8_0": [0], "Q4_0": [0], "Q4_1": [0, 2], "Q5_0": [0], "Q5_1": [0, 2], "Q4_K": [0, 2], "Q5_K": [0, 2],
              "Q6_K": [208]}.get(name, [])
    for off in halves:
        raw[:, off:off + 2] = rng.uniform(-2, 2, nb).astype(np.float16).view(np.uint8).reshape(nb, 2)
    if name in ("F16", "BF16"):
        raw = rng.standard_normal(nb * 8).astype(np.float32).astype(np.float16).view(np.uint8).reshape(nb, -1) \
            if name == "F16" else (rng.standard_normal(nb * 8).astype(np.float32).view(np.uint32) >> 16).astype(np.uint16).view(np.uint8).reshape(nb, -1)
    want = lib.quants.dequantize(raw.reshape(nb, -1), qt).reshape(-1)
    got = G.dequantize(raw.reshape(-1), G.TYPE_BY_NAME[name], want.size)
    assert np.allclose(got, want, rtol=1e-6, atol=1e-6)


@pytest.mark.parametrize("name", ["Q8_0", "Q4_0"])
def test_encoders_are_bit_identical_to_the_library(name):
    x = np.random.default_rng(1).standard_normal((16, 256)).astype(np.float32)
    x[3] = 0.0                                                   # an all-zero block row
    want = np.ascontiguousarray(lib.quants.quantize(x, getattr(lib.GGMLQuantizationType, name))).reshape(-1).view(np.uint8)
    assert np.array_equal(G.quantize(x, G.TYPE_BY_NAME[name]), want)


def test_writer_is_read_by_the_library_and_reader_reads_it_back(tmp_path):
    rng = np.random.default_rng(2)
    a = rng.standard_normal((6, 64)).astype(np.float32)
    b = rng.standard_normal(10).astype(np.float32)
    p = str(tmp_path / "t.gguf")
    G.write_gguf(p, {"general.architecture": "qwen3", "x.count": 7, "x.scale": 0.5, "x.names": ["a", "b"], "x.flag": True},
                 [("a.weight", a.shape, G.T_Q8_0, G.quantize(a, G.T_Q8_0)), ("b", b.shape, G.T_F32, G.quantize(b, G.T_F32))])
    theirs = lib.GGUFReader(p)
    names = [t.name for t in theirs.tensors]
    assert names == ["a.weight", "b"]
    assert list(theirs.tensors[0].shape) == [64, 6]             # fastest dimension first in the file
    with G.GgufReader(p) as r:
        assert r.metadata["x.count"] == 7 and r.metadata["x.names"] == ["a", "b"] and r.metadata["x.flag"] is True
        assert abs(r.metadata["x.scale"] - 0.5) < 1e-7
        assert r.tensors["a.weight"].shape == (6, 64) and r.tensors["a.weight"].type_name == "Q8_0"
        assert np.array_equal(r.read("b"), b)
        assert np.abs(r.read("a.weight") - a).max() < np.abs(a).max() / 100
    with open(p, "r+b") as f:                                     # a truncated file is refused, not read short
        f.truncate(200)
    with pytest.raises(ValueError):
        G.GgufReader(p)


def _tiny():
    cfg = QwenConfig(vocab=96, block_size=32, n_layers=2, d_model=64, n_heads=4, n_kv_heads=2, head_dim=16, d_ff=128)
    return cfg, Qwen3(cfg).init_weights(3)


def test_qwen_roundtrip_through_gguf_and_quantized_tiers(tmp_path):
    cfg, m = _tiny()
    src = str(tmp_path / "q.safetensors")
    st.save_model(src, m)
    x = torch.randint(0, cfg.vocab, (2, 16), dtype=torch.int32)
    want = m(x)
    f16 = str(tmp_path / "q.f16.gguf")
    convert.export_gguf(src, f16)
    back = str(tmp_path / "back.safetensors")
    cfg2 = convert.import_gguf_qwen(f16, back)
    assert cfg2.to_json() == cfg.to_json()
    m2, _, _ = st.load_model(back)
    assert float((m2(x) - want).abs().max()) < 2e-2              # matrices went through fp16
    for tier, tol in (("Q8_0", 0.05), ("Q4_0", 0.6)):
        q = str(tmp_path / f"q.{tier}.gguf")
        info = convert.export_gguf(src, q, tier)
        assert info["quantized"] >= 10                            # the projections above the size floor
        convert.import_gguf_qwen(q, back)
        m3, _, _ = st.load_model(back)
        assert float((m3(x) - want).abs().max()) < tol * float(want.abs().max())


def test_quantize_any_container_states_why_a_tensor_is_kept(tmp_path):
    sd = {"w.big": torch.randn(64, 128), "w.odd": torch.randn(64, 100), "w.small": torch.randn(4, 32),
          "bias": torch.randn(128), "keepme.weight": torch.randn(64, 128)}
    pt = str(tmp_path / "m.pt")
    torch.save({"state_dict": sd}, pt)
    out = str(tmp_path / "m.gguf")
    info = convert.quantize_to_gguf(pt, out, "Q8_0", keep=["keepme"])
    plan = {n: d for n, _, d in info["plan"]}
    assert plan["w.big"] == "Q8_0"
    assert "whole number of 32-element blocks" in plan["w.odd"]
    assert "too small" in plan["w.small"] and "not a matrix" in plan["bias"] and "keep pattern" in plan["keepme.weight"]
    with G.GgufReader(out) as r:
        assert r.tensors["w.big"].type_name == "Q8_0" and r.tensors["bias"].type_name == "F16"
        assert np.abs(r.read("w.big") - sd["w.big"].numpy()).max() < 0.05
    # GGUF in, GGUF out at another tier
    out4 = str(tmp_path / "m4.gguf")
    convert.quantize_to_gguf(out, out4, "Q4_0")
    with G.GgufReader(out4) as r:
        assert r.tensors["w.big"].type_name == "Q4_0"
