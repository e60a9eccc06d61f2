"""Conversions between checkpoint containers:

* ``import_gguf_qwen``  llama.cpp-style GGUF of a Qwen2/Qwen3 model -> framework safetensors
  (tensor names ``blk.N.attn_q.weight`` ..., hyper-parameters from the ``<arch>.*`` keys; Qwen uses
  NeoX rotary layout, which GGUF converters leave unpermuted, so rows map one to one)
* ``export_gguf``       framework checkpoint -> GGUF with the same naming, optionally block-quantised
* ``quantize_to_gguf``  ANY supported checkpoint (safetensors, ``.pt``, GGUF) -> GGUF at a tier; the
  plan names, for every tensor that stays unquantised, the reason (not a matrix / row not a whole
  number of blocks / too small / matched a keep pattern)
* ``read_torch_pt``     a ``torch.save`` archive (zip or legacy pickle) read with ``weights_only``

Reference: crates/checkpoint/src/quantize.rs:79-337 (tier, policy, per-tensor decision with a
reason), gguf.rs / gguf_write.rs, torchpt.rs (zip reader for ``.pt``); crates/gguf (architecture
importer seam)."""
from __future__ import annotations

import json
from typing import Dict, Iterable, Iterator, List, Optional, Tuple

import numpy as np
import torch

from . import gguf as G
from . import st
from .card import ModelCard

_GGUF_LAYER = {
    "ln1.weight": "attn_norm.weight", "ln2.weight": "ffn_norm.weight",
    "attn.wq.weight": "attn_q.weight", "attn.wq.bias": "attn_q.bias",
    "attn.wk.weight": "attn_k.weight", "attn.wk.bias": "attn_k.bias",
    "attn.wv.weight": "attn_v.weight", "attn.wv.bias": "attn_v.bias",
    "attn.wo.weight": "attn_output.weight",
    "attn.q_norm.weight": "attn_q_norm.weight", "attn.k_norm.weight": "attn_k_norm.weight",
    "mlp.gate.weight": "ffn_gate.weight", "mlp.up.weight": "ffn_up.weight", "mlp.down.weight": "ffn_down.weight",
}


def gguf_name(brain_name: str) -> str:
    """The GGUF tensor name of a framework parameter (dense Qwen family)."""
    top = {"tok.weight": "token_embd.weight", "norm.weight": "output_norm.weight", "lm_head.weight": "output.weight"}
    if brain_name in top:
        return top[brain_name]
    parts = brain_name.split(".", 2)
    if parts[0] == "blocks" and parts[2] in _GGUF_LAYER:
        return f"blk.{parts[1]}.{_GGUF_LAYER[parts[2]]}"
    raise KeyError(brain_name)


def config_from_gguf(meta: Dict[str, object], tensors: Dict[str, G.TensorInfo], block: Optional[int] = None):
    from ..models.config import QwenConfig
    arch = str(meta.get("general.architecture", "qwen3"))
    if arch not in ("qwen2", "qwen3"):
        raise ValueError(f"GGUF architecture {arch!r}: this importer reads the dense Qwen2 / Qwen3 family")

    def key(k, default=None):
        v = meta.get(f"{arch}.{k}", default)
        if v is None:
            raise KeyError(f"GGUF metadata lacks {arch}.{k}")
        return v
    d = int(key("embedding_length"))
    heads = int(key("attention.head_count"))
    kv = int(key("attention.head_count_kv", heads))
    hd = int(key("attention.key_length", d // heads))
    vocab = int(tensors["token_embd.weight"].shape[0])
    ctx = int(key("context_length", 4096))
    cfg = QwenConfig(vocab=vocab, block_size=int(block or min(ctx, 4096)), n_layers=int(key("block_count")),
                     d_model=d, n_heads=heads, n_kv_heads=kv, head_dim=hd, d_ff=int(key("feed_forward_length")))
    # GGUF stores these as float32: print-round them so 1e-6 does not come back as 9.99999997e-07
    cfg.rope_theta = float(f'{float(key("rope.freq_base", 1e6)):.7g}')
    cfg.rms_eps = float(f'{float(key("attention.layer_norm_rms_epsilon", 1e-6)):.7g}')
    cfg.max_position_embeddings = ctx
    cfg.tie_embeddings = "output.weight" not in tensors
    cfg.qk_norm = "blk.0.attn_q_norm.weight" in tensors
    cfg.attn_bias = "blk.0.attn_q.bias" in tensors
    return cfg


def import_gguf_qwen(src: str, out: str, block: Optional[int] = None, dtype: str = "F32",
                     model_id: Optional[str] = None):
    """Decode every tensor of a Qwen GGUF (any supported block type) into a framework checkpoint."""
    with G.GgufReader(src) as r:
        cfg = config_from_gguf(r.metadata, r.tensors, block)
        plist = cfg.param_list()
        card = ModelCard(id=model_id or "brain/qwen3", family="qwen",
                         architecture=str(r.metadata.get("general.architecture", "qwen3")),
                         param_count=sum(n for _, n in plist), context_length=cfg.max_position_embeddings,
                         capabilities=["generate", "chat"],
                         source_repo=str(r.metadata.get("general.name", "")) or None)
        meta = card.to_metadata()
        meta[st.CONFIG_KEY] = json.dumps(cfg.to_json(), separators=(",", ":"))
        w = st.StWriter(out, [(n, (k,)) for n, k in plist], meta, dtype)
        try:
            for name, numel in plist:
                g = gguf_name(name)
                if g not in r.tensors:
                    raise KeyError(f"{src}: tensor {g} (for {name}) not found")
                t = torch.from_numpy(np.ascontiguousarray(r.read(g)))
                if t.numel() != numel:
                    raise ValueError(f"{g}: {t.numel()} elements, config expects {numel}")
                w.write(name, t)
        except BaseException:
            w.close(abort=True)
            raise
        w.close()
    return cfg


# ------------------------------------------------------------------------------------ sources
def read_torch_pt(path: str) -> Dict[str, torch.Tensor]:
    """Tensors of a ``torch.save`` file (zip archive or legacy pickle), loaded with
    ``weights_only=True`` (no arbitrary code runs) and memory-mapped when the archive allows it.
    A wrapper dict with a ``state_dict`` / ``model`` entry is unwrapped."""
    try:
        obj = torch.load(path, map_location="cpu", weights_only=True, mmap=True)
    except (RuntimeError, ValueError):
        obj = torch.load(path, map_location="cpu", weights_only=True)
    for k in ("state_dict", "model", "module"):
        if isinstance(obj, dict) and isinstance(obj.get(k), dict):
            obj = obj[k]
    if not isinstance(obj, dict):
        raise ValueError(f"{path}: expected a state dict, got {type(obj).__name__}")
    return {str(k): v for k, v in obj.items() if isinstance(v, torch.Tensor)}


def iter_tensors(src: str) -> Iterator[Tuple[str, Tuple[int, ...], np.ndarray]]:
    """(name, shape, fp32 values) of every tensor of a checkpoint, one at a time, whatever the
    container: ``.safetensors``, ``.gguf``, ``.pt`` / ``.pth`` / ``.bin``."""
    low = src.lower()
    if low.endswith(".gguf"):
        with G.GgufReader(src) as r:
            for n, t in r.tensors.items():
                yield n, t.shape, r.read(n)
    elif low.endswith((".pt", ".pth", ".bin")):
        for n, t in read_torch_pt(src).items():
            yield n, tuple(t.shape), t.detach().float().contiguous().numpy()
    else:
        with st.WeightReader(src) as r:
            shapes = _true_shapes(r)
            for n in r.names():
                v = r.read(n).float().numpy()
                yield n, shapes.get(n, tuple(v.shape)), v


def _true_shapes(r: "st.WeightReader") -> Dict[str, Tuple[int, ...]]:
    """Framework checkpoints store every tensor flat; the matrix shapes come from the model the
    embedded config describes."""
    cfgj = r.config()
    if not cfgj:
        return {}
    try:
        from ..models import build_from_config
        return {n: tuple(t.shape) for n, t in build_from_config(cfgj).reference_state().items()}
    except Exception:
        return {}


# ------------------------------------------------------------------------------------ -> GGUF
MIN_QUANT_ELEMS = 1 << 12


def decide(name: str, shape: Tuple[int, ...], tier: str, keep: Iterable[str] = (),
           min_elems: int = MIN_QUANT_ELEMS) -> Tuple[bool, str]:
    """(quantise?, reason) for one tensor at a tier — every tensor that stays unquantised says why."""
    be = G.TYPES[G.TYPE_BY_NAME[tier]][1]
    numel = int(np.prod(shape)) if shape else 1
    if len(shape) != 2:
        return False, f"not a matrix (rank {len(shape)})"
    if shape[-1] % be:
        return False, f"row of {shape[-1]} is not a whole number of {be}-element blocks"
    if numel < min_elems:
        return False, f"too small ({numel} < {min_elems} elements)"
    for k in keep:
        if k in name:
            return False, f"matched keep pattern {k!r}"
    return True, tier


def quantize_to_gguf(src: str, out: str, tier: str = "Q8_0", keep: Iterable[str] = (),
                     keep_dtype: str = "F16", rename=None, metadata: Optional[Dict[str, object]] = None,
                     plan_only: bool = False) -> Dict:
    """Write every tensor of ``src`` into a GGUF file, matrices block-quantised at ``tier`` (Q8_0 or
    Q4_0), the rest as ``keep_dtype``.  Returns {'plan': [(name, shape, type or reason)], 'bytes_in',
    'bytes_out', 'quantized'}.  ``rename(name) -> name`` maps tensor names (framework -> GGUF)."""
    tier = tier.upper()
    if tier not in ("Q8_0", "Q4_0"):
        raise ValueError(f"tier {tier}: this build encodes Q8_0 and Q4_0")
    keep = list(keep)
    plan, tensors = [], []
    bytes_in = quantized = 0
    for name, shape, vals in iter_tensors(src):
        q, why = decide(name, shape, tier, keep)
        plan.append((name, shape, tier if q else f"{keep_dtype} ({why})"))
        bytes_in += vals.size * 4
        if plan_only:
            continue
        ttype = G.TYPE_BY_NAME[tier if q else keep_dtype]
        tensors.append((rename(name) if rename else name, tuple(shape) or (1,), ttype, G.quantize(vals, ttype)))
        quantized += int(q)
    info = {"plan": plan, "bytes_in": bytes_in, "bytes_out": 0, "quantized": quantized}
    if plan_only:
        return info
    meta = dict(metadata or {})
    meta.setdefault("general.quantization_version", 2)
    meta.setdefault("general.file_type", {"Q8_0": 7, "Q4_0": 2}[tier])
    info["bytes_out"] = G.write_gguf(out, meta, tensors)
    return info


def gguf_metadata_for(cfg, name: str = "brain") -> Dict[str, object]:
    """The ``<arch>.*`` keys a llama.cpp-style reader needs for a dense Qwen model."""
    arch = "qwen3" if cfg.qk_norm else "qwen2"
    return {
        "general.architecture": arch, "general.name": name,
        f"{arch}.block_count": int(cfg.n_layers), f"{arch}.embedding_length": int(cfg.d_model),
        f"{arch}.feed_forward_length": int(cfg.d_ff), f"{arch}.attention.head_count": int(cfg.n_heads),
        f"{arch}.attention.head_count_kv": int(cfg.n_kv_heads), f"{arch}.attention.key_length": int(cfg.head_dim),
        f"{arch}.attention.value_length": int(cfg.head_dim), f"{arch}.context_length": int(cfg.max_position_embeddings),
        f"{arch}.rope.freq_base": float(cfg.rope_theta),
        f"{arch}.attention.layer_norm_rms_epsilon": float(cfg.rms_eps),
    }


def export_gguf(weights: str, out: str, tier: Optional[str] = None, keep: Iterable[str] = ()) -> Dict:
    """Framework Qwen checkpoint -> GGUF with llama.cpp tensor names (and block quantisation when a
    tier is given; norms, biases and anything small stay F32/F16)."""
    from ..models.config import config_from_json
    with st.WeightReader(weights) as r:
        cfgj = r.config()
    if cfgj is None:
        raise ValueError(f"{weights}: no model config in the metadata")
    cfg = config_from_json(cfgj)
    meta = gguf_metadata_for(cfg)
    if tier is None:
        tensors = [(gguf_name(n), tuple(s), G.T_F32 if len(s) != 2 else G.T_F16,
                    G.quantize(v, G.T_F32 if len(s) != 2 else G.T_F16)) for n, s, v in iter_tensors(weights)]
        return {"bytes_out": G.write_gguf(out, meta, tensors), "quantized": 0}
    return quantize_to_gguf(weights, out, tier, keep=list(keep) + ["token_embd", "tok."], keep_dtype="F16",
                            rename=gguf_name, metadata=meta)
