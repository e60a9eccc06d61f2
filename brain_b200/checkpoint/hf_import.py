"""Hugging Face Qwen2/Qwen3 directory -> framework checkpoint (reference:
crates/qwen3/src/import.rs:21-48 name mapping with no transposes, tied ``lm_head`` dropped;
``import_with_block`` optional context override).  Tensors are streamed one at a time through the
native safetensors reader/writer, so an import never holds more than one tensor on the host."""
from __future__ import annotations

import json
import os
from typing import Dict, Optional

import torch

from ..models.config import QwenConfig
from . import st
from .card import ModelCard

_LAYER = {
    "ln1.weight": "input_layernorm.weight",
    "ln2.weight": "post_attention_layernorm.weight",
    "attn.wq.weight": "self_attn.q_proj.weight", "attn.wq.bias": "self_attn.q_proj.bias",
    "attn.wk.weight": "self_attn.k_proj.weight", "attn.wk.bias": "self_attn.k_proj.bias",
    "attn.wv.weight": "self_attn.v_proj.weight", "attn.wv.bias": "self_attn.v_proj.bias",
    "attn.wo.weight": "self_attn.o_proj.weight",
    "attn.q_norm.weight": "self_attn.q_norm.weight", "attn.k_norm.weight": "self_attn.k_norm.weight",
    "mlp.gate.weight": "mlp.gate_proj.weight", "mlp.up.weight": "mlp.up_proj.weight",
    "mlp.down.weight": "mlp.down_proj.weight",
}


def hf_name(brain_name: str) -> str:
    """The Hugging Face tensor name that feeds a framework parameter name."""
    if brain_name == "tok.weight":
        return "model.embed_tokens.weight"
    if brain_name == "norm.weight":
        return "model.norm.weight"
    if brain_name == "lm_head.weight":
        return "lm_head.weight"
    parts = brain_name.split(".", 2)
    if parts[0] == "blocks" and parts[2] in _LAYER:
        return f"model.layers.{parts[1]}.{_LAYER[parts[2]]}"
    raise KeyError(brain_name)


def _rope_theta(hf: dict) -> float:
    """RoPE base of a Hugging Face config: top-level ``rope_theta`` (transformers 4) or
    ``rope_parameters.rope_theta`` (transformers 5).  Scaled variants (yarn, linear, dynamic, llama3)
    change every frequency; they are refused rather than imported with silently different logits."""
    rp = hf.get("rope_parameters") or hf.get("rope_scaling") or {}
    kind = rp.get("rope_type", rp.get("type", "default")) if isinstance(rp, dict) else "default"
    if kind not in (None, "default"):
        raise ValueError(f"RoPE scaling {kind!r} is not supported by this importer")
    theta = hf.get("rope_theta")
    if theta is None and isinstance(rp, dict):
        theta = rp.get("rope_theta")
    return float(theta if theta is not None else 1e6)


def config_from_hf(hf: dict, block: Optional[int] = None) -> QwenConfig:
    d = int(hf["hidden_size"])
    heads = int(hf["num_attention_heads"])
    mtype = hf.get("model_type", "qwen3")
    qwen2 = mtype == "qwen2"
    ctx = int(hf.get("max_position_embeddings", 32768))
    blk = int(block) if block else min(ctx, 4096)
    return QwenConfig(vocab=int(hf["vocab_size"]), block_size=blk, n_layers=int(hf["num_hidden_layers"]),
                      d_model=d, n_heads=heads, n_kv_heads=int(hf.get("num_key_value_heads", heads)),
                      head_dim=int(hf.get("head_dim", d // heads)), d_ff=int(hf["intermediate_size"]),
                      rope_theta=_rope_theta(hf), rms_eps=float(hf.get("rms_norm_eps", 1e-6)),
                      max_position_embeddings=ctx, tie_embeddings=bool(hf.get("tie_word_embeddings", False)),
                      qk_norm=not qwen2, attn_bias=bool(hf.get("attention_bias", qwen2)))


def _shard_index(hf_dir: str) -> Dict[str, str]:
    idx = os.path.join(hf_dir, "model.safetensors.index.json")
    if os.path.exists(idx):
        with open(idx) as f:
            return {k: os.path.join(hf_dir, v) for k, v in json.load(f)["weight_map"].items()}
    single = os.path.join(hf_dir, "model.safetensors")
    if not os.path.exists(single):
        raise FileNotFoundError(f"{hf_dir}: no model.safetensors or model.safetensors.index.json")
    with st.WeightReader(single) as r:
        return {n: single for n in r.names()}


def dequant_block(raw: torch.Tensor, scale_inv: torch.Tensor, block: int = 128) -> torch.Tensor:
    """Block-wise FP8 checkpoint weight -> fp32: ``raw`` [rows, cols] are the decoded E4M3 values and
    ``scale_inv`` [ceil(rows/block), ceil(cols/block)] the per-block multipliers (reference:
    crates/model/src/fp8.rs:29-76).  A shape mismatch is an error, never a silent broadcast."""
    rows, cols = raw.shape
    want = (-(-rows // block), -(-cols // block))
    if tuple(scale_inv.shape) != want:
        raise ValueError(f"scale grid {tuple(scale_inv.shape)} does not match weight {rows}x{cols} at block {block}")
    s = scale_inv.float().repeat_interleave(block, 0)[:rows].repeat_interleave(block, 1)[:, :cols]
    return raw.float() * s


def import_qwen(hf_dir: str, out: str, block: Optional[int] = None, dtype: str = "F32",
                model_id: Optional[str] = None) -> QwenConfig:
    with open(os.path.join(hf_dir, "config.json")) as f:
        hf = json.load(f)
    cfg = config_from_hf(hf, block)
    where = _shard_index(hf_dir)
    if cfg.tie_embeddings is False and "lm_head.weight" not in where:
        cfg.tie_embeddings = True        # some exports omit the flag but ship no separate head
    plist = cfg.param_list()
    card = ModelCard(id=model_id or "brain/qwen3", family="qwen", architecture=hf.get("model_type", "qwen3"),
                     param_count=sum(n for _, n in plist), context_length=cfg.max_position_embeddings,
                     capabilities=["generate", "chat"], source_repo=hf.get("_name_or_path") or None)
    meta = card.to_metadata()
    meta[st.CONFIG_KEY] = json.dumps(cfg.to_json(), separators=(",", ":"))
    w = st.StWriter(out, [(n, (k,)) for n, k in plist], meta, dtype)
    readers: Dict[str, st.WeightReader] = {}
    try:
        for name, numel in plist:
            src = hf_name(name)
            path = where.get(src)
            if path is None:
                raise KeyError(f"{hf_dir}: tensor {src} (for {name}) not found")
            r = readers.get(path)
            if r is None:
                r = readers[path] = st.WeightReader(path)
            t = r.read(src)
            if r.dtype(src) == "F8_E4M3":
                # block-128 FP8 export: the multipliers ship as <name>_scale_inv (bf16)
                sname = src + "_scale_inv"
                spath = where.get(sname)
                if spath is None:
                    raise KeyError(f"{hf_dir}: {src} is FP8 but {sname} is missing")
                rs = readers.get(spath)
                if rs is None:
                    rs = readers[spath] = st.WeightReader(spath)
                blk = int((hf.get("quantization_config") or {}).get("weight_block_size", [128, 128])[0])
                t = dequant_block(t, rs.read(sname), blk)
            if t.numel() != numel:
                raise ValueError(f"{src}: {t.numel()} elements, config expects {numel}")
            w.write(name, t)
    except BaseException:
        w.close(abort=True)
        raise
    finally:
        for r in readers.values():
            r.close()
    w.close()
    return cfg


def moe_config_from_hf(hf: dict, block: Optional[int] = None):
    """``MoeConfig`` of a Hugging Face Qwen3-MoE ``config.json`` (every layer sparse)."""
    from ..models.config import MoeConfig
    if hf.get("mlp_only_layers") or int(hf.get("decoder_sparse_step", 1)) != 1:
        raise ValueError("mixed dense / sparse layer stacks are not supported by this importer")
    d = int(hf["hidden_size"])
    heads = int(hf["num_attention_heads"])
    ctx = int(hf.get("max_position_embeddings", 32768))
    return MoeConfig(family="qwen3_moe", vocab=int(hf["vocab_size"]), block_size=int(block) if block else min(ctx, 4096),
                     n_layers=int(hf["num_hidden_layers"]), d_model=d, n_heads=heads,
                     n_kv_heads=int(hf.get("num_key_value_heads", heads)), head_dim=int(hf.get("head_dim", d // heads)),
                     n_experts=int(hf["num_experts"] if "num_experts" in hf else hf["num_local_experts"]), top_k=int(hf["num_experts_per_tok"]),
                     d_ff=int(hf["moe_intermediate_size"]), rope_theta=_rope_theta(hf),
                     rms_eps=float(hf.get("rms_norm_eps", 1e-6)), aux_coef=float(hf.get("router_aux_loss_coef", 0.001)),
                     norm_topk_prob=bool(hf.get("norm_topk_prob", False)),
                     tie_embeddings=bool(hf.get("tie_word_embeddings", False)))


def import_qwen_moe(hf_dir: str, out: str, block: Optional[int] = None, dtype: str = "F32",
                    model_id: Optional[str] = None):
    """Hugging Face Qwen3-MoE directory -> framework checkpoint.  Attention, norms, embedding and
    head map like the dense model; the router is ``mlp.gate.weight``; experts are read either per
    expert (``mlp.experts.{e}.{gate,up,down}_proj.weight``, the published layout) or from the fused
    ``mlp.experts.gate_up_proj`` [E, 2·ff, d] / ``down_proj`` [E, d, ff] tensors newer transformers
    versions write.  Tensors stream through one at a time (a fused expert tensor is read once per
    layer and sliced)."""
    with open(os.path.join(hf_dir, "config.json")) as f:
        hf = json.load(f)
    cfg = moe_config_from_hf(hf, block)
    where = _shard_index(hf_dir)
    if not cfg.tie_embeddings and "lm_head.weight" not in where:
        cfg.tie_embeddings = True
    plist = cfg.param_list()
    card = ModelCard(id=model_id or "brain/qwen3moe", family="qwen_moe", architecture=hf.get("model_type", "qwen3_moe"),
                     param_count=sum(n for _, n in plist), context_length=int(hf.get("max_position_embeddings", 32768)),
                     capabilities=["generate", "chat"], source_repo=hf.get("_name_or_path") or None)
    meta = card.to_metadata()
    meta[st.CONFIG_KEY] = json.dumps(cfg.to_json(), separators=(",", ":"))
    w = st.StWriter(out, [(n, (k,)) for n, k in plist], meta, dtype)
    readers: Dict[str, st.WeightReader] = {}
    fused: Dict[str, torch.Tensor] = {}      # the current layer's fused expert tensors

    def read(src: str) -> torch.Tensor:
        path = where.get(src)
        if path is None:
            raise KeyError(f"{hf_dir}: tensor {src} not found")
        r = readers.get(path)
        if r is None:
            r = readers[path] = st.WeightReader(path)
        return r.read(src)

    ff, d, E = cfg.d_ff, cfg.d_model, cfg.n_experts
    try:
        for name, numel in plist:
            parts = name.split(".")
            if len(parts) > 3 and parts[2] == "moe":
                base = f"model.layers.{parts[1]}.mlp"
                if parts[3] == "router":
                    fused.clear()
                    t = read(f"{base}.gate.weight")
                else:
                    e, which = int(parts[4]), parts[5]
                    per = f"{base}.experts.{e}.{ {'w_gate': 'gate_proj', 'w_up': 'up_proj', 'w_down': 'down_proj'}[which]}.weight"
                    if per in where:
                        t = read(per)
                    else:
                        key = f"{base}.experts.down_proj" if which == "w_down" else f"{base}.experts.gate_up_proj"
                        if key not in fused:
                            fused[key] = read(key)
                        big = fused[key]
                        if which == "w_down":
                            t = big.reshape(E, d, ff)[e]
                        else:
                            gu = big.reshape(E, 2 * ff, d)[e]
                            t = gu[:ff] if which == "w_gate" else gu[ff:]
            else:
                t = read(hf_name(name))
            if t.numel() != numel:
                raise ValueError(f"{name}: {t.numel()} elements, config expects {numel}")
            w.write(name, t.contiguous())
    except BaseException:
        w.close(abort=True)
        raise
    finally:
        for r in readers.values():
            r.close()
    w.close()
    return cfg


def import_hf(hf_dir: str, out: str, block: Optional[int] = None, dtype: str = "F32",
              model_id: Optional[str] = None):
    """Import a Hugging Face directory by its ``model_type``: qwen2 / qwen3 (dense) or qwen3_moe."""
    with open(os.path.join(hf_dir, "config.json")) as f:
        kind = json.load(f).get("model_type", "qwen3")
    if kind in ("qwen3_moe", "qwen2_moe"):
        return import_qwen_moe(hf_dir, out, block, dtype, model_id)
    return import_qwen(hf_dir, out, block, dtype, model_id)


def export_hf(weights: str, out_dir: str, dtype: str = "BF16") -> None:
    """Inverse mapping: framework checkpoint -> ``config.json`` + ``model.safetensors`` with Hugging
    Face names and 2-D shapes (the reference's ``export`` targets an NPU graph format instead; this
    is the interchange export that makes sense on this hardware)."""
    with st.WeightReader(weights) as r:
        cfg = QwenConfig.from_json(r.config())
        shapes = {}
        for name, numel in cfg.param_list():
            if name.endswith(".weight") and numel not in (cfg.d_model, cfg.head_dim):
                inner = {"wq": cfg.d_model, "wk": cfg.d_model, "wv": cfg.d_model, "wo": cfg.q_dim,
                         "gate": cfg.d_model, "up": cfg.d_model, "down": cfg.d_ff}.get(
                             name.split(".")[-2], cfg.d_model)
                shapes[name] = (numel // inner, inner)
            else:
                shapes[name] = (numel,)
        os.makedirs(out_dir, exist_ok=True)
        hf_cfg = {"model_type": "qwen3" if cfg.qk_norm else "qwen2", "architectures":
                  ["Qwen3ForCausalLM" if cfg.qk_norm else "Qwen2ForCausalLM"],
                  "hidden_size": cfg.d_model, "num_attention_heads": cfg.n_heads,
                  "num_key_value_heads": cfg.n_kv_heads, "head_dim": cfg.head_dim,
                  "num_hidden_layers": cfg.n_layers, "intermediate_size": cfg.d_ff,
                  "vocab_size": cfg.vocab, "rope_theta": cfg.rope_theta, "rms_norm_eps": cfg.rms_eps,
                  "max_position_embeddings": cfg.max_position_embeddings,
                  "tie_word_embeddings": cfg.tie_embeddings, "attention_bias": cfg.attn_bias,
                  "torch_dtype": "bfloat16" if dtype == "BF16" else "float32"}
        with open(os.path.join(out_dir, "config.json"), "w") as f:
            json.dump(hf_cfg, f, indent=1)
        names = [n for n, _ in cfg.param_list() if ".lora_" not in n]
        w = st.StWriter(os.path.join(out_dir, "model.safetensors"),
                        [(hf_name(n), shapes[n]) for n in names], {"format": "pt"}, dtype)
        try:
            for n in names:
                w.write(hf_name(n), r.read(n))
        except BaseException:
            w.close(abort=True)
            raise
        w.close()
