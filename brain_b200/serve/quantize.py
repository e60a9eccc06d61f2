"""Checkpoint quantisation for serving (reference: ``brain quantize``, crates/cli/src/quantize_cli.rs
and crates/checkpoint/src/quantize.rs — each tensor's fate is decided from its shape plus an explicit
``keep`` list, and the printed plan states the decision per tensor).

Output format: a safetensors file whose large 2-D projection weights are stored as ``<name>.q8``
(I8, per-output-row symmetric, ``[numel]``) with ``<name>.scale`` (F32 ``[rows]``); everything else
is copied as BF16.  ``load_quantized`` rebuilds the model with dequantised weights (the serving
engine re-quantises per row to the same int8 values, so W8A8 serving is bit-identical to quantising
the original)."""
from __future__ import annotations

import json
from typing import Dict, Iterable, List, Optional, Tuple

import torch

from ..checkpoint import st

MIN_NUMEL = 1 << 12


def plan(names_shapes: Iterable[Tuple[str, int]], rows_of: Dict[str, int], keep: Iterable[str] = ()) -> List[Tuple[str, str]]:
    """[(name, 'q8'|'bf16')] — quantise a tensor when it is a projection weight with a known row
    count, large enough to matter, and not matched by a ``keep`` fragment; embeddings, norms, biases
    and the LM head stay bf16."""
    keep = list(keep)
    out = []
    for name, numel in names_shapes:
        structural = (name.endswith(".weight") and name in rows_of and numel >= MIN_NUMEL
                      and not any(t in name for t in ("tok.", "token_emb", "lm_head", "norm", "ln1", "ln2", "router")))
        out.append((name, "q8" if structural and not any(k in name for k in keep) else "bf16"))
    return out


def _rows(config: dict) -> Dict[str, int]:
    """Output-row count of every linear weight, from the model the config describes."""
    from ..models import build_from_config
    model = build_from_config(config)
    return {n: t.shape[0] for n, t in model.reference_state().items() if t.dim() == 2}


def quantize_checkpoint(src: str, out: str, keep: Iterable[str] = (), verbose: bool = False) -> Dict:
    with st.WeightReader(src) as r:
        config = r.config()
        if config is None:
            raise ValueError(f"{src}: no model config in the metadata")
        rows = _rows(config)
        names = r.names()
        numels = {}
        for n in names:
            k = 1
            for s in r.shape(n):
                k *= s
            numels[n] = k
        decisions = plan([(n, numels[n]) for n in names], rows, keep)
        specs = []
        for n, d in decisions:
            if d == "q8":
                specs += [(n + ".q8", (numels[n],), "I8"), (n + ".scale", (rows[n],), "F32")]
            else:
                specs.append((n, (numels[n],), "BF16"))
        meta = dict(r.metadata)
        meta["brain.quant"] = json.dumps({"scheme": "w8-per-row-symmetric", "tensors": [n for n, d in decisions if d == "q8"]})
        w = st.StWriter(out, specs, meta)
        bytes_in = bytes_out = n_q = 0
        try:
            for n, d in decisions:
                t = r.read(n).reshape(-1)
                bytes_in += t.numel() * 4
                if d == "q8":
                    m = t.view(rows[n], -1)
                    scale = m.abs().amax(dim=1).clamp_min(1e-12) / 127.0
                    q = torch.clamp(torch.round(m / scale[:, None]), -127, 127).to(torch.int8)
                    w.write(n + ".q8", q)
                    w.write(n + ".scale", scale)
                    bytes_out += q.numel() + 4 * scale.numel()
                    n_q += 1
                else:
                    w.write(n, t)
                    bytes_out += 2 * t.numel()
                if verbose:
                    print(f"{d:>5}  {n}  [{numels[n]}]")
        except BaseException:
            w.close(abort=True)
            raise
        w.close()
    return {"tensors": n_q, "bytes_in": bytes_in, "bytes_out": bytes_out, "plan": decisions}


def load_quantized(path: str, device="cpu", dtype=None):
    """Model with dequantised weights from a file written by :func:`quantize_checkpoint`."""
    from ..models import build_from_config
    with st.WeightReader(path) as r:
        config = r.config()
        model = build_from_config(config)
        state = {}
        names = set(r.names())
        for n in model.reference_state():
            if n in names:
                state[n] = r.read(n)
            elif n + ".q8" in names:
                q = r.read(n + ".q8").float()
                s = r.read(n + ".scale")
                state[n] = (q.view(s.numel(), -1) * s[:, None]).reshape(-1)
        model.load_reference_state(state, strict=True)
    if device != "cpu" or dtype is not None:
        model = model.to(device=device, dtype=dtype)
    return model


# ------------------------------------------------------------------------------------ 4-bit storage
def quantize_weight_q4(w: torch.Tensor):
    """Per-output-row symmetric 4-bit storage: ``w`` [n, k] (k % 8 == 0) -> (int32 words [n, k/8]
    holding 8 two's-complement nibbles each, element b of a group in bits 4b..4b+3; fp32 row scales
    ``max(|row|, 1e-8) / 7``), values clamped to ±7 (reference: crates/model/src/int4.rs:46-73).
    A storage format here: weights are dequantised (to bf16 / int8) when loaded."""
    n, k = w.shape
    if k % 8:
        raise ValueError(f"q4 K must be a multiple of 8 (got {k})")
    wf = w.detach().float()
    sw = wf.abs().amax(dim=1).clamp_min(1e-8) / 7.0
    q = torch.clamp(torch.round(wf / sw[:, None]), -7, 7).to(torch.int64) & 0xF
    shifts = (4 * torch.arange(8, dtype=torch.int64))[None, None, :]
    words = (q.view(n, k // 8, 8) << shifts).sum(dim=-1)
    words = torch.where(words >= (1 << 31), words - (1 << 32), words)      # as signed 32-bit
    return words.to(torch.int32), sw


def dequantize_weight_q4(words: torch.Tensor, sw: torch.Tensor) -> torch.Tensor:
    """Inverse of :func:`quantize_weight_q4`; every nibble is SIGN-extended (bit 3 set = negative)."""
    n, kg = words.shape
    u = words.to(torch.int64) & 0xFFFFFFFF
    shifts = (4 * torch.arange(8, dtype=torch.int64))[None, None, :]
    nib = (u[:, :, None] >> shifts) & 0xF
    nib = torch.where(nib >= 8, nib - 16, nib)
    return nib.reshape(n, kg * 8).float() * sw.float()[:, None]
