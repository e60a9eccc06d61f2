"""Architecture registry: every model family the CLI grammar knows, whether this framework builds
it, and the capability verbs it exposes (reference: crates/arch/src/lib.rs — the id/family table the
CLI resolves against — and the ``ARCH_HANDLERS``/``ARCH_TO_MODEL`` tables of
crates/cli/src/resolve.rs:31-92)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional


@dataclass(frozen=True)
class Arch:
    id: str
    family: str
    summary: str
    verbs: tuple = ()
    built: bool = True
    model_id: Optional[str] = None
    aliases: tuple = ()


_ARCHS: List[Arch] = [
    Arch("gpt2", "gpt", "GPT-2 style decoder (LayerNorm, GELU, learned positions, untied head)",
         ("train", "infer", "eval"), aliases=("gpt",)),
    Arch("qwen3", "qwen", "Qwen3/Qwen2 decoder (RMSNorm, GQA, QK-norm, RoPE, SwiGLU)",
         ("import", "infer", "serve", "export", "precompile", "train", "finetune", "toolcall", "eval",
          "calib"), aliases=("qwen",)),
    Arch("toymoe", "moe", "Top-k routed mixture-of-experts decoder (toy and Qwen3-MoE shapes)",
         ("train", "infer", "eval"), aliases=("qwen3moe", "moe")),
    Arch("splat", "splat", "3D Gaussian splat rasteriser (headless)", ("render", "train"), built=True),
]

# Families of the reference whose models are outside this framework's scope: the grammar still
# recognises them so `brain <arch> …` answers with a clear message instead of "unknown command".
for _id, _fam in [("qwen35", "qwen"), ("qwen35moe", "moe"), ("qwen3omnimoe", "omni"), ("glmdsa", "glm"),
                  ("lfm2", "lfm"), ("qwen3tts", "tts"), ("yolov8", "detect"), ("zipdepth", "depth"),
                  ("flux2", "diffusion"), ("wan", "video"), ("ltxv", "video"), ("worldmirror2", "3d"),
                  ("diamond", "world-model"), ("toypid", "control"), ("s3dit", "diffusion"),
                  ("fastvlm", "vlm"), ("qwen3vl", "vlm"), ("sam2", "segment"), ("scrfd", "face"),
                  ("arcface", "face"), ("vqgan", "codec"), ("codeformer", "restore"),
                  ("rrdbnet", "upscale"), ("clip", "embed"), ("deepseek2ocr", "ocr"),
                  ("nemotronasr", "asr"), ("qwen3asr", "asr"), ("chronos2", "forecast"),
                  ("fincast", "forecast"), ("kronos", "forecast"), ("imageops", "image"),
                  ("demo", "demo"), ("imgpipe", "image")]:
    _ARCHS.append(Arch(_id, _fam, f"{_fam} family (not built by this framework)", (), built=False,
                       model_id=f"brain/{_id}"))

_BY_ID: Dict[str, Arch] = {}
for _a in _ARCHS:
    _BY_ID[_a.id] = _a
    for _al in _a.aliases:
        _BY_ID[_al] = _a


def by_id(s: str) -> Optional[Arch]:
    return _BY_ID.get(s)


def all_archs(built_only: bool = False) -> List[Arch]:
    return [a for a in _ARCHS if a.built or not built_only]
