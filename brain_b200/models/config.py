"""Model configuration records and their checkpoint JSON (the ``brain.config`` metadata string).

Key names and presets follow the reference so checkpoints stay interchangeable:
Qwen ``crates/qwen3/src/config.rs:44-73,100-188,219-238``; GPT ``crates/gpt2/src/model.rs:254-260``;
toy MoE ``crates/toymoe/src/train.rs:100-167``.  The 14B dense and 30B-A3B MoE shapes are presets
added here (the reference has none)."""
from __future__ import annotations

import json
from dataclasses import dataclass, field, asdict
from typing import List, Optional


@dataclass
class LoraCfg:
    rank: int = 8
    alpha: float = 16.0
    targets: List[str] = field(default_factory=lambda: ["wq", "wk", "wv", "wo"])


@dataclass
class QwenConfig:
    vocab: int = 151936
    block_size: int = 1024
    n_layers: int = 28
    d_model: int = 1024
    n_heads: int = 16
    n_kv_heads: int = 8
    head_dim: int = 128
    d_ff: int = 3072
    rope_theta: float = 1.0e6
    rms_eps: float = 1e-6
    max_position_embeddings: int = 0
    tie_embeddings: bool = True
    qk_norm: bool = True
    attn_bias: bool = False
    lora: Optional[LoraCfg] = None

    def __post_init__(self):
        if not self.max_position_embeddings:
            self.max_position_embeddings = self.block_size

    # ---- JSON (checkpoint metadata) ----
    def to_json(self) -> dict:
        v = {
            "model": "qwen", "vocab_size": self.vocab, "block_size": self.block_size,
            "n_layers": self.n_layers, "d_model": self.d_model, "n_heads": self.n_heads,
            "n_kv_heads": self.n_kv_heads, "head_dim": self.head_dim, "d_ff": self.d_ff,
            "rope_theta": self.rope_theta, "rms_norm_eps": self.rms_eps,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_embeddings,
        }
        if not self.qk_norm:
            v["qk_norm"] = False
        if self.attn_bias:
            v["attn_bias"] = True
        if self.lora is not None:
            v["lora"] = {"rank": self.lora.rank, "alpha": self.lora.alpha,
                         "targets": list(self.lora.targets)}
        return v

    @staticmethod
    def from_json(c: dict) -> "QwenConfig":
        lora = None
        if c.get("lora"):
            l = c["lora"]
            lora = LoraCfg(int(l["rank"]), float(l["alpha"]), list(l.get("targets", [])))
        bs = int(c.get("block_size", 1024))
        return QwenConfig(
            vocab=int(c["vocab_size"]), block_size=bs, n_layers=int(c["n_layers"]),
            d_model=int(c["d_model"]), n_heads=int(c["n_heads"]),
            n_kv_heads=int(c.get("n_kv_heads", c["n_heads"])),
            head_dim=int(c.get("head_dim", int(c["d_model"]) // int(c["n_heads"]))),
            d_ff=int(c["d_ff"]), rope_theta=float(c.get("rope_theta", 1e6)),
            rms_eps=float(c.get("rms_norm_eps", 1e-6)),
            max_position_embeddings=int(c.get("max_position_embeddings", bs)),
            tie_embeddings=bool(c.get("tie_word_embeddings", True)),
            qk_norm=bool(c.get("qk_norm", True)), attn_bias=bool(c.get("attn_bias", False)),
            lora=lora)

    # ---- presets ----
    @staticmethod
    def tiny() -> "QwenConfig":
        return QwenConfig(vocab=23, block_size=12, n_layers=2, d_model=16, n_heads=4, n_kv_heads=2,
                          head_dim=8, d_ff=32)

    @staticmethod
    def cli_default(vocab: int, block: int) -> "QwenConfig":
        """The architecture ``brain qwen3 train`` builds (crates/cli/src/qwen_cli.rs:368-475)."""
        return QwenConfig(vocab=vocab, block_size=block, n_layers=6, d_model=384, n_heads=6,
                          n_kv_heads=2, head_dim=64, d_ff=1024)

    @staticmethod
    def preset(name: str, block_size: int = 0) -> "QwenConfig":
        shapes = {
            "0.6b": dict(n_layers=28, d_model=1024, n_heads=16, n_kv_heads=8, d_ff=3072,
                         tie_embeddings=True),
            "1.7b": dict(n_layers=28, d_model=2048, n_heads=16, n_kv_heads=8, d_ff=6144,
                         tie_embeddings=True),
            "4b": dict(n_layers=36, d_model=2560, n_heads=32, n_kv_heads=8, d_ff=9728,
                       tie_embeddings=True),
            "8b": dict(n_layers=36, d_model=4096, n_heads=32, n_kv_heads=8, d_ff=12288,
                       tie_embeddings=False),
            "14b": dict(n_layers=40, d_model=5120, n_heads=40, n_kv_heads=8, d_ff=17408,
                        tie_embeddings=False),
        }
        key = name.lower().replace("qwen3-", "")
        if key not in shapes:
            raise KeyError(f"unknown Qwen3 preset {name!r}; have {sorted(shapes)}")
        c = QwenConfig(vocab=151936, head_dim=128, rope_theta=1e6, **shapes[key])
        if block_size:
            c.block_size = block_size
            c.max_position_embeddings = block_size
        return c

    @property
    def q_dim(self) -> int:
        return self.n_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.n_kv_heads * self.head_dim

    def param_list(self):
        """(name, numel) in checkpoint order (crates/qwen3/src/config.rs:311-366)."""
        d, out = self.d_model, []
        out.append(("tok.weight", self.vocab * d))

        def lin(name, o, i, bias=False):
            out.append((f"{name}.weight", o * i))
            if bias:
                out.append((f"{name}.bias", o))
            if self.lora is not None and name.rsplit(".", 1)[-1] in self.lora.targets:
                out.append((f"{name}.lora_a", self.lora.rank * i))
                out.append((f"{name}.lora_b", o * self.lora.rank))

        for l in range(self.n_layers):
            p = f"blocks.{l}"
            out.append((f"{p}.ln1.weight", d))
            lin(f"{p}.attn.wq", self.q_dim, d, self.attn_bias)
            lin(f"{p}.attn.wk", self.kv_dim, d, self.attn_bias)
            lin(f"{p}.attn.wv", self.kv_dim, d, self.attn_bias)
            if self.qk_norm:
                out.append((f"{p}.attn.q_norm.weight", self.head_dim))
                out.append((f"{p}.attn.k_norm.weight", self.head_dim))
            lin(f"{p}.attn.wo", d, self.q_dim)
            out.append((f"{p}.ln2.weight", d))
            lin(f"{p}.mlp.gate", self.d_ff, d)
            lin(f"{p}.mlp.up", self.d_ff, d)
            lin(f"{p}.mlp.down", d, self.d_ff)
        out.append(("norm.weight", d))
        if not self.tie_embeddings:
            out.append(("lm_head.weight", self.vocab * d))
        return out

    def param_count(self) -> int:
        return sum(n for _, n in self.param_list())


@dataclass
class GptConfig:
    vocab: int = 50257
    block_size: int = 1024
    n_layers: int = 12
    d_model: int = 768
    n_heads: int = 12
    d_ff: int = 3072
    itos: Optional[List[str]] = None

    def to_json(self) -> dict:
        v = {"model": "gpt", "vocab_size": self.vocab, "block_size": self.block_size,
             "n_layers": self.n_layers, "d_model": self.d_model, "n_heads": self.n_heads,
             "d_ff": self.d_ff}
        if self.itos is not None:
            v["itos"] = list(self.itos)
        return v

    @staticmethod
    def from_json(c: dict) -> "GptConfig":
        return GptConfig(vocab=int(c["vocab_size"]), block_size=int(c["block_size"]),
                         n_layers=int(c["n_layers"]), d_model=int(c["d_model"]),
                         n_heads=int(c["n_heads"]), d_ff=int(c.get("d_ff", 4 * int(c["d_model"]))),
                         itos=c.get("itos"))

    @staticmethod
    def small() -> "GptConfig":
        return GptConfig()

    @staticmethod
    def gradcheck() -> "GptConfig":
        """The shape of the CLI gradcheck gate (crates/gradcheck/src/lib.rs:290-300)."""
        return GptConfig(vocab=23, block_size=12, n_layers=2, d_model=16, n_heads=2, d_ff=32)

    def param_list(self):
        d, ff = self.d_model, self.d_ff
        out = [("tok.weight", self.vocab * d), ("pos.weight", self.block_size * d)]
        for l in range(self.n_layers):
            p = f"blocks.{l}"
            out += [(f"{p}.ln1.weight", d), (f"{p}.ln1.bias", d),
                    (f"{p}.attn.qkv.weight", 3 * d * d), (f"{p}.attn.qkv.bias", 3 * d),
                    (f"{p}.attn.out.weight", d * d), (f"{p}.attn.out.bias", d),
                    (f"{p}.ln2.weight", d), (f"{p}.ln2.bias", d),
                    (f"{p}.mlp.fc.weight", ff * d), (f"{p}.mlp.fc.bias", ff),
                    (f"{p}.mlp.proj.weight", d * ff), (f"{p}.mlp.proj.bias", d)]
        out += [("ln.weight", d), ("ln.bias", d), ("lm_head.weight", self.vocab * d)]
        return out

    def param_count(self) -> int:
        return sum(n for _, n in self.param_list())


@dataclass
class MoeConfig:
    """Sparse top-k MoE transformer.  ``family='toymoe'`` keeps the toy model's layout (fused qkv,
    interleaved RoPE, no QK-norm, names ``token_emb``/``norm1``/``norm2``); ``family='qwen3_moe'``
    is the Qwen3-MoE decoder (GQA + QK-norm + NeoX RoPE, names as the dense Qwen3 plus
    ``blocks.{l}.moe.router`` / ``blocks.{l}.moe.experts.{e}.{w_gate,w_up,w_down}``)."""
    family: str = "qwen3_moe"
    vocab: int = 151936
    block_size: int = 4096
    n_layers: int = 48
    d_model: int = 2048
    n_heads: int = 32
    n_kv_heads: int = 4
    head_dim: int = 128
    n_experts: int = 128
    top_k: int = 8
    d_ff: int = 768
    rope_theta: float = 1.0e6
    rms_eps: float = 1e-6
    aux_coef: float = 0.001
    z_coef: float = 0.0
    norm_topk_prob: bool = True
    routed_scaling: float = 1.0
    tie_embeddings: bool = False

    def to_json(self) -> dict:
        v = asdict(self)
        v["model"] = "moe" if self.family == "toymoe" else "qwen_moe"
        v["vocab_size"] = v.pop("vocab")
        v["rms_norm_eps"] = v.pop("rms_eps")
        v["tie_word_embeddings"] = v.pop("tie_embeddings")
        return v

    @staticmethod
    def from_json(c: dict) -> "MoeConfig":
        c = dict(c)
        c.pop("model", None)
        c["vocab"] = c.pop("vocab_size")
        c["rms_eps"] = c.pop("rms_norm_eps", 1e-6)
        c["tie_embeddings"] = c.pop("tie_word_embeddings", False)
        known = {f for f in MoeConfig.__dataclass_fields__}
        return MoeConfig(**{k: v for k, v in c.items() if k in known})

    @staticmethod
    def qwen3_30b_a3b(block_size: int = 4096) -> "MoeConfig":
        return MoeConfig(block_size=block_size)

    @staticmethod
    def toy(vocab: int = 64, block: int = 32) -> "MoeConfig":
        """Defaults of ``brain toymoe train`` (crates/toymoe/src/train.rs:700-730)."""
        return MoeConfig(family="toymoe", vocab=vocab, block_size=block, n_layers=2, d_model=64,
                         n_heads=4, n_kv_heads=4, head_dim=16, n_experts=4, top_k=2, d_ff=128,
                         rope_theta=10000.0, aux_coef=0.01, z_coef=1e-4, tie_embeddings=True)

    @property
    def q_dim(self):
        return self.n_heads * self.head_dim

    @property
    def kv_dim(self):
        return self.n_kv_heads * self.head_dim

    def param_list(self):
        d, out = self.d_model, []
        toy = self.family == "toymoe"
        out.append(("token_emb.weight" if toy else "tok.weight", self.vocab * d))
        for l in range(self.n_layers):
            p = f"blocks.{l}"
            if toy:
                out += [(f"{p}.norm1.weight", d), (f"{p}.attn.qkv.weight", 3 * d * d),
                        (f"{p}.attn.out.weight", d * d), (f"{p}.norm2.weight", d)]
            else:
                out += [(f"{p}.ln1.weight", d), (f"{p}.attn.wq.weight", self.q_dim * d),
                        (f"{p}.attn.wk.weight", self.kv_dim * d),
                        (f"{p}.attn.wv.weight", self.kv_dim * d),
                        (f"{p}.attn.q_norm.weight", self.head_dim),
                        (f"{p}.attn.k_norm.weight", self.head_dim),
                        (f"{p}.attn.wo.weight", d * self.q_dim), (f"{p}.ln2.weight", d)]
            out.append((f"{p}.moe.router.weight", self.n_experts * d))
            for e in range(self.n_experts):
                q = f"{p}.moe.experts.{e}"
                out += [(f"{q}.w_gate.weight", self.d_ff * d), (f"{q}.w_up.weight", self.d_ff * d),
                        (f"{q}.w_down.weight", d * self.d_ff)]
        out.append(("norm.weight", d))
        if not self.tie_embeddings:
            out.append(("lm_head.weight", self.vocab * d))
        return out

    def param_count(self) -> int:
        return sum(n for _, n in self.param_list())


def config_from_json(c) -> object:
    """Rebuild the right config record from a checkpoint's ``brain.config`` JSON."""
    if isinstance(c, str):
        c = json.loads(c)
    kind = c.get("model", "qwen")
    if kind == "gpt":
        return GptConfig.from_json(c)
    if kind in ("moe", "qwen_moe"):
        return MoeConfig.from_json(c)
    return QwenConfig.from_json(c)
