"""Model families: GPT-2, dense Qwen3/Qwen2, sparse MoE (toy and Qwen3-MoE)."""
from .config import GptConfig, LoraCfg, MoeConfig, QwenConfig, config_from_json


def build_from_config(cfg):
    """Instantiate the model a config record (or its checkpoint JSON) describes."""
    if isinstance(cfg, (dict, str)):
        cfg = config_from_json(cfg)
    if isinstance(cfg, GptConfig):
        from .gpt2 import Gpt2
        return Gpt2(cfg)
    if isinstance(cfg, MoeConfig):
        from .moe import MoeModel
        return MoeModel(cfg)
    from .qwen3 import Qwen3
    m = Qwen3(cfg)
    if cfg.lora is not None:
        from .lora import attach_lora
        attach_lora(m, cfg.lora)
    return m
