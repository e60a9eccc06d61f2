"""Render a checkpoint's OWN chat template: the Jinja2 string in ``tokenizer_config.json``
(``chat_template``) or ``chat_template.jinja`` beside the tokenizer, exactly what
``AutoTokenizer.apply_chat_template`` runs (reference: crates/data/src/chat_template.rs, which
interprets it with minijinja instead of hand-porting each family's control flow).

The environment mirrors the Hugging Face one: sandboxed and immutable, ``trim_blocks`` /
``lstrip_blocks`` on, ``raise_exception`` and ``strftime_now`` globals, and a ``tojson`` filter that
writes like Python's ``json.dumps(..., ensure_ascii=False)`` with the source key order kept (tool
schemas must come back out byte for byte)."""
from __future__ import annotations

import json
import os
from datetime import datetime
from typing import Dict, List, Optional, Sequence


class TemplateError(ValueError):
    pass


def _env():
    from jinja2.sandbox import ImmutableSandboxedEnvironment

    def raise_exception(message):
        raise TemplateError(str(message))

    def tojson(x, ensure_ascii=False, indent=None, separators=None, sort_keys=False):
        return json.dumps(x, ensure_ascii=ensure_ascii, indent=indent, separators=separators, sort_keys=sort_keys)

    env = ImmutableSandboxedEnvironment(trim_blocks=True, lstrip_blocks=True)
    env.filters["tojson"] = tojson
    env.globals["raise_exception"] = raise_exception
    env.globals["strftime_now"] = lambda fmt: datetime.now().strftime(fmt)
    return env


class ChatTemplate:
    def __init__(self, source: str, bos_token: str = "", eos_token: str = ""):
        import jinja2
        self.source = source
        self.bos_token, self.eos_token = bos_token, eos_token
        try:
            self._t = _env().from_string(source)
        except jinja2.TemplateError as e:
            raise TemplateError(f"chat template does not compile: {e}") from None

    def render(self, messages: Sequence, add_generation_prompt: bool = True, tools: Optional[List[Dict]] = None,
               **kwargs) -> str:
        import jinja2
        msgs = [dict(m) if isinstance(m, dict) else {"role": m[0], "content": m[1]} for m in messages]
        try:
            return self._t.render(messages=msgs, add_generation_prompt=add_generation_prompt, tools=tools or None,
                                  bos_token=self.bos_token, eos_token=self.eos_token, **kwargs)
        except TemplateError:
            raise
        except jinja2.TemplateError as e:
            raise TemplateError(f"chat template failed: {e}") from None

    @staticmethod
    def beside(tokenizer_path: str) -> Optional["ChatTemplate"]:
        """The template shipped next to ``tokenizer.json`` (``chat_template.jinja`` wins over the
        ``chat_template`` field of ``tokenizer_config.json``); None when there is none."""
        d = tokenizer_path if os.path.isdir(tokenizer_path) else (os.path.dirname(tokenizer_path) or ".")
        cfg: Dict = {}
        cpath = os.path.join(d, "tokenizer_config.json")
        if os.path.exists(cpath):
            try:
                cfg = json.loads(open(cpath, encoding="utf-8").read())
            except ValueError:
                cfg = {}
        src = None
        jpath = os.path.join(d, "chat_template.jinja")
        if os.path.exists(jpath):
            src = open(jpath, encoding="utf-8").read()
        elif isinstance(cfg.get("chat_template"), str):
            src = cfg["chat_template"]
        elif isinstance(cfg.get("chat_template"), list):      # [{"name": "default", "template": …}, …]
            named = {t.get("name"): t.get("template") for t in cfg["chat_template"] if isinstance(t, dict)}
            src = named.get("default") or next(iter(named.values()), None)
        if not src:
            return None

        def tok(v):
            return v.get("content", "") if isinstance(v, dict) else (v or "")
        return ChatTemplate(src, tok(cfg.get("bos_token")), tok(cfg.get("eos_token")))
