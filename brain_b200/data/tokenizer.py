"""Tokenizers: character-level (the ``meta.json`` ``itos`` table of the synthetic datasets) and
byte-level BPE in the GPT-2 / Qwen family (regex pre-tokenisation + byte-to-unicode mapping here,
merge loop native in csrc/runtime/bpe.cpp).  A BPE tokenizer is loaded from a HuggingFace
``tokenizer.json`` (``model.vocab``, ``model.merges``, ``added_tokens``) or built in memory.
Reference: crates/data/src/{tokenizer,bpe,qwen_tokenizer}.rs."""
from __future__ import annotations

import ctypes
import json
from typing import Dict, Iterable, List, Optional, Sequence

import numpy as np

from .. import _host

c = ctypes
_host.register({
    "bbh_bpe_new": (c.c_void_p, []),
    "bbh_bpe_free": (None, [c.c_void_p]),
    "bbh_bpe_add_token": (None, [c.c_void_p, c.c_char_p, c.c_int32, c.c_int32]),
    "bbh_bpe_add_merge": (c.c_int, [c.c_void_p, c.c_char_p, c.c_int32, c.c_char_p, c.c_int32, c.c_int32]),
    "bbh_bpe_encode_word": (c.c_int32, [c.c_void_p, c.c_char_p, c.c_int32, c.c_void_p, c.c_int32]),
    "bbh_bpe_token": (c.c_int32, [c.c_void_p, c.c_int32, c.c_char_p, c.c_int32]),
    "bbh_bpe_vocab_size": (c.c_int32, [c.c_void_p]),
})

GPT2_SPLIT = r"""'s|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+"""
QWEN_SPLIT = (r"""(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n]*"""
              r"""|\s*[\r\n]+|\s+(?!\S)|\s+""")


def bytes_to_unicode() -> Dict[int, str]:
    """The GPT-2 reversible byte -> printable-unicode table."""
    bs = list(range(ord("!"), ord("~") + 1)) + list(range(ord("¡"), ord("¬") + 1)) + \
        list(range(ord("®"), ord("ÿ") + 1))
    cs = bs[:]
    n = 0
    for b in range(256):
        if b not in bs:
            bs.append(b)
            cs.append(256 + n)
            n += 1
    return {b: chr(ch) for b, ch in zip(bs, cs)}


def utf8_complete(b: bytes) -> int:
    """Length of the longest prefix of ``b`` that does not end inside a multi-byte UTF-8 sequence
    (an incomplete but so far valid tail of up to three bytes is left for the next chunk)."""
    n = len(b)
    for k in range(1, min(4, n) + 1):
        ch = b[n - k]
        if ch & 0xC0 == 0x80:
            continue
        need = 4 if ch >= 0xF0 else 3 if ch >= 0xE0 else 2 if ch >= 0xC0 else 1
        return n - k if k < need else n
    return n


class CharTokenizer:
    def __init__(self, itos: Sequence[str]):
        self.itos = list(itos)
        self.stoi = {ch: i for i, ch in enumerate(self.itos)}
        self.vocab_size = len(self.itos)
        self.eos_id = None

    @staticmethod
    def from_text(text: str) -> "CharTokenizer":
        return CharTokenizer(sorted(set(text)))

    def encode(self, text: str) -> List[int]:
        try:
            return [self.stoi[ch] for ch in text]
        except KeyError as e:
            raise ValueError(f"character {e.args[0]!r} is not in the vocabulary") from None

    def decode(self, ids: Iterable[int]) -> str:
        return "".join(self.itos[i] for i in ids if 0 <= i < self.vocab_size)


def _split_pattern(pre) -> Optional[str]:
    """The regex of a tokenizer.json ``pre_tokenizer`` entry: a ``Split`` with a ``Regex`` pattern, or a
    ``ByteLevel`` that applies the GPT-2 pattern itself; None when the entry names neither."""
    if not isinstance(pre, dict):
        return None
    kind = pre.get("type")
    if kind == "Sequence":
        for sub in pre.get("pretokenizers", []):
            pat = _split_pattern(sub)
            if pat is not None:
                return pat
        return None
    if kind == "Split":
        pat = pre.get("pattern", {})
        if isinstance(pat, dict) and "Regex" in pat and pre.get("behavior", "Isolated").lower() == "isolated" \
                and not pre.get("invert", False):
            return pat["Regex"]
        return None
    if kind == "ByteLevel" and pre.get("use_regex", True):
        return GPT2_SPLIT
    return None


def _normal_form(norm) -> Optional[str]:
    """Unicode normal form a tokenizer.json ``normalizer`` entry asks for (NFC / NFD / NFKC / NFKD)."""
    if not isinstance(norm, dict):
        return None
    if norm.get("type") in ("NFC", "NFD", "NFKC", "NFKD"):
        return norm["type"]
    if norm.get("type") == "Sequence":
        for sub in norm.get("normalizers", []):
            f = _normal_form(sub)
            if f:
                return f
    return None


class BpeTokenizer:
    def __init__(self, vocab: Dict[str, int], merges: Sequence, special: Optional[Dict[str, int]] = None,
                 pattern: str = QWEN_SPLIT, eos: Optional[str] = None, normalize: Optional[str] = None):
        import regex
        self._re = regex.compile(pattern)
        self.normalize = normalize      # Unicode normal form applied before splitting ("NFC" for Qwen)
        self._b2u = bytes_to_unicode()
        self._u2b = {v: k for k, v in self._b2u.items()}
        self.special = dict(special or {})
        self._special_re = None
        if self.special:
            self._special_re = regex.compile("(" + "|".join(regex.escape(s) for s in
                                                            sorted(self.special, key=len, reverse=True)) + ")")
        self._id2special = {v: k for k, v in self.special.items()}
        #: ids dropped by ``skip_special``: control tokens only.  Added tokens a tokenizer.json marks
        #: ``"special": false`` (Qwen3's <think>, </think>, <tool_call>, ...) are matched as whole
        #: strings when encoding but are ordinary text when decoding.
        self.control = set(self._id2special)
        lib = _host.lib()
        self._h = lib.bbh_bpe_new()
        for tok, i in vocab.items():
            b = tok.encode("utf-8")
            lib.bbh_bpe_add_token(self._h, b, len(b), i)
        for rank, m in enumerate(merges):
            l, r = m.split(" ", 1) if isinstance(m, str) else m
            lb, rb = l.encode("utf-8"), r.encode("utf-8")
            lib.bbh_bpe_add_merge(self._h, lb, len(lb), rb, len(rb), rank)
        self.vocab_size = max([lib.bbh_bpe_vocab_size(self._h)] + [i + 1 for i in self.special.values()])
        self.eos_id = self.special.get(eos) if eos else None
        self.chat_template = None     # a checkpoint's own Jinja template (data.chat_template.ChatTemplate)
        self._buf = np.empty(4096, dtype=np.int32)

    def __del__(self):
        try:
            if getattr(self, "_h", None):
                _host.lib().bbh_bpe_free(self._h)
                self._h = None
        except Exception:
            pass

    @staticmethod
    def from_file(path: str) -> "BpeTokenizer":
        """Load a HuggingFace ``tokenizer.json``."""
        d = json.loads(open(path, encoding="utf-8").read())
        model = d["model"]
        special = {t["content"]: t["id"] for t in d.get("added_tokens", [])}
        eos = next((s for s in ("<|im_end|>", "<|endoftext|>") if s in special), None)
        # the file's own split pattern and normaliser win; the family heuristic covers files without
        pat = _split_pattern(d.get("pre_tokenizer"))
        if pat is not None:
            import regex
            try:
                regex.compile(pat)
            except regex.error:          # a construct of another regex engine: use the family pattern
                pat = None
        if pat is None:
            pat = QWEN_SPLIT if "<|im_end|>" in special or len(model["vocab"]) > 60000 else GPT2_SPLIT
        tok = BpeTokenizer(model["vocab"], model["merges"], special, pat, eos,
                           normalize=_normal_form(d.get("normalizer")))
        tok.control = {t["id"] for t in d.get("added_tokens", []) if t.get("special", True)}
        from .chat_template import ChatTemplate
        tok.chat_template = ChatTemplate.beside(path)
        return tok

    @staticmethod
    def byte_level(merges: Sequence = (), special: Optional[Dict[str, int]] = None) -> "BpeTokenizer":
        """A 256-symbol byte vocabulary plus the given merges (used by tests and synthetic data)."""
        b2u = bytes_to_unicode()
        vocab = {b2u[b]: b for b in range(256)}
        nxt = 256
        for m in merges:
            l, r = m.split(" ", 1)
            vocab[l + r] = nxt
            nxt += 1
        sp = {s: nxt + i for i, s in enumerate(special or [])} if not isinstance(special, dict) else special
        return BpeTokenizer(vocab, merges, sp, GPT2_SPLIT, eos=next(iter(sp), None) if sp else None)

    def _encode_plain(self, text: str, out: List[int]):
        lib = _host.lib()
        for piece in self._re.findall(text):
            mapped = "".join(self._b2u[b] for b in piece.encode("utf-8")).encode("utf-8")
            if len(mapped) > self._buf.size:
                self._buf = np.empty(len(mapped), dtype=np.int32)
            n = lib.bbh_bpe_encode_word(self._h, mapped, len(mapped), self._buf.ctypes.data, self._buf.size)
            if n < 0:
                raise ValueError(f"cannot encode {piece!r}")
            out.extend(self._buf[:n].tolist())

    def encode(self, text: str, allow_special: bool = True) -> List[int]:
        out: List[int] = []
        if self.normalize:
            import unicodedata
            text = unicodedata.normalize(self.normalize, text)
        if self._special_re is None or not allow_special:
            self._encode_plain(text, out)
            return out
        for part in self._special_re.split(text):
            if not part:
                continue
            if part in self.special:
                out.append(self.special[part])
            else:
                self._encode_plain(part, out)
        return out

    def decode_bytes(self, ids: Iterable[int], skip_special: bool = False) -> bytes:
        """The raw bytes of a token sequence; a multi-byte character may be split across tokens, so
        streaming callers join bytes and decode only complete sequences (:func:`utf8_complete`)."""
        lib = _host.lib()
        buf = ctypes.create_string_buffer(256)
        chunks: List[bytes] = []
        for i in ids:
            i = int(i)
            if i in self._id2special:
                if not (skip_special and i in self.control):
                    chunks.append(self._id2special[i].encode("utf-8"))
                continue
            n = lib.bbh_bpe_token(self._h, i, buf, 256)
            if n <= 0 or n > 256:
                continue
            mapped = buf.raw[:n].decode("utf-8", errors="ignore")
            chunks.append(bytes(self._u2b.get(ch, ord("?")) for ch in mapped))
        return b"".join(chunks)

    def decode(self, ids: Iterable[int], skip_special: bool = False) -> str:
        return self.decode_bytes(ids, skip_special).decode("utf-8", errors="replace")

    def apply_chat_template(self, messages, add_generation_prompt: bool = True,
                            enable_thinking: bool = True, tools=None) -> str:
        """ChatML rendering used by the Qwen family (reference: crates/data/src/qwen_tokenizer.rs
        ``apply_chat_template``): ``<|im_start|>role\ncontent<|im_end|>\n`` per message, an open
        assistant turn when generating, and an empty think block when thinking is disabled.
        ``messages`` is a sequence of (role, content) pairs or {"role", "content"} dicts.  When the
        checkpoint ships its own template (``tokenizer_config.json`` / ``chat_template.jinja``) that
        template is rendered instead."""
        if self.chat_template is not None:
            return self.chat_template.render(messages, add_generation_prompt, tools, enable_thinking=enable_thinking)
        return render_chatml(messages, add_generation_prompt, enable_thinking, tools)


def load_tokenizer(path_or_dir: str):
    """tokenizer.json (BPE) or a dataset directory with meta.json (character level)."""
    import os
    if os.path.isdir(path_or_dir):
        tj = os.path.join(path_or_dir, "tokenizer.json")
        if os.path.exists(tj):
            return BpeTokenizer.from_file(tj)
        from .binio import read_meta
        meta = read_meta(path_or_dir)
        if meta.get("itos"):
            return CharTokenizer(meta["itos"])
        raise FileNotFoundError(f"{path_or_dir}: no tokenizer.json or meta.json with itos")
    return BpeTokenizer.from_file(path_or_dir)


def render_chatml(messages, add_generation_prompt: bool = True, enable_thinking: bool = True,
                  tools=None) -> str:
    out = []
    msgs = [(m["role"], m.get("content") or "") if isinstance(m, dict) else (m[0], m[1]) for m in messages]
    if tools:
        sys_txt = msgs[0][1] + "\n\n" if msgs and msgs[0][0] == "system" else ""
        if msgs and msgs[0][0] == "system":
            msgs = msgs[1:]
        decl = "\n".join(json.dumps(t, separators=(",", ":"), ensure_ascii=False) for t in tools)
        out.append("<|im_start|>system\n" + sys_txt + "# Tools\n\nYou may call one or more functions to assist "
                   "with the user query.\n\nYou are provided with function signatures within <tools></tools> "
                   "XML tags:\n<tools>\n" + decl + "\n</tools>\n\nFor each function call, return a json object "
                   "with function name and arguments within <tool_call></tool_call> XML tags:\n<tool_call>\n"
                   "{\"name\": <function-name>, \"arguments\": <args-json-object>}\n</tool_call><|im_end|>\n")
    for role, content in msgs:
        if role == "tool":
            out.append(f"<|im_start|>user\n<tool_response>\n{content}\n</tool_response><|im_end|>\n")
        else:
            out.append(f"<|im_start|>{role}\n{content}<|im_end|>\n")
    if add_generation_prompt:
        out.append("<|im_start|>assistant\n")
        if not enable_thinking:
            out.append("<think>\n\n</think>\n\n")
    return "".join(out)
