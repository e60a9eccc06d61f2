"""Resident (servable) models (reference: crates/cli/src/resident_llm.rs — the language-model
resident with its ``generate`` action contract, pool sizing ``num_blocks = 2·ceil(ctx/16) +
max_batch``, ``max_prefill = min(ctx, 512)``, ctx default 24 576 (:321, :411-418) — and
crates/cli/src/resident_mock.rs — the deterministic weight-free mock under ``BRAIN_MOCK``).

Unlike the reference, which runs one executor batch to completion before taking the next group
(resident_llm.rs:697-775), the language model here feeds ONE long-lived continuous-batching
scheduler from a dedicated serving thread: requests join and leave the running batch every step."""
from __future__ import annotations

import json
import os
import queue
import threading
import time
from typing import Callable, Dict, List, Optional

from ..utils import trace
from .capability import (ActionError, ActionSpec, Blob, BlobSpec, Invocation, Manifest, Outcome, ParamSpec,
                         Progress, generate_spec, last_user_text)

ProgressFn = Callable[[Progress], None]


class ResidentModel:
    id: str = ""

    def manifest(self) -> Manifest:
        raise NotImplementedError

    def run(self, action: str, inv: Invocation, progress: ProgressFn) -> Outcome:
        raise NotImplementedError

    def context_length(self) -> Optional[int]:
        return None

    def max_concurrency(self) -> int:
        return 1

    def close(self) -> None:
        pass


# ------------------------------------------------------------------------------------ mock
FAIL_TRIGGER = "__mock_fail__"
TOOL_CALL_TRIGGER = "__MOCK_TOOL_CALL__"
_MOCK_TOOL_CALLS = [("get_weather", '{"location": "Paris"}'), ("set_timer", '{"minutes": 5}')]
_MOCK_REASONING = "checking which tool to call"
EMBED_DIM = 8


class MockResident(ResidentModel):
    """Every action is a pure function of its inputs; exercises the whole serving path without
    weights or a GPU."""
    id = "brain/mock"

    def manifest(self) -> Manifest:
        gen = generate_spec("deterministic mock chat generation")
        for p in gen.params:
            if p.name == "max_new":
                p.default = 1024
            if p.name == "temp":
                p.default = 1.0
            if p.name == "top_k":
                p.default = 0
        embed = ActionSpec("embed", "deterministic mock text embedding", False,
                           [ParamSpec("text", "str", "input text")], [BlobSpec("text", "text", "input text")],
                           [BlobSpec("embeddings", "bytes", "mean vector, f32 little-endian, meta.shape=[1,DIM]")])
        return Manifest(self.id, "deterministic mock model (chat + embeddings)", [gen, embed], 32768)

    def max_concurrency(self) -> int:
        return 256

    def context_length(self):
        return 32768

    def run(self, action, inv, progress):
        if action == "generate":
            return self._generate(inv, progress)
        if action == "embed":
            return self._embed(inv)
        raise ActionError(f"mock: unknown action '{action}'")

    def _generate(self, inv: Invocation, progress: ProgressFn) -> Outcome:
        p = inv.params
        max_new = max(int(p.get("max_new", 1024)), 1)
        user = last_user_text(p)
        if FAIL_TRIGGER in user:
            # an internal-looking message: the HTTP layer must not leak it
            raise RuntimeError("mock resident action failed: /srv/secret/model.bin: boom (internal failure)")
        delay = float(os.environ.get("BRAIN_MOCK_DELAY_MS", "0") or 0) / 1e3
        t_end = time.time() + delay
        while time.time() < t_end:
            if inv.cancel.is_cancelled():
                raise ActionError("cancelled", "cancelled")
            time.sleep(min(0.025, max(t_end - time.time(), 0)))
        n_prompt = max(len(user.split()), 1)
        if TOOL_CALL_TRIGGER in user:
            n = min(max(user.count(TOOL_CALL_TRIGGER), 1), len(_MOCK_TOOL_CALLS))
            progress(Progress("reasoning", text=_MOCK_REASONING))
            calls = []
            for i, (name, args) in enumerate(_MOCK_TOOL_CALLS[:n]):
                progress(Progress("tool_call_start", data={"index": i, "id": f"call_{i}", "name": name}))
                mid = len(args) // 2
                for frag in (args[:mid], args[mid:]):
                    if frag:
                        progress(Progress("tool_call_args", text=frag, data={"index": i}))
                progress(Progress("tool_call_end", data={"index": i}))
                calls.append({"id": f"call_{i}", "name": name, "arguments": args})
            return Outcome({"prompt_tokens": n_prompt, "completion_tokens": n, "finish_reason": "tool_calls",
                            "reasoning_content": _MOCK_REASONING, "tool_calls": json.dumps(calls)},
                           {"text": Blob("text", b"")})
        reply = f"You said: {user.strip()}" if user.strip() else "mock reply ready"
        words = reply.split()
        stops = []
        if p.get("stop"):
            try:
                stops = [s for s in json.loads(p["stop"]) if isinstance(s, str) and s]
            except ValueError:
                stops = []
        pieces: List[str] = []
        hit_stop = False
        for i, w in enumerate(words):
            if len(pieces) >= max_new:
                break
            if any(s in w for s in stops):
                hit_stop = True
                break
            pieces.append(w if i == 0 else " " + w)
        finish = "length" if not hit_stop and len(pieces) < len(words) else "stop"
        for i, piece in enumerate(pieces):
            if inv.cancel.is_cancelled():
                raise ActionError("cancelled", "cancelled")
            progress(Progress("token", i, len(pieces), piece))
        return Outcome({"prompt_tokens": n_prompt, "completion_tokens": len(pieces), "finish_reason": finish},
                       {"text": Blob("text", "".join(pieces).encode())})

    def _embed(self, inv: Invocation) -> Outcome:
        import math
        import struct
        b = inv.blobs.get("text")
        text = b.data.decode("utf-8", errors="replace") if b else inv.params.get("text")
        if text is None:
            raise ActionError("mock: embed needs a `text` param or a `text` input blob")
        v = [0.0] * EMBED_DIM
        for i, ch in enumerate(text.encode("utf-8")):
            v[i % EMBED_DIM] += float(ch)
        n = max(len(text.encode("utf-8")), 1)
        mean = [math.sin(x / n) for x in v]
        raw = struct.pack(f"<{EMBED_DIM}f", *mean)
        return Outcome({"mean": mean, "tokens": max(len(text.split()), 1), "dim": EMBED_DIM},
                       {"embeddings": Blob("bytes", raw, {"shape": [1, EMBED_DIM]})})


# ------------------------------------------------------------------------------------ GPT (char level)
class GptResident(ResidentModel):
    """A character-level GPT checkpoint (``brain gpt2 train``) behind the ``generate`` action: the
    prompt is continued token by token without a KV cache — these are small models — and every
    character is streamed as it is sampled (reference: ``brain serve --stdio --gpt <ckpt>``,
    crates/cli/src/run_cli.rs:186-263)."""

    def __init__(self, model, itos, model_id: str = "brain/gpt2", defaults: Optional[Dict] = None):
        from ..data.tokenizer import CharTokenizer
        self.id = model_id
        self.model = model.eval()
        self.tok = CharTokenizer(itos)
        self.defaults = dict(defaults or {})
        self._lock = threading.Lock()

    def manifest(self) -> Manifest:
        gen = generate_spec("character-level text continuation")
        for p in gen.params:
            if p.name in self.defaults:
                p.default = self.defaults[p.name]
            if p.name == "chat":
                p.default = False
        return Manifest(self.id, "GPT-2 style decoder (character vocabulary)", [gen], self.model.cfg.block_size)

    def context_length(self):
        return self.model.cfg.block_size

    def run(self, action: str, inv: Invocation, progress: ProgressFn) -> Outcome:
        if action != "generate":
            raise ActionError(f"{self.id}: unknown action '{action}'")
        import torch
        from ..data.rng import Rng
        p = inv.params
        text = last_user_text(p) or "\n"
        try:
            ids = self.tok.encode(text)
        except ValueError as e:
            raise ActionError("invalid_request", str(e)) from None
        max_new = max(int(p.get("max_new", 128)), 1)
        temp, top_k = float(p.get("temp", 0.8)), int(p.get("top_k", 40))
        rng = Rng(int(p.get("seed", 0)) or 1234)
        block = self.model.cfg.block_size
        dev = next(self.model.parameters()).device
        out: List[int] = []
        with self._lock, torch.no_grad():
            for i in range(max_new):
                if inv.cancel.is_cancelled():
                    raise ActionError("cancelled", "cancelled")
                ctx = torch.tensor([(ids + out)[-block:]], device=dev, dtype=torch.int32)
                logits = self.model(ctx)[0, -1].float()
                if temp <= 0:
                    nxt = int(logits.argmax())
                else:
                    logits = logits / temp
                    if 0 < top_k < logits.numel():
                        thr = torch.topk(logits, top_k).values[-1]
                        logits = torch.where(logits < thr, torch.full_like(logits, float("-inf")), logits)
                    cdf = torch.cumsum(torch.softmax(logits, dim=-1).cpu(), 0)
                    nxt = int(torch.searchsorted(cdf, torch.tensor(rng.next_f32())).clamp_max(cdf.numel() - 1))
                out.append(nxt)
                progress(Progress("token", i, max_new, self.tok.decode([nxt])))
        return Outcome({"prompt_tokens": len(ids), "completion_tokens": len(out), "finish_reason": "length"},
                       {"text": Blob("text", self.tok.decode(out).encode())})


def load_gpt(path: str, device: str = "auto", defaults: Optional[Dict] = None) -> GptResident:
    from ..checkpoint import st
    from ..train import pick_device
    model, cfg, card = st.load_model(path, device=pick_device(device))
    itos = (cfg or {}).get("itos")
    if not itos:
        raise ValueError(f"{path}: the checkpoint carries no character vocabulary (train it with `brain gpt2 train`)")
    return GptResident(model, itos, card.id if card is not None and card.id else "brain/gpt2", defaults)


# ------------------------------------------------------------------------------------ language model
class _Job:
    __slots__ = ("prompt", "max_new", "params", "seed", "ignore_eos", "stops", "on_token", "done", "rid",
                 "text", "emitted", "n_tokens", "finish", "error", "cancel", "n_prompt", "held", "raw")

    def __init__(self):
        self.done = threading.Event()
        self.rid = None
        self.text = ""
        self.emitted = 0
        self.n_tokens = 0
        self.finish = None
        self.error = None
        self.held = ""
        self.raw = b""             # bytes of an unfinished multi-byte character


class LlmResident(ResidentModel):
    """A Qwen-family checkpoint behind a paged-KV engine and one continuous-batching scheduler."""

    def __init__(self, model, tokenizer, model_id: str = "brain/qwen3", ctx: Optional[int] = None,
                 max_batch: Optional[int] = None, weights: str = "bf16", block_size: int = 16, tp=None,
                 kv_dtype: str = "bf16", kv_clip=None):
        from ..serve.engine import QwenEngine
        from ..serve.scheduler import Scheduler
        self.id = model_id
        self.tok = tokenizer
        env_ctx = int(os.environ.get("BRAIN_QWEN_CTX", "24576"))
        self.ctx = min(ctx or env_ctx, max(model.cfg.max_position_embeddings, model.cfg.block_size))
        self.max_batch = max_batch or int(os.environ.get("BRAIN_SCHED_MAX_BATCH", "16"))
        blocks_per_ctx = -(-self.ctx // block_size)
        pool = int(os.environ.get("BRAIN_SCHED_NUM_BLOCKS", "0")) or 2 * blocks_per_ctx + self.max_batch
        self.engine = QwenEngine(model, block_size=block_size, num_blocks=pool, max_seq_len=self.ctx,
                                 max_prefill=min(self.ctx, 512), weights=weights, tp=tp,
                                 kv_dtype=kv_dtype, kv_clip=kv_clip)
        ids = tokenizer.encode("<|im_end|>") if hasattr(tokenizer, "special") else []
        self.eos = ids[0] if len(ids) == 1 else getattr(tokenizer, "eos_id", None)
        # One forward per step for prompt chunks + decode rows is the default on the GPU.  On the CPU
        # backend it stays opt-in: there a burst of concurrent requests gave one request a different
        # first token than its serial run about once in ten bursts (none in thirty with two forwards);
        # the cause has not been found, and the CPU backend gains nothing from the shared launches.
        mixed_default = "1" if self.engine.device.type == "cuda" else "0"
        # admission policy: "name" or "name:arg", e.g. max_queue_depth:64, ttft_budget:1000 (ms)
        pol, _, pol_arg = os.environ.get("BRAIN_SCHED_POLICY", "unbounded_queue").partition(":")
        self.sched = Scheduler(self.engine, max_batch=self.max_batch, eos=self.eos,
                               mixed=os.environ.get("BRAIN_SERVE_MIXED", mixed_default) == "1",
                               policy=pol, policy_arg=float(pol_arg or 0))
        self._inbox: "queue.Queue[_Job]" = queue.Queue()
        self._jobs: Dict[int, _Job] = {}
        self._stop = threading.Event()
        self._wake = threading.Event()
        self._thread = threading.Thread(target=self._loop, name=f"serve:{model_id}", daemon=True)
        self._thread.start()

    # ---- contract
    def manifest(self) -> Manifest:
        return Manifest(self.id, "Qwen-family decoder served with paged KV and continuous batching",
                        [generate_spec("chat / text generation")], self.ctx)

    def context_length(self):
        return self.ctx

    def max_concurrency(self) -> int:
        return 256

    def close(self):
        self._stop.set()
        self._wake.set()
        self._thread.join(timeout=5)

    def stats(self) -> Dict[str, int]:
        return self.sched.stats()

    # ---- request side (any thread)
    def build_prompt(self, p: Dict) -> List[int]:
        if p.get("messages"):
            msgs = json.loads(p["messages"])
            if p.get("system"):
                msgs = [{"role": "system", "content": p["system"]}] + msgs
            tools = json.loads(p["tools"]) if p.get("tools") and p.get("tool_choice") != "none" else None
            text = self.tok.apply_chat_template(msgs, True, bool(p.get("enable_thinking", True)), tools)
        elif p.get("chat", True) and hasattr(self.tok, "apply_chat_template"):
            msgs = ([{"role": "system", "content": p["system"]}] if p.get("system") else []) + \
                   [{"role": "user", "content": p.get("prompt") or ""}]
            text = self.tok.apply_chat_template(msgs, True, bool(p.get("enable_thinking", True)))
        else:
            text = p.get("prompt") or ""
        return self.tok.encode(text)

    def run(self, action, inv, progress):
        from ..data.chat import parse_tool_calls, split_reasoning
        from ..serve.sampling import SampleParams
        if action != "generate":
            raise ActionError(f"{self.id}: unknown action '{action}'")
        p = inv.params
        job = _Job()
        job.prompt = self.build_prompt(p)
        if not job.prompt:
            raise ActionError("empty prompt")
        job.n_prompt = len(job.prompt)
        job.max_new = max(int(p.get("max_new", 128)), 1)
        job.params = SampleParams(float(p.get("temp", 0.8)), int(p.get("top_k", 40)), float(p.get("top_p", 1.0)))
        job.seed = int(p.get("seed", 0))
        job.ignore_eos = bool(p.get("ignore_eos", False))
        job.stops = [s for s in json.loads(p["stop"]) if s] if p.get("stop") else []
        n = [0]
        from ..data.chat import ReasoningStream
        think = ReasoningStream()       # text inside <think>…</think> streams as reasoning, not content

        def on_token(piece: str):
            for kind, text in think.feed(piece):
                progress(Progress(kind, n[0], job.max_new, text))
            n[0] += 1
        job.on_token = on_token
        job.cancel = inv.cancel
        inv.cancel.on_cancel(self._wake.set)
        self._inbox.put(job)
        self._wake.set()
        job.done.wait()
        if job.error is not None:
            raise job.error
        for kind, text in think.flush():         # a held "<" that never became a marker
            progress(Progress(kind, n[0], job.max_new, text))
        reasoning, visible = split_reasoning(job.text)
        calls, visible2 = parse_tool_calls(visible) if p.get("tools") else ([], visible)
        out = {"prompt_tokens": job.n_prompt, "completion_tokens": job.n_tokens, "finish_reason": job.finish}
        if reasoning:
            out["reasoning_content"] = reasoning
        if calls:
            out["finish_reason"] = "tool_calls"
            out["tool_calls"] = json.dumps([{"id": f"call_{i}", "name": c["name"],
                                             "arguments": json.dumps(c["arguments"])} for i, c in enumerate(calls)])
            visible = visible2
        return Outcome(out, {"text": Blob("text", visible.encode())})

    # ---- serving thread
    def _finish(self, job: _Job, finish: Optional[str], error: Optional[Exception] = None):
        if error is None and finish != "stop_sequence":
            tail = job.held + job.raw.decode("utf-8", errors="replace")
            if tail:
                job.text += tail
                job.on_token(tail)
        job.held, job.raw = "", b""
        job.finish, job.error = finish, error
        if job.rid is not None:
            self._jobs.pop(job.rid, None)
            try:
                self.sched.forget(job.rid)
            except Exception:
                pass
        job.done.set()

    def _deliver(self, job: _Job, new_tokens: List[int]) -> bool:
        """Decode incrementally, hold back text that could be the start of a stop sequence;
        returns True when a stop sequence ended the job."""
        job.n_tokens += len(new_tokens)
        # only the new tokens are decoded (a request of n tokens costs n token lookups, not n^2 / 2);
        # bytes of a character that is split across tokens wait in job.raw for their continuation
        if hasattr(self.tok, "decode_bytes"):
            raw = job.raw + self.tok.decode_bytes(new_tokens, skip_special=True)
        else:
            raw = job.raw + self.tok.decode(new_tokens).encode("utf-8")
        from ..data.tokenizer import utf8_complete
        cut = utf8_complete(raw)
        job.raw = raw[cut:]
        pending = job.held + raw[:cut].decode("utf-8", errors="replace")
        for s in job.stops:
            k = pending.find(s)
            if k >= 0:
                piece = pending[:k]
                if piece:
                    job.text += piece
                    job.on_token(piece)
                job.held = ""
                return True
        hold = 0
        for s in job.stops:
            for k in range(min(len(s) - 1, len(pending)), 0, -1):
                if pending.endswith(s[:k]):
                    hold = max(hold, k)
                    break
        piece = pending[:len(pending) - hold] if hold else pending
        job.held = pending[len(piece):]
        if piece:
            job.text += piece
            job.on_token(piece)
        return False

    def _loop(self):
        from ..serve.scheduler import RejectReason
        while not self._stop.is_set():
            while True:
                try:
                    job = self._inbox.get_nowait()
                except queue.Empty:
                    break
                if job.cancel.is_cancelled():
                    self._finish(job, None, ActionError("cancelled", "cancelled"))
                    continue
                try:
                    job.rid = self.sched.submit(job.prompt, job.max_new, job.params, job.seed, job.ignore_eos)
                    self._jobs[job.rid] = job
                except RejectReason as e:
                    kind = {"exceeds_capacity": "context_length_exceeded",
                            "policy_rejected": "rate_limit_exceeded"}.get(e.kind, "invalid_request")
                    self._finish(job, None, ActionError(str(e), kind))
            for job in [j for j in self._jobs.values() if j.cancel.is_cancelled()]:
                self.sched.cancel(job.rid)
                self._finish(job, None, ActionError("cancelled", "cancelled"))
            if self.sched.is_idle():
                self._wake.wait(0.05)
                self._wake.clear()
                continue
            try:
                rep = self.sched.step()
            except Exception as e:  # noqa: BLE001 - one failed step fails its requests, the loop survives
                trace.event("serve", 1, "scheduler step failed", error=repr(e))
                for job in list(self._jobs.values()):
                    try:
                        self.sched.cancel(job.rid)
                    except Exception:
                        pass
                    self._finish(job, None, e)
                continue
            for rid, toks in rep.new_tokens.items():
                job = self._jobs.get(rid)
                if job is None:
                    continue
                try:
                    if self._deliver(job, toks):
                        self.sched.cancel(rid)
                        self._finish(job, "stop_sequence")
                except Exception as e:  # noqa: BLE001
                    self.sched.cancel(rid)
                    self._finish(job, None, e)
            for rid in rep.finished:
                job = self._jobs.get(rid)
                if job is not None:
                    info = self.sched.info(rid)
                    self._finish(job, "length" if info.finish in ("length", "max_new") else "stop")


# ------------------------------------------------------------------------------------ registry
def resolve_env_model():
    """``BRAIN_QWEN_WEIGHTS`` (a file) or ``BRAIN_MODEL`` (a ``<vendor>/<repo>[:owner:name:tag]``
    reference looked up in the model store; nothing is fetched) -> (weights, tokenizer, adapter
    file or None, served id or None); None when neither is set.  Raises FileNotFoundError for a
    reference that is not on disk."""
    w = os.environ.get("BRAIN_QWEN_WEIGHTS")
    if w:
        t = os.environ.get("BRAIN_QWEN_TOKENIZER") or os.path.join(os.path.dirname(w) or ".", "tokenizer.json")
        return w, t, None, None
    name = os.environ.get("BRAIN_MODEL")
    if not name:
        return None
    from ..modelref import ModelRef, canonical
    from ..modelstore import Store, default_root
    ref = ModelRef.parse(canonical(name))
    root = default_root()
    m = Store(root).local(ref) if root else None
    if m is None:
        raise FileNotFoundError(f"model {ref} is not in the model store ({root}); nothing is fetched automatically")
    t = os.environ.get("BRAIN_QWEN_TOKENIZER") or m.tokenizer or os.path.join(m.dir, "tokenizer.json")
    return m.weights, t, m.adapter, str(ref)


def load_llm_from_env(device: str = "auto") -> Optional[LlmResident]:
    sel = resolve_env_model()
    if sel is None:
        return None
    w, t, adapter, served_id = sel
    import torch
    from ..checkpoint import st
    from ..data.tokenizer import load_tokenizer
    from ..train import pick_device
    dev = pick_device(device)
    model, _, card = st.load_model(w, device=dev, dtype=torch.bfloat16 if dev.type == "cuda" else torch.float32)
    if adapter:
        from ..models.lora import fold_adapter_into
        tens, acfg, _ = st.load(adapter)
        fold_adapter_into(model, {k: v.to(dev) for k, v in tens.items()}, int(acfg["rank"]),
                          float(acfg.get("alpha", acfg["rank"])))
    model.eval()
    mode = "int8" if os.environ.get("BRAIN_QWEN_INT8") == "1" and dev.type == "cuda" else "bf16"
    kv8 = os.environ.get("BRAIN_QWEN_KV_INT8") == "1"
    clip = None
    if kv8 and os.environ.get("BRAIN_QWEN_KV_CALIB") == "1":
        from ..serve.calib import load_kv_clip
        clip = load_kv_clip(w)
    mid = served_id or (card.id if card is not None and card.id else "brain/qwen3")
    return LlmResident(model, load_tokenizer(t), mid, weights=mode, kv_dtype="int8" if kv8 else "bf16", kv_clip=clip)


def registry_from_env(load: bool = True, device: str = "auto") -> Dict[str, ResidentModel]:
    """Models selected by the environment: ``BRAIN_MOCK`` (non-empty), ``BRAIN_QWEN_WEIGHTS`` (a
    checkpoint file) or ``BRAIN_MODEL`` (a reference into the model store).
    ``load=False`` lists what would be served without reading weights (for ``brain caps``)."""
    reg: Dict[str, ResidentModel] = {}
    if os.environ.get("BRAIN_MOCK"):
        reg[MockResident.id] = MockResident()
    if os.environ.get("BRAIN_GPT_WEIGHTS"):
        if load:
            g = load_gpt(os.environ["BRAIN_GPT_WEIGHTS"], device)
            reg[g.id] = g
        else:
            class _GptStub(ResidentModel):
                id = "brain/gpt2"

                def manifest(self):
                    return Manifest(self.id, "GPT-2 style decoder (character vocabulary)",
                                    [generate_spec("character-level text continuation")])
            reg[_GptStub.id] = _GptStub()
    if os.environ.get("BRAIN_QWEN_WEIGHTS") or os.environ.get("BRAIN_MODEL"):
        if load:
            m = load_llm_from_env(device)
            reg[m.id] = m
        else:
            class _Stub(ResidentModel):
                id = os.environ.get("BRAIN_MODEL") or "brain/qwen3"

                def manifest(self):
                    return Manifest(self.id, "Qwen-family decoder", [generate_spec("chat / text generation")])
            reg[_Stub.id] = _Stub()
    return reg
