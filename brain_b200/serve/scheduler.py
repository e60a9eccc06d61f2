"""Continuous-batching scheduler (native core in csrc/runtime/serving.cpp) driving a paged decoder.

Per ``step``: admit waiting requests FIFO while their whole budget (prompt + max_new) fits the free
KV blocks and the prefill-token budget (2 x max_prefill, always at least one request) remains,
evicting LRU prefix-cache blocks first; run the planned prefill chunks (first token sampled when a
prompt completes); run ONE batched decode over every running sequence (a window of k on-device
greedy steps when the wait queue is empty and all are greedy); reap finished sequences (EOS is not
appended; blocks are released, prompt blocks stay in the prefix cache).
Reference: crates/model/src/serve.rs:374-776 (Scheduler), :262-307 (admission policies)."""
from __future__ import annotations

import ctypes
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Protocol, Sequence, Tuple

import numpy as np

from .. import _host
from ..data.rng import Rng
from .sampling import SampleParams, sample_from_topk

c = ctypes
_host.register({
    "bbh_sched_new": (c.c_void_p, [c.c_uint32] * 6 + [c.c_int64, c.c_uint32, c.c_int, c.c_double, c.c_int]),
    "bbh_sched_free": (None, [c.c_void_p]),
    "bbh_sched_submit": (c.c_int64, [c.c_void_p, c.c_void_p, c.c_uint32, c.c_uint32, c.c_float,
                                     c.c_uint32, c.c_float, c.c_uint64, c.c_int]),
    "bbh_sched_last_need": (c.c_uint64, [c.c_void_p]),
    "bbh_sched_last_bad_token": (c.c_uint64, [c.c_void_p]),
    "bbh_sched_cancel": (c.c_int, [c.c_void_p, c.c_int64]),
    "bbh_sched_idle": (c.c_int, [c.c_void_p]),
    "bbh_sched_plan": (None, [c.c_void_p, c.POINTER(c.c_uint32), c.POINTER(c.c_uint32), c.POINTER(c.c_uint32)]),
    "bbh_sched_prefill_item": (None, [c.c_void_p, c.c_uint32, c.POINTER(c.c_int64), c.POINTER(c.c_uint32),
                                      c.POINTER(c.c_uint32), c.POINTER(c.c_int)]),
    "bbh_sched_decode_batch": (None, [c.c_void_p, c.c_void_p, c.c_void_p, c.c_void_p, c.c_void_p, c.c_uint32]),
    "bbh_sched_commit_prefill": (None, [c.c_void_p, c.c_int64, c.c_uint32, c.c_int, c.c_uint32]),
    "bbh_sched_commit_decode": (None, [c.c_void_p, c.c_void_p, c.c_uint32, c.c_uint32]),
    "bbh_sched_seq_info": (c.c_int, [c.c_void_p, c.c_int64, c.POINTER(c.c_int), c.POINTER(c.c_int),
                                     c.POINTER(c.c_uint32), c.POINTER(c.c_uint32), c.POINTER(c.c_uint32),
                                     c.POINTER(c.c_uint32), c.POINTER(c.c_float), c.POINTER(c.c_uint32),
                                     c.POINTER(c.c_float), c.POINTER(c.c_uint64)]),
    "bbh_sched_seq_output": (None, [c.c_void_p, c.c_int64, c.c_void_p]),
    "bbh_sched_seq_prompt": (None, [c.c_void_p, c.c_int64, c.c_void_p]),
    "bbh_sched_seq_table": (c.c_uint32, [c.c_void_p, c.c_int64, c.c_void_p, c.c_uint32]),
    "bbh_sched_forget": (None, [c.c_void_p, c.c_int64]),
    "bbh_sched_decode_all_greedy": (c.c_int, [c.c_void_p]),
    "bbh_sched_set_admit": (None, [c.c_void_p, c.c_uint32, c.c_uint32]),
    "bbh_sched_set_prefill_budget": (None, [c.c_void_p, c.c_uint32]),
    "bbh_sched_step_report": (c.c_uint32, [c.c_void_p, c.c_void_p, c.c_void_p, c.c_void_p, c.c_uint32, c.c_void_p,
                                           c.c_uint32]),
    "bbh_sched_step_tokens": (c.c_uint32, [c.c_void_p]),
    "bbh_sched_set_service_ms": (None, [c.c_void_p, c.c_double]),
    "bbh_sched_set_prefill_rate": (None, [c.c_void_p, c.c_double]),
    "bbh_sched_pending_prefill": (c.c_uint64, [c.c_void_p]),
    "bbh_sched_stats": (None, [c.c_void_p, c.c_void_p]),
})

WAITING, RUNNING, FINISHED, CANCELLED = 0, 1, 2, 3
FINISH_NAMES = {0: None, 1: "stop", 2: "length"}


class RejectReason(Exception):
    """Raised by ``submit``; ``kind`` is one of exceeds_capacity / invalid_token / policy_rejected /
    empty_prompt.  The message of ``exceeds_capacity`` carries the numbers the HTTP layer maps to
    ``context_length_exceeded``."""

    def __init__(self, kind: str, msg: str):
        super().__init__(msg)
        self.kind = kind


class PagedDecoder(Protocol):
    """What the scheduler needs from a model engine."""

    vocab: int
    block_size: int
    num_blocks: int
    max_prefill_tokens: int
    max_seq_len: int
    topk_capacity: int

    def prefill_chunk(self, tokens: np.ndarray, start: int, block_table: np.ndarray, last: bool,
                      greedy: bool): ...
    def decode(self, tokens: np.ndarray, positions: np.ndarray, block_tables: np.ndarray,
               window: int, greedy: bool): ...


@dataclass
class StepReport:
    admitted: int = 0
    prefill_tokens: int = 0
    decoded: int = 0
    window: int = 1
    mixed: bool = False            # prompt chunks and the decode batch shared one forward
    finished: List[int] = field(default_factory=list)
    new_tokens: Dict[int, List[int]] = field(default_factory=dict)


@dataclass
class SeqInfo:
    state: int
    finish: Optional[str]
    n_prompt: int
    n_out: int
    prefilled: int
    prefix_hit: int
    params: SampleParams
    seed: int


class Scheduler:
    def __init__(self, decoder: PagedDecoder, max_batch: int = 16, eos: Optional[int] = None,
                 window: int = 4, policy: str = "unbounded_queue", policy_arg: float = 0.0,
                 prefix_cache: bool = True, admit_batch: int = 1, admit_max_wait: int = 64,
                 prefill_budget: int = 0, mixed: bool = False):
        """``admit_batch`` > 1 batches admissions: new requests join only once that many slots are
        free (or ``admit_max_wait`` steps passed), trading a little queueing delay for far fewer
        prefill-carrying steps under a saturated closed loop.  ``mixed``: a step that carries both
        prompt chunks and a decode batch runs them as ONE forward when the decoder offers
        ``mixed_step`` (one set of per-layer launches and all-reduces instead of two).

        Admission policies (``policy`` / ``policy_arg``): ``max_queue_depth`` rejects once that many
        requests wait; ``deadline_aware`` rejects while queue length x mean time in the system
        exceeds ``policy_arg`` ms; ``ttft_budget`` rejects a request whose first token, at the
        measured prefill rate, would come later than ``policy_arg`` ms (prompt tokens queued and
        mid-prefill ahead of it plus its own).  Both measured quantities are running means that
        ``step`` keeps from its own clock; nothing is rejected before the first measurement."""
        self.dec = decoder
        self.mixed = bool(mixed)
        pol = {"unbounded_queue": 0, "max_queue_depth": 1, "deadline_aware": 2, "ttft_budget": 3}[policy]
        self._measure = pol >= 2
        self.clock = time.perf_counter      # replaceable (tests drive a synthetic clock)
        self._t_submit: Dict[int, float] = {}
        self.service_ms = 0.0               # running mean: submit -> finished
        self.prefill_tokens_per_ms = 0.0    # running mean over steps that carried prompt tokens
        self.max_blocks = (decoder.max_seq_len + decoder.block_size - 1) // decoder.block_size
        self._h = _host.lib().bbh_sched_new(
            decoder.num_blocks, decoder.block_size, max_batch, decoder.max_prefill_tokens,
            decoder.max_seq_len, decoder.vocab, -1 if eos is None else int(eos), window, pol,
            float(policy_arg), int(prefix_cache))
        if not self._h:
            raise ValueError("invalid scheduler configuration")
        if admit_batch > 1:
            _host.lib().bbh_sched_set_admit(self._h, int(admit_batch), int(admit_max_wait))
        if prefill_budget > 0:      # prompt tokens per step (default 2 x max_prefill)
            _host.lib().bbh_sched_set_prefill_budget(self._h, int(prefill_budget))
        self._rngs: Dict[int, Rng] = {}
        self.max_batch = max_batch

    def __del__(self):
        try:
            if getattr(self, "_h", None):
                _host.lib().bbh_sched_free(self._h)
                self._h = None
        except Exception:      # interpreter shutdown: the library handle may already be gone
            pass

    # ------------------------------------------------------------------ queue
    def submit(self, prompt: Sequence[int], max_new: int, params: Optional[SampleParams] = None,
               seed: int = 0, ignore_eos: bool = False) -> int:
        params = params or SampleParams.greedy()
        p = np.ascontiguousarray(np.asarray(prompt, dtype=np.int64))
        if p.size and (p.min() < 0 or p.max() >= self.dec.vocab):
            bad = int(p[(p < 0) | (p >= self.dec.vocab)][0])
            raise RejectReason("invalid_token", f"token {bad} is outside the vocabulary of {self.dec.vocab}")
        p = p.astype(np.uint32)
        rid = int(_host.lib().bbh_sched_submit(self._h, p.ctypes.data, p.size, int(max_new),
                                               float(params.temp), int(params.top_k),
                                               float(params.top_p), int(seed), int(ignore_eos)))
        if rid == -1:
            need = int(_host.lib().bbh_sched_last_need(self._h))
            raise RejectReason("exceeds_capacity",
                               f"needs {need} tokens, engine capacity is {self.dec.max_seq_len}")
        if rid == -2:
            bad = int(_host.lib().bbh_sched_last_bad_token(self._h))
            raise RejectReason("invalid_token", f"token {bad} is outside the vocabulary of {self.dec.vocab}")
        if rid == -3:
            raise RejectReason("policy_rejected", "admission policy rejected the request")
        if rid == -4:
            raise RejectReason("empty_prompt", "empty prompt")
        self._rngs[rid] = Rng(seed)
        if self._measure:
            self._t_submit[rid] = self.clock()
        return rid

    def cancel(self, rid: int) -> List[int]:
        toks = self.tokens_of(rid)
        _host.lib().bbh_sched_cancel(self._h, rid)
        self._t_submit.pop(rid, None)
        return toks

    def is_idle(self) -> bool:
        return bool(_host.lib().bbh_sched_idle(self._h))

    def info(self, rid: int) -> SeqInfo:
        st, fin = c.c_int(), c.c_int()
        a, b, d, e, k = (c.c_uint32() for _ in range(5))
        t, p = c.c_float(), c.c_float()
        s = c.c_uint64()
        if _host.lib().bbh_sched_seq_info(self._h, rid, c.byref(st), c.byref(fin), c.byref(a), c.byref(b),
                                          c.byref(d), c.byref(e), c.byref(t), c.byref(k), c.byref(p),
                                          c.byref(s)) != 0:
            raise KeyError(rid)
        return SeqInfo(st.value, FINISH_NAMES[fin.value], a.value, b.value, d.value, e.value,
                       SampleParams(t.value, k.value, p.value), s.value)

    def tokens_of(self, rid: int) -> List[int]:
        n = self.info(rid).n_out
        out = np.empty(max(n, 1), dtype=np.uint32)
        _host.lib().bbh_sched_seq_output(self._h, rid, out.ctypes.data)
        return out[:n].tolist()

    def forget(self, rid: int) -> None:
        _host.lib().bbh_sched_forget(self._h, rid)
        self._rngs.pop(rid, None)

    def stats(self) -> Dict[str, int]:
        out = np.zeros(12, dtype=np.uint64)
        _host.lib().bbh_sched_stats(self._h, out.ctypes.data)
        names = ["free_blocks", "num_blocks", "waiting", "running", "steps", "submitted", "finished",
                 "cancelled", "generated", "kv_prefix_hit_tokens", "kv_prefix_lookup_tokens",
                 "prefix_entries"]
        return {n: int(v) for n, v in zip(names, out)}

    # ------------------------------------------------------------------ step
    def _pick(self, rid: int, greedy_tok, topk) -> int:
        info = self.info(rid)
        if info.params.is_greedy() or topk is None:
            return int(greedy_tok)
        return sample_from_topk(topk, info.params, self._rngs[rid])

    def pending_prefill_tokens(self) -> int:
        """Prompt tokens queued or mid-prefill (what a new request's first token waits for)."""
        return int(_host.lib().bbh_sched_pending_prefill(self._h))

    def _update_measurements(self, rep: "StepReport", t0: float) -> None:
        """Feed the admission policies: a step's prompt tokens over its duration (decode rows that
        shared the step count as prefill time, which errs toward rejecting), and the time each
        finished request spent in the system."""
        lib = _host.lib()
        now = self.clock()
        ms = (now - t0) * 1e3
        if rep.prefill_tokens and ms > 0:
            rate = rep.prefill_tokens / ms
            self.prefill_tokens_per_ms = rate if self.prefill_tokens_per_ms == 0 else \
                0.8 * self.prefill_tokens_per_ms + 0.2 * rate
            lib.bbh_sched_set_prefill_rate(self._h, self.prefill_tokens_per_ms)
        for rid in rep.finished:
            ts = self._t_submit.pop(rid, None)
            if ts is not None:
                took = (now - ts) * 1e3
                self.service_ms = took if self.service_ms == 0 else 0.8 * self.service_ms + 0.2 * took
                lib.bbh_sched_set_service_ms(self._h, self.service_ms)

    def step(self) -> StepReport:
        lib = _host.lib()
        t_step = self.clock() if self._measure else 0.0
        npf, nd, win = c.c_uint32(), c.c_uint32(), c.c_uint32()
        lib.bbh_sched_plan(self._h, c.byref(npf), c.byref(nd), c.byref(win))
        rep = StepReport(window=win.value)
        # ---- prefill chunks (packed into one forward when the decoder can)
        plan = []
        for i in range(npf.value):
            rid, s, e, last = c.c_int64(), c.c_uint32(), c.c_uint32(), c.c_int()
            lib.bbh_sched_prefill_item(self._h, i, c.byref(rid), c.byref(s), c.byref(e), c.byref(last))
            rid_v = rid.value
            info = self.info(rid_v)
            prompt = np.empty(info.n_prompt, dtype=np.uint32)
            lib.bbh_sched_seq_prompt(self._h, rid_v, prompt.ctypes.data)
            bt = np.full(self.max_blocks, -1, dtype=np.int32)
            lib.bbh_sched_seq_table(self._h, rid_v, bt.ctypes.data, self.max_blocks)
            plan.append((rid_v, s.value, e.value, bool(last.value), info.params.is_greedy(),
                         prompt[s.value:e.value].astype(np.int32), bt))
            if s.value == info.prefix_hit:
                rep.admitted += 1
            rep.prefill_tokens += e.value - s.value
        n = nd.value
        ids = toks = pos = bts = None
        if n:
            ids = np.empty(n, dtype=np.int64)
            toks = np.empty(n, dtype=np.int32)
            pos = np.empty(n, dtype=np.int32)
            bts = np.empty((n, self.max_blocks), dtype=np.int32)
            lib.bbh_sched_decode_batch(self._h, ids.ctypes.data, toks.ctypes.data, pos.ctypes.data,
                                       bts.ctypes.data, self.max_blocks)
        all_greedy = bool(lib.bbh_sched_decode_all_greedy(self._h)) if n else True
        outs = decoded = None
        mixed = getattr(self.dec, "mixed_step", None) if self.mixed else None
        if plan and n and mixed is not None and win.value == 1:
            # the decode set was fixed by the plan, so both kinds of rows can share one forward
            g = all_greedy and all(p[4] for p in plan if p[3])
            outs, g_toks, topks = mixed([(p[5], p[1], p[6], p[3], p[4]) for p in plan], toks, pos, bts, g)
            decoded = (g_toks, topks)
            rep.mixed = True
        elif plan:
            batch = getattr(self.dec, "prefill_batch", None)
            if batch is not None and len(plan) > 1:
                outs = batch([(p[5], p[1], p[6], p[3], p[4]) for p in plan])
            else:
                outs = [self.dec.prefill_chunk(p[5], p[1], p[6], p[3], p[4]) for p in plan]
        if n and decoded is None:
            decoded = self.dec.decode(toks, pos, bts, win.value, all_greedy)
        # the tokens were read back, so the device is idle: one look at the error word before the
        # commits.  A kernel whose bounded wait ran out raises here and the caller fails the step's
        # requests instead of committing garbage tokens.
        chk = getattr(self.dec, "check_device", None)
        if chk is not None and (plan or n):
            chk()
        if plan:
            for p, (tok, topk) in zip(plan, outs):
                if p[3]:
                    lib.bbh_sched_commit_prefill(self._h, p[0], p[2], 1, self._pick(p[0], tok, topk))
                else:
                    lib.bbh_sched_commit_prefill(self._h, p[0], p[2], 0, 0)
        # ---- one batched decode
        if n:
            greedy_toks, topks = decoded
            if all_greedy:
                out = np.ascontiguousarray(np.asarray(greedy_toks, dtype=np.uint32).reshape(n, win.value))
            else:
                out = np.empty((n, win.value), dtype=np.uint32)
                for i, r in enumerate(ids):
                    out[i, 0] = self._pick(int(r), greedy_toks[i][0], topks[i] if topks is not None else None)
            lib.bbh_sched_commit_decode(self._h, out.ctypes.data, n, win.value)
            rep.decoded = n
        # ---- report: what this step's commits produced, fetched in one native call
        ne = int(lib.bbh_sched_step_report(self._h, None, None, None, 0, None, 0))
        if ne:
            nt = max(int(lib.bbh_sched_step_tokens(self._h)), 1)
            e_ids = np.empty(ne, dtype=np.int64)
            e_new = np.empty(ne, dtype=np.uint32)
            e_fin = np.empty(ne, dtype=np.int32)
            e_tok = np.empty(nt, dtype=np.uint32)
            lib.bbh_sched_step_report(self._h, e_ids.ctypes.data, e_new.ctypes.data, e_fin.ctypes.data, ne,
                                      e_tok.ctypes.data, nt)
            t = 0
            tok_list = e_tok.tolist()
            for rid_v, k, fin in zip(e_ids.tolist(), e_new.tolist(), e_fin.tolist()):
                if k:
                    prev = rep.new_tokens.get(rid_v)
                    rep.new_tokens[rid_v] = (prev + tok_list[t:t + k]) if prev else tok_list[t:t + k]
                    t += k
                if fin and rid_v not in rep.finished:
                    rep.finished.append(rid_v)
        if self._measure:
            self._update_measurements(rep, t_step)
        return rep

    def run_until_idle(self, max_steps: int = 1 << 30) -> None:
        steps = 0
        while not self.is_idle() and steps < max_steps:
            self.step()
            steps += 1
