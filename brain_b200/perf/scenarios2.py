"""Tier-2 scenarios that exercise the layers AROUND the engine (reference:
crates/perf/src/scenarios/{residency,placement,frontend}.rs, listed at scenarios/mod.rs:135-137):

* ``residency``  a catalogue several times larger than the device budget served by ONE residency
  manager under Zipf popularity that is re-rolled mid-run: aggregate goodput, warm vs cold
  time-to-first-artifact, eviction regret (evicted and needed again soon) and Jain fairness
  across models, so a policy that pins the hot head and starves the tail fails visibly.
* ``placement``  the same workload on each device alone and on the mix the placer chooses:
  ``placement_efficiency = observed / best single device`` (above 1: the mix really shared work).
* ``frontend``   host-side stages (tokenise, chat template, JSONL encode / decode, detokenise,
  stream flush) timed per request: host cores needed to keep one device saturated at a given
  request rate.

All three run on the real ``api.residency.Residency`` / tokenizer / JSONL code with synthetic
models and text; none of them needs a GPU."""
from __future__ import annotations

import json
import math
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from typing import Callable, Dict, List, Optional, Sequence

from ..data.rng import Rng


def jain(xs: Sequence[float]) -> float:
    xs = [float(x) for x in xs]
    s, s2 = sum(xs), sum(x * x for x in xs)
    return (s * s) / (len(xs) * s2) if s2 > 0 else 1.0


def _pct(xs: List[float], q: float) -> Optional[float]:
    if not xs:
        return None
    xs = sorted(xs)
    return xs[min(len(xs) - 1, int(math.ceil(q * len(xs))) - 1)]


def _zipf(n: int, alpha: float) -> List[float]:
    w = [1.0 / (i + 1) ** alpha for i in range(n)]
    t = sum(w)
    return [x / t for x in w]


# ------------------------------------------------------------------------------------ residency
class _SynthModel:
    """A resident with a service time; ``close`` is what an eviction calls."""

    def __init__(self, mid: str, service_ms: float):
        self.id, self.service_ms, self.closed = mid, service_ms, False

    def max_concurrency(self) -> int:
        return 4

    def run(self) -> None:
        time.sleep(self.service_ms / 1e3)

    def close(self) -> None:
        self.closed = True


class _SynthSupplier:
    def __init__(self, mid: str, nbytes: int, load_ms: float, service_ms: float):
        self.id, self.nbytes, self.load_ms, self.service_ms = mid, nbytes, load_ms, service_ms
        self.loads = 0

    def estimate_bytes(self) -> int:
        return self.nbytes

    def stub(self):
        return _SynthModel(self.id, self.service_ms)

    def load(self, device: str):
        time.sleep(self.load_ms / 1e3)      # weight read + upload, proportional to size
        self.loads += 1
        return _SynthModel(self.id, self.service_ms)


def residency(n_models: int = 12, budget_models: float = 3.0, requests: int = 240, concurrency: int = 6,
              alpha: float = 1.1, seed: int = 0, load_ms_per_unit: float = 12.0, service_ms: float = 2.0,
              slo_cold_ms: float = 250.0, regret_window: int = 12) -> Dict:
    """Many models over one budget.  Pass: every request served, no model starved (each model that
    was asked for was served), fairness of per-model completion ratio >= 0.9, cold TTFA p99 within
    ``slo_cold_ms``, and eviction regret (evicted, then asked for again within ``regret_window``
    requests) below three quarters: with a working set twice the budget some regret is structural, a
    value near one means the cache thrashes."""
    from ..api.residency import InsufficientMemory, Residency
    rng = Rng(seed)
    unit = 1 << 20
    sizes = [unit * (1 + int(rng.next_u64() % 3)) for _ in range(n_models)]          # 1..3 units
    sups = {f"m{i}": _SynthSupplier(f"m{i}", sizes[i], load_ms_per_unit * sizes[i] / unit, service_ms)
            for i in range(n_models)}
    budget = int(budget_models * sum(sizes) / n_models)
    res = Residency(sups, {"dev0": budget}, busy_wait_s=5.0)
    order = list(range(n_models))
    pop = _zipf(n_models, alpha)
    plan = []
    for r in range(requests):
        if r == requests // 2:                    # traffic shift: the cold tail becomes the hot head
            order = order[::-1]
        u = (rng.next_u64() >> 11) / float(1 << 53)
        acc, pick = 0.0, n_models - 1
        for i, p in enumerate(pop):
            acc += p
            if u < acc:
                pick = i
                break
        plan.append(f"m{order[pick]}")
    lock = threading.Lock()
    asked: Dict[str, int] = {}
    served: Dict[str, int] = {}
    warm, cold, failed = [], [], 0
    evicted_at: Dict[str, int] = {}
    regrets = [0]
    seq = [0]
    prev_on_evict = res.on_evict

    def on_evict(mid, model):
        with lock:
            evicted_at[mid] = seq[0]
        if prev_on_evict:
            prev_on_evict(mid, model)
    res.on_evict = on_evict

    def one(mid: str):
        nonlocal failed
        with lock:
            asked[mid] = asked.get(mid, 0) + 1
            seq[0] += 1
            me = seq[0]
            if mid in evicted_at and me - evicted_at.pop(mid) <= regret_window:
                regrets[0] += 1                  # thrown out and needed again almost at once
        t0 = time.perf_counter()
        was_resident = mid in res.entries
        try:
            m = res.acquire(mid, timeout_s=10.0)
        except (InsufficientMemory, TimeoutError):
            with lock:
                failed += 1
            return
        try:
            ttfa = (time.perf_counter() - t0) * 1e3
            m.run()
        finally:
            res.release(mid)
        with lock:
            served[mid] = served.get(mid, 0) + 1
            (warm if was_resident else cold).append(ttfa)

    t0 = time.perf_counter()
    with ThreadPoolExecutor(max_workers=concurrency) as ex:
        list(ex.map(one, plan))
    wall = time.perf_counter() - t0
    st = res.stats()
    res.close()
    ratios = [served.get(m, 0) / asked[m] for m in asked]
    fairness = jain(ratios)
    regret = regrets[0] / max(st["evictions"], 1)
    out = {
        "scenario": "residency", "models": n_models, "budget_bytes": budget, "catalogue_bytes": sum(sizes),
        "oversubscription": round(sum(sizes) / budget, 2), "requests": requests, "served": sum(served.values()),
        "failed": failed, "goodput_per_s": round(sum(served.values()) / wall, 1),
        "loads": st["loads"], "evictions": st["evictions"], "hit_rate": round(len(warm) / max(len(warm) + len(cold), 1), 3),
        "ttfa_warm_p50_ms": _pct(warm, 0.5), "ttfa_cold_p50_ms": _pct(cold, 0.5), "ttfa_cold_p99_ms": _pct(cold, 0.99),
        "eviction_regret": round(regret, 3), "fairness": round(fairness, 3),
        "starved_models": sorted(m for m in asked if served.get(m, 0) == 0),
    }
    out["passed"] = bool(failed == 0 and not out["starved_models"] and fairness >= 0.9
                         and (out["ttfa_cold_p99_ms"] or 0.0) <= slo_cold_ms and regret < 0.75
                         and out["oversubscription"] >= 3.0)
    return out


# ------------------------------------------------------------------------------------ placement
def placement(device_rates: Optional[Dict[str, float]] = None, requests: int = 160, work_units: float = 1.0,
              seed: int = 0) -> Dict:
    """Measure each device alone, then the mix through the residency manager's placer (which puts a
    model on the device with the most free budget): efficiency = mixed goodput / best single."""
    from ..api.residency import Residency
    rates = dict(device_rates or {"gpu0": 400.0, "gpu1": 400.0, "cpu": 40.0})      # work units per second

    def run(devs: List[str]) -> float:
        # one replica of the model per device it is placed on; a request goes to the least-loaded replica
        sups = {f"replica-{i}": _SynthSupplier(f"replica-{i}", 1 << 20, 1.0, 0.0) for i in range(len(devs))}
        res = Residency(sups, {d: 1 << 20 for d in devs})
        placed = {}
        for mid in sups:
            res.acquire(mid)
            placed[mid] = res.entries[mid].device
            res.release(mid)
        load = {mid: 0.0 for mid in sups}
        lock = threading.Lock()

        def one(_):
            with lock:
                # expected finish time if sent to each replica: the placer's oracle-free heuristic
                mid = min(load, key=lambda m: (load[m] + work_units) / rates[placed[m]])
                load[mid] += work_units
            time.sleep(work_units / rates[placed[mid]])
            with lock:
                load[mid] -= work_units
        t0 = time.perf_counter()
        with ThreadPoolExecutor(max_workers=2 * len(devs)) as ex:
            list(ex.map(one, range(requests)))
        wall = time.perf_counter() - t0
        res.close()
        assert sorted(placed.values()) == sorted(devs), "the placer must spread replicas over the devices"
        return requests / wall

    single = {d: run([d]) for d in rates}
    mixed = run(list(rates))
    best = max(single.values())
    eff = mixed / best
    return {"scenario": "placement", "single_goodput_per_s": {k: round(v, 1) for k, v in single.items()},
            "mixed_goodput_per_s": round(mixed, 1), "placement_efficiency": round(eff, 3),
            "passed": bool(eff >= 1.2)}    # two equal fast devices + a slow one must beat the best single one clearly


# ------------------------------------------------------------------------------------ frontend
def frontend(requests: int = 200, prompt_words: int = 180, out_tokens: int = 128, device_rate_per_s: float = 200.0,
             seed: int = 0) -> Dict:
    """Per-request host cost of every front-end stage on this machine and the host cores needed to
    keep one device busy at ``device_rate_per_s`` requests per second."""
    from ..data.tokenizer import BpeTokenizer, bytes_to_unicode, render_chatml
    rng = Rng(seed)
    words = ["alpha", "beta", "gamma", "delta", "tensor", "kernel", "stream", "token", "cache", "block"]
    # a byte-level BPE (the native merge loop the servers use) whose merges build these words
    b2u = bytes_to_unicode()
    vocab = {b2u[b]: b for b in range(256)}
    merges = []
    for w in words:
        for pre in (" " + w, w):
            sym = [b2u[b] for b in pre.encode()]
            cur = sym[0]
            for nxt in sym[1:]:
                if cur + nxt not in vocab:
                    vocab[cur + nxt] = len(vocab)
                    merges.append((cur, nxt))
                cur += nxt
    tok = BpeTokenizer(vocab, merges, special={"<|im_start|>": len(vocab), "<|im_end|>": len(vocab) + 1})
    stages: Dict[str, List[float]] = {k: [] for k in ("chat_template", "tokenise", "jsonl_decode", "jsonl_encode",
                                                       "detokenise", "stream_flush")}

    def timed(name, fn):
        t0 = time.perf_counter()
        r = fn()
        stages[name].append((time.perf_counter() - t0) * 1e6)
        return r

    class _Sink:
        def __init__(self):
            self.n = 0

        def write(self, b):
            self.n += len(b)

        def flush(self):
            pass
    sink = _Sink()
    for _ in range(requests):
        text = " ".join(words[int(rng.next_u64() % len(words))] for _ in range(prompt_words))
        line = json.dumps({"id": 1, "method": "invoke", "params": {"model": "m", "action": "chat",
                                                                     "input": {"messages": [{"role": "user", "content": text}]}}})
        req = timed("jsonl_decode", lambda: json.loads(line))
        msgs = req["params"]["input"]["messages"]
        prompt = timed("chat_template", lambda: render_chatml(msgs, add_generation_prompt=True))
        ids = timed("tokenise", lambda: tok.encode(prompt))
        out_ids = [int(256 + rng.next_u64() % (len(vocab) - 256)) for _ in range(out_tokens)]
        pieces = timed("detokenise", lambda: [tok.decode([t]) for t in out_ids])
        frames = timed("jsonl_encode", lambda: [json.dumps({"id": 1, "event": "delta", "data": {"text": p}}) for p in pieces])

        def flush():
            for f in frames:
                sink.write(f.encode() + b"\n")
                sink.flush()
        timed("stream_flush", flush)
        assert len(ids) >= prompt_words
    per_stage = {k: round(sum(v) / len(v), 1) for k, v in stages.items()}
    total_us = sum(per_stage.values())
    cores = total_us * 1e-6 * device_rate_per_s
    worst = max(per_stage, key=per_stage.get)
    return {"scenario": "frontend", "requests": requests, "stage_us_per_request": per_stage,
            "host_us_per_request": round(total_us, 1), "device_rate_per_s": device_rate_per_s,
            "host_cores_per_saturated_device": round(cores, 3), "dominant_stage": worst,
            "passed": bool(total_us > 0 and sink.n > 0)}
