"""Which models are loaded, where, and what happens when memory runs out (reference:
crates/residency/src/lib.rs:34-129 — per-device budgets, least-recently-used eviction of idle
residents, placement on the device with the most room, ``ModelSupplier``s that load on first use;
nothing is ever fetched here: a supplier reads a file that is already on disk).

A ``Supplier`` knows a model's id, what it will cost in device memory, how to describe it without
loading it (``stub``) and how to load it.  ``Residency.acquire`` returns a loaded model and pins it
until the matching ``release``; loading evicts idle residents in least-recently-used order when the
budget of the chosen device would be exceeded, and fails with ``InsufficientMemory`` when even
that is not enough (a model in use is never evicted)."""
from __future__ import annotations

import threading
import time
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional

from ..utils import trace
from .capability import Manifest, generate_spec
from .resident import ResidentModel


class InsufficientMemory(RuntimeError):
    pass


class Supplier:
    id: str = ""

    def estimate_bytes(self) -> int:
        raise NotImplementedError

    def stub(self) -> ResidentModel:
        """Manifest / context length without weights (model listings, request validation)."""
        raise NotImplementedError

    def load(self, device: str) -> ResidentModel:
        raise NotImplementedError


class _Stub(ResidentModel):
    def __init__(self, mid: str, summary: str, ctx: Optional[int]):
        self.id, self._summary, self._ctx = mid, summary, ctx

    def manifest(self) -> Manifest:
        return Manifest(self.id, self._summary, [generate_spec("chat / text generation")], self._ctx)

    def context_length(self):
        return self._ctx


class StoreSupplier(Supplier):
    """A model of the on-disk store (``modelstore.LocalModel``), served by the paged-KV engine."""

    def __init__(self, local, ctx: Optional[int] = None, max_batch: Optional[int] = None, weights: str = "bf16",
                 kv_dtype: str = "bf16"):
        self.local = local
        self.id = str(local.reference)
        self.ctx, self.max_batch, self.weights, self.kv_dtype = ctx, max_batch, weights, kv_dtype
        card = local.card
        self._ctx_card = getattr(card, "context_length", None) if card is not None else None

    def estimate_bytes(self) -> int:
        import os
        from ..checkpoint.st import WeightReader
        n = 0
        with WeightReader(self.local.weights) as r:        # header only
            for name in r.names():
                k = 1
                for d in r.shape(name):
                    k *= d
                n += k
        per = 1 if self.weights == "int8" else 2
        return n * per + (os.path.getsize(self.local.adapter) if self.local.adapter else 0)

    def stub(self) -> ResidentModel:
        return _Stub(self.id, "Qwen-family decoder (loaded on first use)", self.ctx or self._ctx_card)

    def load(self, device: str) -> ResidentModel:
        import torch
        from ..checkpoint import st
        from ..data.tokenizer import load_tokenizer
        from ..train import pick_device
        from .resident import LlmResident
        dev = pick_device(device)
        model, _, _ = st.load_model(self.local.weights, device=dev,
                                    dtype=torch.bfloat16 if dev.type == "cuda" else torch.float32)
        if self.local.adapter:
            from ..models.lora import fold_adapter_into
            tens, acfg, _ = st.load(self.local.adapter)
            fold_adapter_into(model, {k: v.to(dev) for k, v in tens.items()}, int(acfg["rank"]),
                              float(acfg.get("alpha", acfg["rank"])))
        model.eval()
        tok = load_tokenizer(self.local.tokenizer or self.local.dir)
        return LlmResident(model, tok, self.id, ctx=self.ctx, max_batch=self.max_batch,
                           weights=self.weights if dev.type == "cuda" else "bf16", kv_dtype=self.kv_dtype)


@dataclass
class _Entry:
    model: ResidentModel
    device: str
    nbytes: int
    in_use: int = 0
    last_used: float = 0.0
    pinned: bool = False


class Residency:
    def __init__(self, suppliers: Dict[str, Supplier], budgets: Dict[str, int],
                 pinned: Optional[Dict[str, ResidentModel]] = None,
                 on_evict: Optional[Callable[[str, ResidentModel], None]] = None, busy_wait_s: float = 0.0):
        """``budgets``: device name -> bytes available to models.  ``pinned``: models that are
        resident from the start, cost nothing against the budgets and are never evicted."""
        self.suppliers = dict(suppliers)
        self.budgets = dict(budgets)
        self.entries: Dict[str, _Entry] = {}
        self.on_evict = on_evict
        #: how long a load may wait for a busy resident to go idle when nothing can be evicted
        #: (0: fail at once with InsufficientMemory; a server sets a few seconds)
        self.busy_wait_s = float(busy_wait_s)
        self._lock = threading.Lock()
        self._freed = threading.Condition(self._lock)    # signalled when a resident becomes idle
        self._loading: Dict[str, threading.Event] = {}
        self.loads = self.evictions = 0
        # eviction order: decayed request count per model (half-life 32 requests of any model), so a
        # burst of one-off requests for the cold tail does not push out the models everybody uses;
        # ties fall back to least recently used
        self._heat: Dict[str, float] = {}
        self._heat_tick: Dict[str, int] = {}
        self._tick = 0
        for mid, m in (pinned or {}).items():
            self.entries[mid] = _Entry(m, "-", 0, pinned=True)

    # ---- queries
    def known(self) -> List[str]:
        return sorted(set(self.entries) | set(self.suppliers))

    def resident(self) -> List[str]:
        return sorted(self.entries)

    def describe(self, mid: str) -> Optional[ResidentModel]:
        """The loaded model, else its supplier's stub, else None."""
        e = self.entries.get(mid)
        if e is not None:
            return e.model
        s = self.suppliers.get(mid)
        return s.stub() if s is not None else None

    def used(self, device: str) -> int:
        return sum(e.nbytes for e in self.entries.values() if e.device == device)

    def stats(self) -> Dict:
        return {"resident": {k: {"device": e.device, "bytes": e.nbytes, "in_use": e.in_use, "pinned": e.pinned}
                             for k, e in self.entries.items()},
                "budgets": dict(self.budgets), "loads": self.loads, "evictions": self.evictions}

    def _touch(self, mid: str) -> None:
        self._tick += 1
        self._heat[mid] = self._heat_now(mid) + 1.0
        self._heat_tick[mid] = self._tick

    def _heat_now(self, mid: str) -> float:
        return self._heat.get(mid, 0.0) * 0.5 ** ((self._tick - self._heat_tick.get(mid, self._tick)) / 32.0)

    # ---- placement / eviction (call with the lock held)
    def _place(self, need: int) -> Optional[str]:
        """The device with the most free budget that can hold ``need`` bytes, evicting idle residents
        (least recently used first) where necessary; None when no device can."""
        order = sorted(self.budgets, key=lambda d: self.budgets[d] - self.used(d), reverse=True)
        for dev in order:
            if self.budgets[dev] - self.used(dev) >= need:
                return dev
        for dev in order:
            if need > self.budgets[dev]:
                continue
            idle = sorted((round(self._heat_now(k), 3), e.last_used, k) for k, e in self.entries.items()
                          if e.device == dev and e.in_use == 0 and not e.pinned)
            freed, victims = self.budgets[dev] - self.used(dev), []
            for _, _, k in idle:
                if freed >= need:
                    break
                victims.append(k)
                freed += self.entries[k].nbytes
            if freed >= need:
                for k in victims:
                    self._evict(k)
                return dev
        return None

    def _evict(self, mid: str) -> None:
        e = self.entries.pop(mid)
        self.evictions += 1
        trace.event("residency", 3, "evict", model=mid, device=e.device, bytes=e.nbytes)
        if self.on_evict is not None:
            self.on_evict(mid, e.model)
        try:
            e.model.close()
        except Exception:   # noqa: BLE001 - an eviction must not fail the request that caused it
            pass

    # ---- acquire / release
    def acquire(self, mid: str, timeout_s: float = 180.0) -> ResidentModel:
        deadline = time.time() + timeout_s
        with self._lock:
            self._touch(mid)
        while True:
            with self._lock:
                e = self.entries.get(mid)
                if e is not None:
                    e.in_use += 1
                    e.last_used = time.time()
                    return e.model
                sup = self.suppliers.get(mid)
                if sup is None:
                    raise KeyError(mid)
                waiter = self._loading.get(mid)
                if waiter is None:
                    self._loading[mid] = threading.Event()
                    break
            if not waiter.wait(max(deadline - time.time(), 0.0)):
                raise TimeoutError(f"model '{mid}' was still loading after {timeout_s:.0f} s")
        # this thread loads; others wait on the event
        try:
            need = int(sup.estimate_bytes())
            with self._lock:
                dev = self._place(need)
                # every candidate victim is busy right now: a model that fits some device's budget
                # waits for a resident to go idle instead of failing the request
                give_up = min(deadline, time.time() + self.busy_wait_s)
                while dev is None and any(need <= b for b in self.budgets.values()) and time.time() < give_up:
                    self._freed.wait(min(0.05, max(give_up - time.time(), 0.0)))
                    dev = self._place(need)
            if dev is None:
                raise InsufficientMemory(f"model '{mid}' needs {need / 2**30:.2f} GiB; no device has that much "
                                         "free even after evicting every idle model")
            t0 = time.time()
            model = sup.load(dev)
            trace.event("residency", 3, "load", model=mid, device=dev, bytes=need, seconds=time.time() - t0)
            with self._lock:
                self.entries[mid] = _Entry(model, dev, need, in_use=1, last_used=time.time())
                self.loads += 1
            return model
        finally:
            with self._lock:
                self._loading.pop(mid).set()

    def release(self, mid: str) -> None:
        with self._lock:
            e = self.entries.get(mid)
            if e is not None and e.in_use > 0:
                e.in_use -= 1
                e.last_used = time.time()
                if e.in_use == 0:
                    self._freed.notify_all()

    def close(self) -> None:
        with self._lock:
            for mid in [k for k, e in self.entries.items() if not e.pinned]:
                self._evict(mid)
