"""Executor: one lane per resident model, bounded concurrency, admission deadlines, failure
containment (reference: crates/residency/src/executor.rs:443-481 stats/in-flight accounting,
:1368,1450 lane panics converted to error replies while the lane survives;
crates/residency/src/admission.rs:21-37 — a request not admitted within its deadline is answered
"busy", the HTTP edge sheds load past 256 concurrent)."""
from __future__ import annotations

import threading
import time
from concurrent.futures import ThreadPoolExecutor
from dataclasses import dataclass, field
from typing import Callable, Dict, Optional

from ..utils import trace
from .capability import ActionError, Invocation, Outcome, Progress, ValidationError
from .resident import ResidentModel

ADMIT_DEADLINE_S = 10.0
COLD_ADMIT_DEADLINE_S = 180.0
EDGE_MAX_CONCURRENT = 256


class Busy(RuntimeError):
    """Not admitted before the deadline (HTTP 429) or shed at the edge (HTTP 503)."""

    def __init__(self, message: str, shed: bool = False):
        super().__init__(message)
        self.shed = shed


@dataclass
class LaneStats:
    submitted: int = 0
    completed: int = 0
    failed: int = 0
    cancelled: int = 0
    rejected: int = 0
    in_flight: int = 0
    busy_seconds: float = 0.0


class _Lane:
    def __init__(self, model: ResidentModel):
        self.model = model
        self.slots = threading.BoundedSemaphore(max(model.max_concurrency(), 1))
        self.stats = LaneStats()
        self.lock = threading.Lock()
        self.warm = False


class Executor:
    def __init__(self, models: Dict[str, ResidentModel], admit_deadline_s: float = ADMIT_DEADLINE_S,
                 edge_limit: int = EDGE_MAX_CONCURRENT, workers: int = 320, residency=None):
        """``models`` are resident from the start; ``residency`` (api.residency.Residency) adds models
        that are loaded on first use and evicted least-recently-used when memory runs out."""
        self.lanes = {mid: _Lane(m) for mid, m in models.items()}
        self.residency = residency
        if residency is not None:
            residency.on_evict = self._evicted
        self.admit_deadline_s = admit_deadline_s
        self.edge_limit = edge_limit
        self._edge = 0
        self._edge_lock = threading.Lock()
        self._lanes_lock = threading.Lock()
        self.pool = ThreadPoolExecutor(max_workers=workers, thread_name_prefix="lane")
        self.started = time.time()

    # ---- lookup
    def models(self) -> Dict[str, ResidentModel]:
        """Every model a request may name: loaded ones, and stubs of those loaded on first use."""
        out = {k: l.model for k, l in self.lanes.items()}
        if self.residency is not None:
            for mid in self.residency.known():
                if mid not in out:
                    out[mid] = self.residency.describe(mid)
        return out

    def get(self, model_id: str) -> Optional[ResidentModel]:
        lane = self.lanes.get(model_id)
        if lane:
            return lane.model
        return self.residency.describe(model_id) if self.residency is not None else None

    def _evicted(self, model_id: str, model) -> None:
        # only the lane of the model that was evicted goes: a request that raced the eviction and
        # already re-loaded the model holds a newer lane under the same id
        with self._lanes_lock:
            lane = self.lanes.get(model_id)
            if lane is not None and lane.model is model:
                self.lanes.pop(model_id, None)

    def _lane(self, model_id: str):
        """(lane, release) — loads the model through the residency manager when it is not resident."""
        lane = self.lanes.get(model_id)
        if lane is not None and (self.residency is None or model_id not in self.residency.suppliers):
            return lane, None
        if self.residency is None or model_id not in self.residency.known():
            raise KeyError(model_id)
        from .residency import InsufficientMemory
        try:
            model = self.residency.acquire(model_id, COLD_ADMIT_DEADLINE_S)
        except (InsufficientMemory, TimeoutError) as e:
            raise Busy(str(e))
        with self._lanes_lock:      # two first requests must share one lane (one semaphore, one stats)
            lane = self.lanes.get(model_id)
            if lane is None or lane.model is not model:
                lane = self.lanes[model_id] = _Lane(model)
        return lane, (lambda: self.residency.release(model_id))

    def in_flight(self) -> int:
        return self._edge

    def stats(self) -> Dict:
        out = {mid: vars(l.stats).copy() for mid, l in self.lanes.items()}
        if self.residency is not None:
            out["_residency"] = self.residency.stats()
        return out

    # ---- edge admission (called by the HTTP layer before any work)
    def edge_enter(self) -> None:
        with self._edge_lock:
            if self._edge >= self.edge_limit:
                raise Busy("server is at capacity", shed=True)
            self._edge += 1

    def edge_leave(self) -> None:
        with self._edge_lock:
            self._edge -= 1

    # ---- run (blocking; call from a worker thread)
    def run(self, model_id: str, action: str, inv: Invocation,
            progress: Optional[Callable[[Progress], None]] = None) -> Outcome:
        described = self.get(model_id)
        if described is None:
            raise KeyError(model_id)
        spec = described.manifest().action(action)
        if spec is None:
            raise ActionError(f"model '{model_id}' has no action '{action}'", "not_implemented")
        inv.params = spec.validate(inv.params, inv.blobs)     # before any load: a bad request costs nothing
        lane, release = self._lane(model_id)
        try:
            return self._run_on(lane, model_id, action, inv, progress)
        finally:
            if release is not None:
                release()

    def _run_on(self, lane, model_id: str, action: str, inv: Invocation,
                progress: Optional[Callable[[Progress], None]] = None) -> Outcome:
        deadline = self.admit_deadline_s if lane.warm else max(self.admit_deadline_s, COLD_ADMIT_DEADLINE_S)
        t0 = time.time()
        with lane.lock:
            lane.stats.submitted += 1
        got = False
        while time.time() - t0 < deadline:
            if lane.slots.acquire(timeout=0.05):
                got = True
                break
            if inv.cancel.is_cancelled():
                break
        if not got:
            with lane.lock:
                lane.stats.rejected += 1
            if inv.cancel.is_cancelled():
                raise ActionError("cancelled", "cancelled")
            raise Busy(f"model '{model_id}' did not admit the request within {deadline:.0f} s")
        with lane.lock:
            lane.stats.in_flight += 1
        t1 = time.time()
        try:
            out = lane.model.run(action, inv, progress or (lambda p: None))
            lane.warm = True
            with lane.lock:
                lane.stats.completed += 1
            return out
        except ActionError as e:
            with lane.lock:
                if e.kind == "cancelled":
                    lane.stats.cancelled += 1
                else:
                    lane.stats.failed += 1
            raise
        except BaseException as e:  # noqa: BLE001 - contain: the lane keeps serving
            with lane.lock:
                lane.stats.failed += 1
            trace.event("executor", 1, "action failed", model=model_id, action=action, error=repr(e))
            raise
        finally:
            with lane.lock:
                lane.stats.in_flight -= 1
                lane.stats.busy_seconds += time.time() - t1
            lane.slots.release()

    def submit(self, model_id: str, action: str, inv: Invocation, progress=None):
        return self.pool.submit(self.run, model_id, action, inv, progress)

    def close(self):
        if self.residency is not None:
            self.residency.close()
        for lane in list(self.lanes.values()):
            try:
                lane.model.close()
            except Exception:
                pass
        self.pool.shutdown(wait=False, cancel_futures=True)
