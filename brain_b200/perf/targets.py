"""Perf targets (reference: crates/perf/src/target.rs — the ``submit``/``step`` → emissions
contract and the in-crate ``FakeTarget``; crates/perf/src/targets.rs — ``qwen-synth:LxDxH[xV]``
random-init synthetic Qwen (no weights needed) and ``http:`` variants through the real HTTP
stack)."""
from __future__ import annotations

import json
import threading
import time
import urllib.request
from dataclasses import dataclass
from typing import Dict, List, Optional

import numpy as np

from .workload import PerfRequest


@dataclass
class Emission:
    id: int
    kind: str              # admitted | artifact | done | failed | rejected
    at: float
    count: int = 1
    error: Optional[str] = None


class PerfTarget:
    info: Dict = {}

    def submit(self, req: PerfRequest) -> int:
        raise NotImplementedError

    def step(self, out: List[Emission]) -> bool:
        """Advance; append emissions; return True while work remains."""
        raise NotImplementedError

    def outputs(self, rid: int) -> List[int]:
        return []

    def close(self):
        pass


class FakeTarget(PerfTarget):
    """Deterministic target for harness tests: ``prefill_steps`` steps to first token, then one
    token per step, at most ``max_concurrent`` running."""

    def __init__(self, max_concurrent: int = 4, prefill_steps: int = 2, step_s: float = 0.0):
        self.max_c, self.pre, self.step_s = max_concurrent, prefill_steps, step_s
        self.wait: List[int] = []
        self.run: Dict[int, List[int]] = {}       # id -> [steps_left_prefill, tokens_left]
        self.reqs: Dict[int, PerfRequest] = {}
        self.out: Dict[int, List[int]] = {}
        self.next = 0
        self.info = {"model": "fake", "artifact_unit": "token"}

    def submit(self, req):
        rid = self.next
        self.next += 1
        self.reqs[rid] = req
        self.wait.append(rid)
        self.out[rid] = []
        return rid

    def step(self, out):
        if self.step_s:
            time.sleep(self.step_s)
        now = time.perf_counter()
        while self.wait and len(self.run) < self.max_c:
            rid = self.wait.pop(0)
            self.run[rid] = [self.pre, self.reqs[rid].max_new]
            out.append(Emission(rid, "admitted", now))
        for rid in list(self.run):
            st = self.run[rid]
            if st[0] > 1:
                st[0] -= 1
                continue
            st[0] = 0
            st[1] -= 1
            self.out[rid].append((int(self.reqs[rid].prompt.sum()) + len(self.out[rid])) % 1000)
            out.append(Emission(rid, "artifact", now))
            if st[1] == 0:
                out.append(Emission(rid, "done", now))
                del self.run[rid]
        return bool(self.wait or self.run)

    def outputs(self, rid):
        return self.out[rid]

    def cancel(self, rid):
        self.run.pop(rid, None)
        if rid in self.wait:
            self.wait.remove(rid)


class SchedulerTarget(PerfTarget):
    """A model behind the paged-KV engine and continuous-batching scheduler, driven in-process."""

    def __init__(self, model, max_batch: int = 256, ctx: int = 4096, block_size: int = 16, weights: str = "bf16",
                 num_blocks: Optional[int] = None, tp=None, name: str = "qwen", engine=None, admit_batch: int = 1,
                 prefix_cache: bool = True, prefill_budget: int = 0, policy: str = "unbounded_queue",
                 policy_arg: float = 0.0, admit_max_wait: int = 64, window: int = 4, mixed: bool = False):
        from ..serve.engine import QwenEngine
        from ..serve.scheduler import Scheduler
        per_seq = -(-ctx // block_size)
        nb = num_blocks or per_seq * max_batch + max_batch
        self.engine = engine or QwenEngine(model, block_size=block_size, num_blocks=nb, max_seq_len=ctx,
                                           max_prefill=min(ctx, 2048), weights=weights, tp=tp)
        self.sched = Scheduler(self.engine, max_batch=max_batch, eos=None, admit_batch=admit_batch,
                               prefix_cache=prefix_cache, prefill_budget=prefill_budget, policy=policy,
                               policy_arg=policy_arg, admit_max_wait=admit_max_wait, window=window, mixed=mixed)
        self.live: Dict[int, bool] = {}
        self.admitted: Dict[int, bool] = {}
        self.info = {"model": name, "artifact_unit": "token", "max_batch": max_batch, "ctx": ctx,
                     "weights": weights, "kv_pool_gb": self.engine.kv_pool_bytes() / 2**30}

    def submit(self, req):
        from ..serve.sampling import SampleParams
        rid = self.sched.submit(req.prompt, req.max_new, SampleParams.greedy(), req.seed, req.ignore_stop)
        self.live[rid] = True
        return rid

    def step(self, out):
        if self.sched.is_idle():
            return False
        rep = self.sched.step()
        if self.engine.cuda:
            import torch
            torch.cuda.current_stream().synchronize()
        now = time.perf_counter()
        for rid, toks in rep.new_tokens.items():
            if rid not in self.admitted:
                self.admitted[rid] = True
                out.append(Emission(rid, "admitted", now))
            out.append(Emission(rid, "artifact", now, len(toks)))
        for rid in rep.finished:
            out.append(Emission(rid, "done", now))
        return not self.sched.is_idle()

    def outputs(self, rid):
        return self.sched.tokens_of(rid)

    def cancel(self, rid):
        self.sched.cancel(rid)
        self.live.pop(rid, None)

    def free_blocks(self) -> int:
        """Blocks available to new work: free ones plus those only the prefix cache still holds."""
        st = self.sched.stats()
        return int(st["free_blocks"]) + int(st.get("prefix_entries", 0))

    def prefill_tokens(self) -> int:
        return int(self.engine.acct["prefill_tokens"])


def synth_qwen(spec: str, device=None, dtype=None):
    """``LxDxH[xV]`` -> random-init Qwen (layers, d_model, heads[, vocab]); kv heads = max(H/4, 1),
    head_dim = D/H (>= 64 on CUDA so the flash kernels apply), d_ff = 3D."""
    import torch
    from ..models.config import QwenConfig
    from ..models.qwen3 import Qwen3
    parts = [int(x) for x in spec.lower().split("x")]
    L, D, H = parts[:3]
    V = parts[3] if len(parts) > 3 else 32000
    hd = D // H
    cfg = QwenConfig(vocab=V, block_size=32768, n_layers=L, d_model=D, n_heads=H, n_kv_heads=max(H // 4, 1),
                     head_dim=hd, d_ff=3 * D, max_position_embeddings=32768)
    m = Qwen3(cfg).init_weights(11).eval()
    if device is not None:
        m = m.to(device=device, dtype=dtype or (torch.bfloat16 if str(device).startswith("cuda") else torch.float32))
    return m


class HttpTarget(PerfTarget):
    """Closed-box target: every request is a streamed ``/v1/chat/completions`` call on its own
    thread; emissions are timestamped as SSE chunks arrive."""

    def __init__(self, base_url: str, api_key: str, model: str, tokenizer=None):
        self.base, self.key, self.model, self.tok = base_url.rstrip("/"), api_key, model, tokenizer
        self.lock = threading.Lock()
        self.pending: List[Emission] = []
        self.active = 0
        self.next = 0
        self.texts: Dict[int, List[str]] = {}
        self.info = {"model": model, "artifact_unit": "chunk", "transport": "http"}

    def _prompt(self, req: PerfRequest) -> str:
        if self.tok is not None:
            return self.tok.decode(req.prompt.tolist())
        return " ".join(f"w{int(t) % 997}" for t in req.prompt[: max(req.prompt.size // 2, 1)])

    def _worker(self, rid: int, req: PerfRequest):
        body = json.dumps({"model": self.model, "stream": True, "max_tokens": req.max_new, "temperature": 0,
                           "messages": [{"role": "user", "content": self._prompt(req)}]}).encode()
        hreq = urllib.request.Request(self.base + "/v1/chat/completions", data=body, headers={
            "Authorization": f"Bearer {self.key}", "Content-Type": "application/json"})
        try:
            with urllib.request.urlopen(hreq, timeout=600) as r:
                first = True
                for raw in r:
                    line = raw.decode().strip()
                    if not line.startswith("data:") or line.endswith("[DONE]"):
                        continue
                    obj = json.loads(line[5:])
                    for ch in obj.get("choices", []):
                        piece = ch.get("delta", {}).get("content")
                        if piece:
                            now = time.perf_counter()
                            with self.lock:
                                if first:
                                    self.pending.append(Emission(rid, "admitted", now))
                                    first = False
                                self.pending.append(Emission(rid, "artifact", now))
                                self.texts[rid].append(piece)
            with self.lock:
                self.pending.append(Emission(rid, "done", time.perf_counter()))
        except Exception as e:  # noqa: BLE001
            kind = "rejected" if "429" in str(e) or "503" in str(e) else "failed"
            with self.lock:
                self.pending.append(Emission(rid, kind, time.perf_counter(), error=str(e)))
        finally:
            with self.lock:
                self.active -= 1

    def submit(self, req):
        rid = self.next
        self.next += 1
        self.texts[rid] = []
        with self.lock:
            self.active += 1
        threading.Thread(target=self._worker, args=(rid, req), daemon=True).start()
        return rid

    def step(self, out):
        time.sleep(0.002)
        with self.lock:
            out.extend(self.pending)
            self.pending.clear()
            return self.active > 0 or bool(self.pending)

    def outputs(self, rid):
        return ["".join(self.texts[rid])]
