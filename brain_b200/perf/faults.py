"""Fault scenarios with host-side injection (reference: crates/perf/src/scenarios/faults.rs:20-104 —
the ``Fault`` kinds and the acceptance rule: the failure is REPORTED, no surviving answer is
CORRUPTED, and UNRELATED work survives).  Nothing here faults, traps or hangs a device: a failed
launch is an exception raised before the launch, a dead worker is a thread that raises, memory
exhaustion is an exhausted block pool, a hung rank is a rank that never joins a host collective."""
from __future__ import annotations

import os
import tempfile
import threading
from dataclasses import dataclass
from typing import Callable, Dict, List

import torch


@dataclass
class FaultResult:
    fault: str
    reported: bool
    clean: bool        # surviving answers equal the fault-free answers
    survived: bool     # unrelated / later work completed
    detail: str = ""

    @property
    def passed(self) -> bool:
        return self.reported and self.clean and self.survived

    def to_json(self) -> Dict:
        return {"fault": self.fault, "reported": self.reported, "clean": self.clean, "survived": self.survived,
                "passed": self.passed, "detail": self.detail}


def _tiny_llm():
    from ..api.resident import LlmResident
    from ..data.tokenizer import BpeTokenizer
    from ..models.config import QwenConfig
    from ..models.qwen3 import Qwen3
    tok = BpeTokenizer.byte_level([], {"<|im_start|>": 256, "<|im_end|>": 257, "<|endoftext|>": 258})
    cfg = QwenConfig(vocab=264, block_size=128, n_layers=1, d_model=32, n_heads=4, n_kv_heads=2, head_dim=8, d_ff=64)
    return LlmResident(Qwen3(cfg).init_weights(7).eval(), tok, "brain/tiny", ctx=128, max_batch=4)


def _gen(llm, prompt: str, n: int = 8) -> str:
    from ..api.capability import Invocation
    inv = Invocation(llm.manifest().action("generate").validate(
        dict(prompt=prompt, chat=False, max_new=n, temp=0.0, ignore_eos=True)))
    return llm.run("generate", inv, lambda p: None).text()


def kernel_failure() -> FaultResult:
    """One decode call fails on the host side of the launch: the requests of that step get an
    error, the serving loop survives, and a later request returns exactly the fault-free text."""
    llm = _tiny_llm()
    try:
        want = _gen(llm, "after the fault")
        armed = {"n": 2}

        def hook(op):
            if op == "decode":
                armed["n"] -= 1
                if armed["n"] == 0:
                    raise RuntimeError("injected launch failure")
        llm.engine.fault_hook = hook
        reported = False
        try:
            _gen(llm, "this request dies", 16)
        except Exception:  # noqa: BLE001
            reported = True
        llm.engine.fault_hook = None
        got = _gen(llm, "after the fault")
        st = llm.stats()
        return FaultResult("kernel_failure", reported, got == want, st["running"] == 0 and st["waiting"] == 0,
                           f"free_blocks={st['free_blocks']}")
    finally:
        llm.close()


def device_oom() -> FaultResult:
    """The KV block pool cannot hold a request: it is refused with a capacity error; requests that
    fit are served before and after."""
    from ..api.capability import ActionError
    llm = _tiny_llm()
    try:
        want = _gen(llm, "small")
        reported = False
        try:
            _gen(llm, "x" * 400, 8)
        except ActionError as e:
            reported = e.kind == "context_length_exceeded"
        got = _gen(llm, "small")
        return FaultResult("device_oom", reported, got == want, True)
    finally:
        llm.close()


def weight_read_failure() -> FaultResult:
    """A truncated checkpoint is refused with an I/O error instead of serving garbage; an intact
    file next to it still loads."""
    from ..checkpoint import st
    from ..models.config import GptConfig
    from ..models.gpt2 import Gpt2
    with tempfile.TemporaryDirectory() as d:
        good = os.path.join(d, "good.safetensors")
        bad = os.path.join(d, "bad.safetensors")
        m = Gpt2(GptConfig(vocab=20, block_size=8, n_layers=1, d_model=16, n_heads=2, d_ff=32)).init_weights(1)
        st.save_model(good, m)
        raw = open(good, "rb").read()
        open(bad, "wb").write(raw[: len(raw) // 2])
        reported = False
        try:
            st.load_model(bad)
        except Exception:  # noqa: BLE001 - any refusal counts; silence would not
            reported = True
        m2, _, _ = st.load_model(good)
        x = torch.randint(0, 20, (1, 8), dtype=torch.int32)
        clean = torch.equal(m(x), m2(x))
        return FaultResult("weight_read_failure", reported, clean, True)


def worker_death() -> FaultResult:
    """A data-parallel replica thread dies inside forward/backward: the step raises (the other
    replica is released from the collective, it does not wait forever) and a fresh group trains."""
    from ..models.config import GptConfig
    from ..models.gpt2 import Gpt2
    from ..parallel.dp import DataParallel
    cfg = GptConfig(vocab=20, block_size=8, n_layers=1, d_model=16, n_heads=2, d_ff=32)
    mk = lambda: Gpt2(cfg).init_weights(1)
    x = torch.randint(0, 20, (2, 8), dtype=torch.int32)
    y = torch.randint(0, 20, (2, 8))
    dp = DataParallel(mk, 2)
    orig = dp.models[1].loss

    def dying(*a, **k):
        raise RuntimeError("injected worker death")
    dp.models[1].loss = dying
    reported = False
    done = threading.Event()

    def run():
        nonlocal reported
        try:
            dp.train_step([(x, y), (x, y)], 1e-3)
        except Exception:  # noqa: BLE001
            reported = True
        done.set()
    t = threading.Thread(target=run, daemon=True)
    t.start()
    finished = done.wait(30)
    dp.models[1].loss = orig
    dp2 = DataParallel(mk, 2)
    l0 = dp2.train_step([(x, y), (x, y)], 1e-2)
    l1 = dp2.train_step([(x, y), (x, y)], 1e-2)
    return FaultResult("worker_death", reported and finished, True, l1 < l0, "step raised within 30 s" if finished else "step hung")


def hung_rank() -> FaultResult:
    """A rank never joins a host collective: the waiting rank gets a timeout error within the
    bound instead of blocking forever, and a complete group works afterwards."""
    from ..parallel.collective import HostCollective
    group = HostCollective.group(2, timeout_s=0.5)
    reported = False
    t = torch.ones(4)
    done = threading.Event()

    def lone():
        nonlocal reported
        try:
            group[0].all_reduce(t)
        except Exception:  # noqa: BLE001
            reported = True
        done.set()
    th = threading.Thread(target=lone, daemon=True)
    th.start()
    finished = done.wait(40)
    g2 = HostCollective.group(2)
    outs = [torch.ones(4), torch.ones(4) * 2]
    ths = [threading.Thread(target=lambda r=r: g2[r].all_reduce(outs[r])) for r in range(2)]
    [x.start() for x in ths]
    [x.join(10) for x in ths]
    ok = torch.equal(outs[0], torch.full((4,), 3.0)) and torch.equal(outs[1], outs[0])
    return FaultResult("hung_rank", reported and finished, True, ok)


SCENARIOS: Dict[str, Callable[[], FaultResult]] = {
    "kernel_failure": kernel_failure, "device_oom": device_oom, "weight_read_failure": weight_read_failure,
    "worker_death": worker_death, "hung_rank": hung_rank,
}


def run_all(names: List[str] = None) -> List[FaultResult]:
    return [SCENARIOS[n]() for n in (names or list(SCENARIOS))]
