"""Residency manager: lazy loading through suppliers, per-device budgets, least-recently-used
eviction of idle models only, one load for concurrent first requests, and the executor / HTTP view
of models that are not loaded yet."""
import json
import threading
import time
import urllib.request

import pytest

from brain_b200.api.capability import Invocation
from brain_b200.api.executor import Busy, Executor
from brain_b200.api.residency import InsufficientMemory, Residency, Supplier, _Stub
from brain_b200.api.resident import MockResident


class FakeSupplier(Supplier):
    def __init__(self, mid, nbytes, load_s=0.0):
        self.id, self.nbytes, self.load_s = mid, nbytes, load_s
        self.loads = 0
        self.closed = 0

    def estimate_bytes(self):
        return self.nbytes

    def stub(self):
        return _Stub(self.id, "fake", 1024)

    def load(self, device):
        time.sleep(self.load_s)
        self.loads += 1
        sup = self

        class M(MockResident):
            id = sup.id

            def close(self):
                sup.closed += 1
        return M()


def test_budget_lru_and_pinning():
    a, b, c, big = (FakeSupplier(n, s) for n, s in (("t/a", 40), ("t/b", 40), ("t/c", 40), ("t/big", 500)))
    r = Residency({s.id: s for s in (a, b, c, big)}, {"dev0": 100})
    assert r.known() == ["t/a", "t/b", "t/big", "t/c"] and r.resident() == []
    assert r.describe("t/a").manifest().model == "t/a" and r.describe("nope") is None
    ma = r.acquire("t/a")
    r.acquire("t/b")
    r.release("t/b")
    assert r.used("dev0") == 80
    r.acquire("t/c")                    # does not fit: b is idle and goes, a is in use and stays
    assert r.resident() == ["t/a", "t/c"] and b.closed == 1 and a.closed == 0 and r.evictions == 1
    with pytest.raises(InsufficientMemory):
        r.acquire("t/b")                # a and c are both in use: nothing can be evicted
    r.release("t/a")
    r.release("t/c")
    time.sleep(0.01)
    r.acquire("t/a")                    # touch a: c is now the least recently used
    r.release("t/a")
    r.acquire("t/b")
    assert r.resident() == ["t/a", "t/b"] and c.closed == 1
    with pytest.raises(InsufficientMemory):
        r.acquire("t/big")              # larger than the device's whole budget
    with pytest.raises(KeyError):
        r.acquire("t/unknown")
    assert ma.manifest().model == "t/a" and r.stats()["loads"] == 4


def test_placement_prefers_the_emptier_device_and_concurrent_first_requests_load_once():
    a, b, slow = FakeSupplier("t/a", 60), FakeSupplier("t/b", 60), FakeSupplier("t/slow", 10, load_s=0.2)
    r = Residency({s.id: s for s in (a, b, slow)}, {"dev0": 100, "dev1": 100})
    r.acquire("t/a")
    r.acquire("t/b")
    devs = {r.stats()["resident"][k]["device"] for k in ("t/a", "t/b")}
    assert devs == {"dev0", "dev1"}
    got = []
    ths = [threading.Thread(target=lambda: got.append(r.acquire("t/slow"))) for _ in range(5)]
    [t.start() for t in ths]
    [t.join(10) for t in ths]
    assert len(got) == 5 and slow.loads == 1 and all(g is got[0] for g in got)
    assert r.stats()["resident"]["t/slow"]["in_use"] == 5


def test_executor_and_http_serve_models_that_load_on_first_use():
    from brain_b200.api.server import Server
    lazy, big = FakeSupplier("acme/lazy", 10), FakeSupplier("acme/big", 10_000)
    res = Residency({lazy.id: lazy, big.id: big}, {"dev0": 100})
    ex = Executor({MockResident.id: MockResident()}, residency=res)
    assert set(ex.models()) == {"brain/mock", "acme/lazy", "acme/big"} and lazy.loads == 0
    spec = ex.get("acme/lazy").manifest().action("generate")
    out = ex.run("acme/lazy", "generate", Invocation(spec.validate({"prompt": "hi there"})))
    assert out.text() == "You said: hi there" and lazy.loads == 1
    assert res.stats()["resident"]["acme/lazy"]["in_use"] == 0        # released after the request
    with pytest.raises(Busy):
        ex.run("acme/big", "generate", Invocation({"prompt": "x"}))
    with pytest.raises(KeyError):
        ex.run("acme/none", "generate", Invocation({"prompt": "x"}))
    s = Server(ex, {"openai": 0}).start_background()
    try:
        base, key = f"http://127.0.0.1:{s.bound['openai']}", s.keys["openai"]
        hdr = {"Authorization": f"Bearer {key}", "Content-Type": "application/json"}
        with urllib.request.urlopen(urllib.request.Request(base + "/v1/models", headers=hdr), timeout=10) as r:
            ids = {m["id"] for m in json.loads(r.read())["data"]}
        assert {"brain/mock", "acme/lazy", "acme/big"} <= ids
        body = json.dumps({"model": "acme/lazy", "messages": [{"role": "user", "content": "again"}]}).encode()
        with urllib.request.urlopen(urllib.request.Request(base + "/v1/chat/completions", data=body, headers=hdr),
                                    timeout=30) as r:
            assert json.loads(r.read())["choices"][0]["message"]["content"] == "You said: again"
        body = json.dumps({"model": "acme/big", "messages": [{"role": "user", "content": "x"}]}).encode()
        with pytest.raises(urllib.error.HTTPError) as e:
            urllib.request.urlopen(urllib.request.Request(base + "/v1/chat/completions", data=body, headers=hdr), timeout=30)
        assert e.value.code == 429
    finally:
        s.shutdown()
        ex.close()
    assert lazy.closed == 1


def test_serve_stdio_loads_store_models_on_first_use(tmp_path):
    """``brain serve --stdio --models-dir D``: every model of the store is listed, none is loaded
    until a request names it, and the request is answered by the real engine."""
    import os
    from brain_b200.checkpoint import st
    from brain_b200.data.tokenizer import bytes_to_unicode
    from brain_b200.modelref import ModelRef
    from brain_b200.modelstore import Store
    from brain_b200.models.config import QwenConfig
    from brain_b200.models.qwen3 import Qwen3
    from brain_py import Brain
    cfg = QwenConfig(vocab=264, block_size=64, n_layers=1, d_model=32, n_heads=4, n_kv_heads=2, head_dim=8, d_ff=64)
    w = str(tmp_path / "w.safetensors")
    st.save_model(w, Qwen3(cfg).init_weights(3))
    b2u = bytes_to_unicode()
    tok = tmp_path / "tokenizer.json"
    tok.write_text(json.dumps({"model": {"vocab": {b2u[b]: b for b in range(256)}, "merges": []},
                               "added_tokens": [{"content": "<|im_start|>", "id": 256}, {"content": "<|im_end|>", "id": 257}]}))
    root = str(tmp_path / "models")
    Store(root).install(ModelRef.parse("acme/tiny-a"), w, str(tok))
    Store(root).install(ModelRef.parse("acme/tiny-b"), w, str(tok))
    with Brain(transport="jsonl", args=["--models-dir", root], device="cpu", env={"BRAIN_QWEN_CTX": "64"}) as b:
        assert sorted(b.models()) == ["acme/tiny-a", "acme/tiny-b"]
        out = b.generate(prompt="hi", model="acme/tiny-b", max_new=4, temp=0.0, chat=False)
        assert out.get("completion_tokens") == 4 and out.get("prompt_tokens") == 2
