"""The language-model resident on the CPU backend: continuous batching through one long-lived
scheduler gives the same greedy text as serial generation, stop sequences and cancellation work,
capacity errors map to ``context_length_exceeded``, and the HTTP layer serves it."""
import json
import os
import sys
import threading

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from brain_b200.api.capability import ActionError, CancelToken, Invocation  # noqa: E402
from brain_b200.api.errors import from_exception  # noqa: E402
from brain_b200.api.executor import Executor  # noqa: E402
from brain_b200.api.resident import LlmResident  # noqa: E402
from brain_b200.data.tokenizer import BpeTokenizer  # noqa: E402
from brain_b200.models.config import QwenConfig  # noqa: E402
from brain_b200.models.qwen3 import Qwen3  # noqa: E402
from brain_b200.train import generate  # noqa: E402


@pytest.fixture(scope="module")
def llm():
    tok = BpeTokenizer.byte_level(["t h", "th e"], {"<|im_start|>": 258, "<|im_end|>": 259, "<|endoftext|>": 260})
    cfg = QwenConfig(vocab=264, block_size=256, n_layers=2, d_model=32, n_heads=4, n_kv_heads=2, head_dim=8, d_ff=64)
    m = Qwen3(cfg).init_weights(7).eval()
    r = LlmResident(m, tok, "brain/tiny", ctx=256, max_batch=4)
    yield r, m, tok
    r.close()


def run(r, **params):
    inv = Invocation(r.manifest().action("generate").validate(params))
    pieces = []
    out = r.run("generate", inv, lambda p: pieces.append(p.text))
    return out, pieces


def test_matches_serial_greedy_and_streams(llm):
    r, m, tok = llm
    prompt = "the quick brown fox"
    out, pieces = run(r, prompt=prompt, chat=False, max_new=12, temp=0.0, ignore_eos=True)
    ids = tok.encode(prompt)
    want = generate(m, ids, 12, temp=0.0)
    assert out.outputs["completion_tokens"] == 12 and out.outputs["finish_reason"] == "length"
    assert out.outputs["prompt_tokens"] == len(ids)
    assert out.text() == tok.decode(want, skip_special=True)
    assert "".join(pieces) == out.text()


def test_concurrent_equals_serial(llm):
    r, m, tok = llm
    prompts = [f"prompt number {i} says" for i in range(6)]
    serial = [run(r, prompt=p, chat=False, max_new=10, temp=0.0, ignore_eos=True)[0].text() for p in prompts]
    got = [None] * len(prompts)

    def work(i):
        got[i] = run(r, prompt=prompts[i], chat=False, max_new=10, temp=0.0, ignore_eos=True)[0].text()
    ts = [threading.Thread(target=work, args=(i,)) for i in range(len(prompts))]
    [t.start() for t in ts]
    [t.join() for t in ts]
    assert got == serial
    assert r.stats()["finished"] >= 12


def test_chat_template_and_sampling_seed(llm):
    r, m, tok = llm
    a, _ = run(r, messages=json.dumps([{"role": "user", "content": "hi"}]), max_new=8, temp=0.9, top_k=20, seed=3, ignore_eos=True)
    b, _ = run(r, messages=json.dumps([{"role": "user", "content": "hi"}]), max_new=8, temp=0.9, top_k=20, seed=3, ignore_eos=True)
    assert a.text() == b.text()
    want = len(tok.encode(tok.apply_chat_template([("user", "hi")], True)))
    assert a.outputs["prompt_tokens"] == want


def test_stop_sequence_truncates(llm):
    r, m, tok = llm
    full, _ = run(r, prompt="abc abc abc", chat=False, max_new=24, temp=0.0, ignore_eos=True)
    text = full.text()
    visible = [c for c in text[3:] if c.isprintable() and c != "�"]
    if not visible:
        pytest.skip("tiny random model produced no printable text to stop on")
    stop = visible[0]
    out, pieces = run(r, prompt="abc abc abc", chat=False, max_new=24, temp=0.0, ignore_eos=True, stop=json.dumps([stop]))
    assert out.outputs["finish_reason"] == "stop_sequence"
    assert out.text() == text[:text.index(stop)] and stop not in "".join(pieces)


def test_capacity_error_maps_to_context_length(llm):
    r, _, _ = llm
    with pytest.raises(ActionError) as e:
        run(r, prompt="x" * 300, chat=False, max_new=8)
    err = from_exception(e.value)
    assert err.code == "context_length_exceeded" and err.status == 400 and "256" in err.message


def test_policy_rejection_maps_to_429(monkeypatch):
    """A request the scheduler's admission policy turns away is a rate-limit error (HTTP 429 with
    Retry-After), not a client error.  Queue depth 0 rejects everything, which needs no timing."""
    monkeypatch.setenv("BRAIN_SCHED_POLICY", "max_queue_depth:0")
    tok = BpeTokenizer.byte_level(["t h"], {"<|im_start|>": 258, "<|im_end|>": 259, "<|endoftext|>": 260})
    cfg = QwenConfig(vocab=264, block_size=64, n_layers=1, d_model=32, n_heads=4, n_kv_heads=2, head_dim=8, d_ff=64)
    r = LlmResident(Qwen3(cfg).init_weights(3).eval(), tok, "brain/tiny", ctx=64, max_batch=2)
    try:
        with pytest.raises(ActionError) as e:
            run(r, prompt="hello", chat=False, max_new=4)
        err = from_exception(e.value)
        assert err.code == "rate_limit_exceeded" and err.status == 429 and err.headers() == {"Retry-After": "1"}
    finally:
        r.close()


def test_cancel_frees_blocks(llm):
    r, _, _ = llm
    free0 = r.stats()["free_blocks"]
    tok = CancelToken()
    inv = Invocation(r.manifest().action("generate").validate(dict(prompt="go on", chat=False, max_new=200, temp=0.0, ignore_eos=True)), cancel=tok)
    n = [0]

    def prog(p):
        n[0] += 1
        if n[0] == 3:
            tok.cancel()
    with pytest.raises(ActionError) as e:
        r.run("generate", inv, prog)
    assert e.value.kind == "cancelled" and n[0] < 200
    out, _ = run(r, prompt="after", chat=False, max_new=4, temp=0.0, ignore_eos=True)
    assert out.outputs["completion_tokens"] == 4
    assert r.stats()["free_blocks"] >= free0 - 2       # only prefix-cache blocks may stay resident


def test_http_serves_the_model(llm):
    from brain_b200.api.server import Server
    import urllib.request
    r, _, _ = llm
    ex = Executor({r.id: r})
    s = Server(ex, {"openai": 0}).start_background()
    try:
        body = json.dumps({"model": "brain/tiny", "messages": [{"role": "user", "content": "hello"}], "max_tokens": 6,
                           "temperature": 0}).encode()
        req = urllib.request.Request(f"http://127.0.0.1:{s.bound['openai']}/v1/chat/completions", data=body,
                                     headers={"Authorization": "Bearer " + s.keys["openai"], "Content-Type": "application/json"})
        d = json.load(urllib.request.urlopen(req, timeout=60))
        assert d["usage"]["completion_tokens"] <= 6 and d["choices"][0]["finish_reason"] in ("stop", "length")
        req = urllib.request.Request(f"http://127.0.0.1:{s.bound['openai']}/v1/models",
                                     headers={"Authorization": "Bearer " + s.keys["openai"]})
        d = json.load(urllib.request.urlopen(req, timeout=60))
        assert d["data"][0]["context_length"] == 256
    finally:
        s.shutdown()
        ex.pool.shutdown(wait=False)


def test_streaming_joins_characters_split_across_tokens():
    """Tokens are decoded once each as they arrive; a multi-byte character whose bytes come in
    different tokens is emitted when its last byte arrives, a stop sequence straddling two tokens
    still stops, and the streamed pieces concatenate to the one-shot decoding."""
    from types import SimpleNamespace
    from brain_b200.api.resident import LlmResident, _Job
    from brain_b200.data.tokenizer import BpeTokenizer, utf8_complete
    assert utf8_complete("é".encode()[:1]) == 0 and utf8_complete("aé".encode()) == 3
    assert utf8_complete("a🙂".encode()[:3]) == 1 and utf8_complete(b"abc") == 3 and utf8_complete(b"") == 0
    assert utf8_complete(b"a\x80\x80") == 3          # stray continuation bytes are not held back
    tok = BpeTokenizer.byte_level()                  # one token per byte
    me = SimpleNamespace(tok=tok)
    text = "naïve 🙂 日本 done"
    ids = tok.encode(text)
    assert len(ids) == len(text.encode())

    def stream(stops, chunk):
        job = _Job()
        job.stops = stops
        pieces = []
        job.on_token = pieces.append
        stopped = False
        for i in range(0, len(ids), chunk):
            if LlmResident._deliver(me, job, ids[i:i + chunk]):
                stopped = True
                break
        if not stopped:          # what _finish does with the tail
            tail = job.held + job.raw.decode("utf-8", errors="replace")
            if tail:
                pieces.append(tail)
        return pieces, stopped, job
    for chunk in (1, 2, 3, 5):
        pieces, stopped, job = stream([], chunk)
        assert "".join(pieces) == text and not stopped
        assert all("�" not in p for p in pieces)
        assert job.n_tokens == len(ids)
    pieces, stopped, _ = stream(["本 d"], 1)
    assert stopped and "".join(pieces) == "naïve 🙂 日"
    pieces, stopped, _ = stream(["zzz", "🙂 日x"], 2)      # a prefix of a stop is held, then released
    assert not stopped and "".join(pieces) == text


def test_reasoning_stream_routes_think_blocks():
    from brain_b200.data.chat import ReasoningStream, split_reasoning
    text = "<think>\nlet me see < 3 </thin no</think>\n\nThe answer is <b>4</b>."
    for size in (1, 2, 3, 7, 100):
        rs = ReasoningStream()
        got = []
        for i in range(0, len(text), size):
            got += rs.feed(text[i:i + size])
        got += rs.flush()
        reasoning = "".join(t for k, t in got if k == "reasoning")
        visible = "".join(t for k, t in got if k == "token")
        assert "<think>" not in reasoning + visible and "</think>" not in reasoning + visible
        want_r, want_v = split_reasoning(text)
        assert reasoning.strip() == want_r and visible.strip() == want_v
    rs = ReasoningStream()
    assert rs.feed("plain <") == [("token", "plain ")] and rs.flush() == [("token", "<")]
