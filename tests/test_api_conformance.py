"""HTTP conformance against the deterministic mock model: auth on every path, error schema and
status codes, request validation, non-stream and SSE shapes for the OpenAI, OpenRouter and Anthropic
dialects, the JSONL stdio protocol, and the brain_py transports.  Model of the reference's suite:
crates/apiserve/tests/*.rs (conformance vs ``BRAIN_MOCK``) and brain-py/tests/test_client.py."""
import json
import os
import stat
import sys
import threading
import urllib.error
import urllib.request

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from brain_b200.api import auth  # noqa: E402
from brain_b200.api.executor import Executor  # noqa: E402
from brain_b200.api.resident import FAIL_TRIGGER, TOOL_CALL_TRIGGER, MockResident  # noqa: E402
from brain_b200.api.server import Server  # noqa: E402
from brain_py import Brain, BrainAnthropic, BrainError, BrainOpenAI  # noqa: E402


@pytest.fixture(scope="module")
def srv():
    ex = Executor({MockResident.id: MockResident()})
    s = Server(ex, {"openai": 0, "anthropic": 0, "openrouter": 0}).start_background()
    yield s
    s.shutdown()
    ex.close()


def call(srv, provider, path, body=None, key="ok", method=None, headers=None, raw=None):
    url = f"http://127.0.0.1:{srv.bound[provider]}{path}"
    h = {"Content-Type": "application/json"}
    if key == "ok":
        key = srv.keys[provider]
    if key:
        if provider == "anthropic":
            h["x-api-key"] = key
        else:
            h["Authorization"] = f"Bearer {key}"
    h.update(headers or {})
    data = raw if raw is not None else (json.dumps(body).encode() if body is not None else None)
    req = urllib.request.Request(url, data=data, headers=h, method=method or ("POST" if data is not None else "GET"))
    try:
        with urllib.request.urlopen(req, timeout=30) as r:
            return r.status, dict(r.headers), r.read()
    except urllib.error.HTTPError as e:
        return e.code, dict(e.headers), e.read()


def chat(srv, content="hello world", provider="openai", **kw):
    body = {"model": "brain/mock", "messages": [{"role": "user", "content": content}]}
    body.update(kw)
    return call(srv, provider, "/v1/chat/completions", body)


def sse(raw: bytes):
    out, event = [], None
    for line in raw.decode().split("\n"):
        if line.startswith("event:"):
            event = line[6:].strip()
        elif line.startswith("data:"):
            out.append((event, line[5:].strip()))
            event = None
    return out


# ------------------------------------------------------------------------------------ auth
def test_key_format_and_file(tmp_path):
    k = auth.new_key()
    assert k.startswith("sk-brain-") and len(k) == 9 + 32 and int(k[9:], 16) >= 0
    p = tmp_path / "keys.json"
    auth.write_keys(str(p), {"openai": k})
    assert json.loads(p.read_text()) == {"openai": k}
    assert stat.S_IMODE(os.stat(p).st_mode) == 0o600


@pytest.mark.parametrize("provider", ["openai", "openrouter", "anthropic"])
def test_401_on_every_path_including_unknown(srv, provider):
    for path in ("/v1/models", "/v1/chat/completions", "/nope", "/v1/messages"):
        for key in (None, "sk-brain-" + "0" * 32):
            st, _, body = call(srv, provider, path, key=key)
            assert st == 401, (path, key)
            err = json.loads(body)
            if provider == "anthropic":
                assert err["type"] == "error" and err["error"]["type"] == "authentication_error"
            else:
                assert err["error"]["code"] == "invalid_api_key" and err["error"]["param"] is None


def test_unknown_route_with_key_is_404(srv):
    st, _, body = call(srv, "openai", "/v1/nope")
    assert st == 404 and json.loads(body)["error"]["type"] == "invalid_request_error"


# ------------------------------------------------------------------------------------ models
def test_models_listing_with_and_without_v1(srv):
    for path in ("/v1/models", "/models"):
        st, _, body = call(srv, "openai", path)
        d = json.loads(body)
        assert st == 200 and d["object"] == "list"
        m = d["data"][0]
        assert m["id"] == "brain/mock" and m["object"] == "model" and m["owned_by"] == "brain" and m["created"] == 1767225600
    st, _, body = call(srv, "openai", "/v1/models/brain/mock")
    assert st == 200 and json.loads(body)["id"] == "brain/mock"
    st, _, body = call(srv, "openai", "/v1/models/brain/none")
    assert st == 404 and json.loads(body)["error"]["code"] == "model_not_found"


# ------------------------------------------------------------------------------------ chat (non-stream)
def test_chat_completion_shape(srv):
    st, _, body = chat(srv, "hello world")
    d = json.loads(body)
    assert st == 200 and d["object"] == "chat.completion" and d["id"].startswith("chatcmpl-") and d["created"] == 1767225600
    ch = d["choices"][0]
    assert ch["index"] == 0 and ch["logprobs"] is None and ch["finish_reason"] == "stop"
    assert ch["message"] == {"role": "assistant", "content": "You said: hello world", "refusal": None}
    u = d["usage"]
    assert u == {"prompt_tokens": 2, "completion_tokens": 4, "total_tokens": 6}


def test_chat_without_v1_prefix_and_openrouter(srv):
    st, _, body = call(srv, "openai", "/chat/completions", {"model": "brain/mock", "messages": [{"role": "user", "content": "a"}]})
    assert st == 200
    st, _, body = chat(srv, "via router", provider="openrouter")
    assert st == 200 and json.loads(body)["choices"][0]["message"]["content"] == "You said: via router"


def test_max_tokens_and_length_finish(srv):
    st, _, body = chat(srv, "one two three four five", max_tokens=3)
    d = json.loads(body)
    assert d["choices"][0]["finish_reason"] == "length" and d["usage"]["completion_tokens"] == 3
    st, _, body = chat(srv, "one two three four five", max_completion_tokens=2, max_tokens=50)
    assert json.loads(body)["usage"]["completion_tokens"] == 2


def test_stop_string_and_array(srv):
    for stop in ("three", ["zzz", "three"]):
        st, _, body = chat(srv, "one two three four", stop=stop)
        d = json.loads(body)
        assert d["choices"][0]["message"]["content"] == "You said: one two" and d["choices"][0]["finish_reason"] == "stop"


def test_content_parts_and_roles(srv):
    body = {"model": "brain/mock", "messages": [
        {"role": "developer", "content": "be brief"},
        {"role": "user", "content": [{"type": "text", "text": "part one"}, {"type": "text", "text": " part two"}]}]}
    st, _, raw = call(srv, "openai", "/v1/chat/completions", body)
    assert st == 200 and json.loads(raw)["choices"][0]["message"]["content"] == "You said: part one part two"


@pytest.mark.parametrize("body,frag", [
    ({"messages": [{"role": "user", "content": "x"}]}, "model"),
    ({"model": "brain/mock"}, "messages"),
    ({"model": "brain/mock", "messages": []}, "messages"),
    ({"model": "brain/mock", "messages": [{"role": "user", "content": "x"}], "n": 2}, "n=1"),
    ({"model": "brain/mock", "messages": [{"role": "user", "content": "x"}], "max_tokens": 0}, "max_tokens"),
    ({"model": "brain/mock", "messages": [{"role": "user", "content": "x"}], "temperature": "hot"}, "temperature"),
    ({"model": "brain/mock", "messages": [{"role": "user", "content": "x"}], "stop": 5}, "stop"),
    ({"model": "brain/mock", "messages": [{"role": "user", "content": "x"}], "tool_choice": "maybe"}, "tool_choice"),
    ({"model": "brain/mock", "messages": [{"role": "user", "content": "x"}],
      "tools": [{"type": "function", "function": {"name": "n" * 65}}]}, "64"),
    ({"model": "brain/mock", "messages": [{"role": "user", "content": "x"}],
      "tools": [{"type": "function", "function": {"name": f"t{i}"}} for i in range(129)]}, "128"),
])
def test_invalid_requests_are_400(srv, body, frag):
    st, _, raw = call(srv, "openai", "/v1/chat/completions", body)
    err = json.loads(raw)["error"]
    assert st == 400 and err["code"] == "invalid_request" and err["type"] == "invalid_request_error" and frag in err["message"]


def test_bad_json_unknown_model_and_body_cap(srv):
    st, _, raw = call(srv, "openai", "/v1/chat/completions", raw=b"{not json")
    assert st == 400 and json.loads(raw)["error"]["code"] == "invalid_request"
    st, _, raw = call(srv, "openai", "/v1/chat/completions", {"model": "gpt-17", "messages": [{"role": "user", "content": "x"}]})
    assert st == 404 and json.loads(raw)["error"]["code"] == "model_not_found"
    big = json.dumps({"model": "brain/mock", "messages": [{"role": "user", "content": "x" * (9 << 20)}]}).encode()
    st, _, raw = call(srv, "openai", "/v1/chat/completions", raw=big)
    assert st == 413


def test_internal_errors_do_not_leak(srv):
    st, _, raw = chat(srv, f"please {FAIL_TRIGGER}")
    assert st == 500
    text = raw.decode()
    assert "secret" not in text and "boom" not in text and json.loads(raw)["error"]["type"] == "server_error"


def test_tool_calls_non_stream(srv):
    tools = [{"type": "function", "function": {"name": "get_weather", "parameters": {"type": "object"}}}]
    st, _, raw = chat(srv, f"{TOOL_CALL_TRIGGER} {TOOL_CALL_TRIGGER}", tools=tools, tool_choice="auto")
    d = json.loads(raw)
    ch = d["choices"][0]
    assert st == 200 and ch["finish_reason"] == "tool_calls" and ch["message"]["content"] is None
    assert ch["message"]["reasoning_content"] == "checking which tool to call"
    calls = ch["message"]["tool_calls"]
    assert [c["function"]["name"] for c in calls] == ["get_weather", "set_timer"]
    assert calls[0]["type"] == "function" and json.loads(calls[0]["function"]["arguments"]) == {"location": "Paris"}


def test_embeddings_and_images(srv):
    st, _, raw = call(srv, "openai", "/v1/embeddings", {"model": "brain/mock", "input": ["a b", "c"]})
    d = json.loads(raw)
    assert st == 200 and d["object"] == "list" and len(d["data"]) == 2 and len(d["data"][0]["embedding"]) == 8
    assert d["data"][1]["index"] == 1 and d["usage"]["prompt_tokens"] == 3
    st, _, raw = call(srv, "openai", "/v1/images/generations", {"model": "brain/mock", "prompt": "a cat"})
    assert st == 501 and json.loads(raw)["error"]["code"] == "not_implemented"


# ------------------------------------------------------------------------------------ SSE
def test_sse_sequence_and_usage_chunk(srv):
    st, hdr, raw = chat(srv, "alpha beta", stream=True, stream_options={"include_usage": True})
    assert st == 200 and hdr["Content-Type"].startswith("text/event-stream")
    ev = sse(raw)
    assert ev[-1][1] == "[DONE]"
    chunks = [json.loads(d) for _, d in ev[:-1]]
    assert all(c["object"] == "chat.completion.chunk" for c in chunks)
    assert chunks[0]["choices"][0]["delta"] == {"role": "assistant", "content": ""}
    pieces = [c["choices"][0]["delta"]["content"] for c in chunks[1:-2]]
    assert "".join(pieces) == "You said: alpha beta"
    term = chunks[-2]["choices"][0]
    assert term["delta"] == {} and term["finish_reason"] == "stop"
    assert chunks[-1]["choices"] == [] and chunks[-1]["usage"]["completion_tokens"] == 4
    st, _, raw = chat(srv, "alpha", stream=True)
    assert all("usage" not in json.loads(d) for _, d in sse(raw)[:-1])


def test_sse_midstream_failure(srv):
    st, _, raw = chat(srv, FAIL_TRIGGER, stream=True)
    ev = sse(raw)
    assert st == 200 and ev[-1][1] == "[DONE]" and ev[-2][0] == "error"
    assert json.loads(ev[-2][1])["error"]["type"] == "server_error" and "secret" not in raw.decode()
    assert not any(e is None and "assistant" in d for e, d in ev[:-2])     # no assistant chunk announced


def test_sse_tool_call_deltas(srv):
    st, _, raw = chat(srv, TOOL_CALL_TRIGGER, stream=True, tools=[{"type": "function", "function": {"name": "get_weather"}}])
    chunks = [json.loads(d) for _, d in sse(raw)[:-1]]
    deltas = [c["choices"][0]["delta"] for c in chunks if c["choices"]]
    assert any("reasoning_content" in d for d in deltas)
    starts = [d["tool_calls"][0] for d in deltas if "tool_calls" in d and "id" in d["tool_calls"][0]]
    assert starts[0]["function"]["name"] == "get_weather" and starts[0]["function"]["arguments"] == ""
    args = "".join(d["tool_calls"][0]["function"]["arguments"] for d in deltas if "tool_calls" in d)
    assert json.loads(args) == {"location": "Paris"}
    assert chunks[-1]["choices"][0]["finish_reason"] == "tool_calls"


# ------------------------------------------------------------------------------------ anthropic
def test_anthropic_messages(srv):
    body = {"model": "brain/mock", "max_tokens": 64, "system": [{"type": "text", "text": "sys"}],
            "messages": [{"role": "user", "content": [{"type": "text", "text": "hi there"}]}]}
    st, _, raw = call(srv, "anthropic", "/v1/messages", body)
    d = json.loads(raw)
    assert st == 200 and d["type"] == "message" and d["role"] == "assistant" and d["id"].startswith("msg_")
    assert d["content"] == [{"type": "text", "text": "You said: hi there"}] and d["stop_reason"] == "end_turn"
    assert d["usage"] == {"input_tokens": 2, "output_tokens": 4}
    st, _, raw = call(srv, "anthropic", "/v1/messages", dict(body, max_tokens=2))
    assert json.loads(raw)["stop_reason"] == "max_tokens"
    st, _, raw = call(srv, "anthropic", "/v1/messages", dict(body, stop_sequences=["there"]))
    assert json.loads(raw)["content"][0]["text"] == "You said: hi"
    b2 = dict(body)
    del b2["max_tokens"]
    st, _, raw = call(srv, "anthropic", "/v1/messages", b2)
    assert st == 400 and json.loads(raw)["error"]["type"] == "invalid_request_error"
    st, _, raw = call(srv, "anthropic", "/v1/messages", dict(body, tools=[{"name": "t"}]))
    assert st == 400
    st, _, raw = call(srv, "anthropic", "/v1/messages/count_tokens", {"model": "brain/mock", "messages": [{"role": "user", "content": "x" * 40}]})
    assert st == 200 and json.loads(raw) == {"input_tokens": 10}


def test_anthropic_sse_events(srv):
    body = {"model": "brain/mock", "max_tokens": 64, "stream": True, "messages": [{"role": "user", "content": "a b"}]}
    st, _, raw = call(srv, "anthropic", "/v1/messages", body)
    names = [e for e, _ in sse(raw)]
    assert names[:2] == ["message_start", "content_block_start"]
    assert names[-3:] == ["content_block_stop", "message_delta", "message_stop"]
    assert set(names[2:-3]) == {"content_block_delta"}
    text = "".join(json.loads(d)["delta"]["text"] for e, d in sse(raw) if e == "content_block_delta")
    assert text == "You said: a b"


# ------------------------------------------------------------------------------------ admission
def test_edge_load_shed_is_503_with_retry_after():
    ex = Executor({MockResident.id: MockResident()}, edge_limit=0)
    s = Server(ex, {"openai": 0}).start_background()
    try:
        st, hdr, raw = call(s, "openai", "/v1/models")
        assert st == 503 and hdr.get("Retry-After") == "1" and json.loads(raw)["error"]["code"] == "server_error"
    finally:
        s.shutdown()
        ex.close()


def test_admission_deadline_is_429(monkeypatch):
    class OneAtATime(MockResident):
        def max_concurrency(self):
            return 1
    monkeypatch.setenv("BRAIN_MOCK_DELAY_MS", "1500")
    ex = Executor({MockResident.id: OneAtATime()}, admit_deadline_s=0.2)
    ex.lanes[MockResident.id].warm = True
    s = Server(ex, {"openai": 0}).start_background()
    try:
        res = {}
        t = threading.Thread(target=lambda: res.setdefault("first", chat(s, "slow one")))
        t.start()
        import time
        time.sleep(0.4)
        st, hdr, raw = chat(s, "second")
        t.join()
        assert res["first"][0] == 200
        assert st == 429 and hdr.get("Retry-After") == "1" and json.loads(raw)["error"]["code"] == "rate_limit_exceeded"
    finally:
        s.shutdown()
        ex.close()


# ------------------------------------------------------------------------------------ brain_py transports
def test_brain_py_openai_and_anthropic(srv):
    oa = BrainOpenAI(f"http://127.0.0.1:{srv.bound['openai']}", srv.keys["openai"])
    assert oa.models() == ["brain/mock"]
    assert oa.generate(prompt="ping pong", model="brain/mock").text() == "You said: ping pong"
    toks = []
    out = oa.generate(prompt="a b c", model="brain/mock", on_token=toks.append)
    assert "".join(toks) == out.text() == "You said: a b c" and out.get("completion_tokens") == 5
    assert len(oa.embed("hello", model="brain/mock")) == 8
    with pytest.raises(BrainError) as e:
        BrainOpenAI(f"http://127.0.0.1:{srv.bound['openai']}", "bad").models()
    assert e.value.status == 401
    an = BrainAnthropic(f"http://127.0.0.1:{srv.bound['anthropic']}", srv.keys["anthropic"])
    assert an.chat("yo", model="brain/mock", max_new=16) == "You said: yo"
    toks = []
    an.generate(prompt="x y", model="brain/mock", on_token=toks.append)
    assert "".join(toks) == "You said: x y"
    assert an.count_tokens([{"role": "user", "content": "12345678"}]) == 2


def test_brain_py_jsonl_stdio():
    with Brain(transport="jsonl", env={"BRAIN_MOCK": "1"}, device="cpu") as b:
        mans = b.manifests()
        assert mans[0]["model"] == "brain/mock"
        gen = next(a for a in mans[0]["actions"] if a["name"] == "generate")
        assert gen["streaming"] and any(p["name"] == "messages" for p in gen["params"])
        out = b.generate(prompt="hello there", model="brain/mock")
        assert out.text() == "You said: hello there" and out.get("finish_reason") == "stop"
        toks = []
        b.generate(prompt="a b", model="brain/mock", on_token=toks.append)
        assert "".join(toks) == "You said: a b"
        assert b.converse("hey") == "You said: hey"
        with pytest.raises(BrainError):
            b.run("brain/mock", "generate", {"bogus": 1})
        with pytest.raises(BrainError):
            b.run("brain/none", "generate", {"prompt": "x"})
        assert len(b.embed("abc")) == 8
        with pytest.raises(BrainError):
            b.text2image("a cat")              # no resident provides the action


def test_stats_snapshot_and_brain_top(srv, capsys):
    """GET /stats carries the whole snapshot (models with their actions, executor, accounting), is
    refused without a key, and ``brain top --once`` renders it."""
    from brain_b200.cli.main import main
    code, _, body = call(srv, "openai", "/stats")
    assert code == 200
    snap = json.loads(body)
    assert {"ts", "accelerators", "models", "executor", "requests", "connections", "accounting"} <= set(snap)
    assert snap["models"][0]["id"] == MockResident.id and "generate" in snap["models"][0]["actions"]
    assert call(srv, "openai", "/stats", key=None)[0] == 401
    url = f"http://127.0.0.1:{srv.bound['openai']}"
    assert main(["top", "--url", url, "--key", srv.keys["openai"], "--once"]) == 0
    out = capsys.readouterr().out
    assert "brain top" in out and MockResident.id in out and "connections" in out
    assert main(["top", "--url", url, "--key", "sk-brain-" + "0" * 32, "--once"]) == 1
    assert main(["top", "--url", url]) == 2


def test_serve_stdio_with_a_gpt_checkpoint(tmp_path):
    """``brain serve --stdio --gpt <ckpt>``: a character-level GPT checkpoint is served through the
    same capability API (manifest, streamed tokens, seeded sampling, vocabulary errors)."""
    import torch
    from brain_b200.checkpoint import st
    from brain_b200.models.config import GptConfig
    from brain_b200.models.gpt2 import Gpt2
    itos = list("\n abcdefghijklmnopqrstuvwxyz=+0123456789")
    cfg = GptConfig(vocab=len(itos), block_size=32, n_layers=1, d_model=16, n_heads=2, d_ff=32)
    m = Gpt2(cfg).init_weights(1)
    ck = str(tmp_path / "g.safetensors")
    conf = m.config_json()
    conf["itos"] = itos
    st.save(ck, m.reference_state(), conf, None)
    with Brain(transport="jsonl", args=["--gpt", ck, "--max-new", "6", "--seed", "7"], device="cpu") as b:
        man = next(x for x in b.manifests() if x["model"] == "brain/gpt2")
        gen = next(a for a in man["actions"] if a["name"] == "generate")
        assert next(p for p in gen["params"] if p["name"] == "max_new")["default"] == 6
        toks = []
        out = b.generate(prompt="abc", model="brain/gpt2", on_token=toks.append)
        assert len(out.text()) == 6 and "".join(toks) == out.text() and out.get("completion_tokens") == 6
        again = b.generate(prompt="abc", model="brain/gpt2")
        assert again.text() == out.text()                       # same seed, same text
        greedy = b.generate(prompt="abc", model="brain/gpt2", temp=0.0, max_new=4)
        assert len(greedy.text()) == 4
        with pytest.raises(BrainError):
            b.generate(prompt="ABC!", model="brain/gpt2")        # characters outside the vocabulary


def test_jsonl_protocol_over_unix_socket_and_tcp(tmp_path):
    """The stdio protocol served per connection over a Unix socket and a loopback TCP port."""
    import socket
    from brain_b200.api.stdio import SocketServer
    ex = Executor({MockResident.id: MockResident()})

    def talk(sock):
        rd, wr = sock.makefile("r", encoding="utf-8"), sock.makefile("w", encoding="utf-8")
        assert json.loads(rd.readline())["event"] == "ready"
        wr.write(json.dumps({"event": "action_request", "req_id": "7", "model": "brain/mock", "action": "generate",
                             "params": {"prompt": "over a socket"}}) + "\n")
        wr.flush()
        text, final = "", None
        while final is None:
            ev = json.loads(rd.readline())
            assert ev.get("req_id") == "7"
            if ev["event"] == "action_progress":
                text += ev.get("message", "")
            elif ev["event"] in ("action_result", "error"):
                final = ev
        assert final["event"] == "action_result" and text == "You said: over a socket"
    path = str(tmp_path / "brain.sock")
    open(path, "w").write("stale")                       # a stale file at the path is replaced
    u = SocketServer(ex, unix_path=path).start()
    t = SocketServer(ex, tcp_port=0).start()
    try:
        assert oct(os.stat(path).st_mode & 0o777) == "0o600"
        with socket.socket(socket.AF_UNIX, socket.SOCK_STREAM) as s:
            s.connect(path)
            talk(s)
        with socket.create_connection(("127.0.0.1", t.port), timeout=10) as s:
            talk(s)
        with pytest.raises(ValueError):
            SocketServer(ex)
    finally:
        u.close()
        t.close()
        ex.close()
    assert not os.path.exists(path)


# ------------------------------------------------------------------------------------ response schemas
# A compact restatement of the required fields and types of the published response objects (the
# reference validates against vendored OpenAPI documents, crates/apiserve/tests/api.rs); a value is a
# type, a tuple of alternatives, a dict of required fields, a one-element list (array of that), or
# a callable predicate.  Keys ending in "?" are optional but typed when present.
NULLABLE_STR = (str, type(None))
USAGE = {"prompt_tokens": int, "completion_tokens": int, "total_tokens": int}
TOOL_CALL = {"id": str, "type": lambda v: v == "function", "function": {"name": str, "arguments": str}}
CHAT_COMPLETION = {
    "id": str, "object": lambda v: v == "chat.completion", "created": int, "model": str,
    "choices": [{"index": int, "finish_reason": lambda v: v in ("stop", "length", "tool_calls", "content_filter"),
                 "message": {"role": lambda v: v == "assistant", "content": NULLABLE_STR, "tool_calls?": [TOOL_CALL]}}],
    "usage": USAGE}
CHAT_CHUNK = {
    "id": str, "object": lambda v: v == "chat.completion.chunk", "created": int, "model": str,
    "choices": [{"index": int, "delta": dict,
                 "finish_reason": lambda v: v in (None, "stop", "length", "tool_calls", "content_filter")}],
    "usage?": (USAGE, type(None))}
MODEL_LIST = {"object": lambda v: v == "list", "data": [{"id": str, "object": lambda v: v == "model",
                                                          "created": int, "owned_by": str}]}
EMBEDDINGS = {"object": lambda v: v == "list", "model": str, "usage": {"prompt_tokens": int, "total_tokens": int},
              "data": [{"object": lambda v: v == "embedding", "index": int, "embedding": [float]}]}
OPENAI_ERROR = {"error": {"message": str, "type": str, "param": NULLABLE_STR, "code": NULLABLE_STR}}
ANTHROPIC_MESSAGE = {
    "id": str, "type": lambda v: v == "message", "role": lambda v: v == "assistant", "model": str,
    "content": [{"type": lambda v: v in ("text", "tool_use", "thinking")}],
    "stop_reason": lambda v: v in ("end_turn", "max_tokens", "stop_sequence", "tool_use"),
    "stop_sequence": NULLABLE_STR, "usage": {"input_tokens": int, "output_tokens": int}}
ANTHROPIC_ERROR = {"type": lambda v: v == "error", "error": {"type": str, "message": str}}


def conforms(value, schema, path="$"):
    """Raise AssertionError naming the first path where ``value`` departs from ``schema``."""
    if isinstance(schema, dict):
        assert isinstance(value, dict), f"{path}: expected an object, got {type(value).__name__}"
        for key, sub in schema.items():
            opt = key.endswith("?")
            k = key[:-1] if opt else key
            if k not in value:
                assert opt, f"{path}.{k}: missing"
                continue
            conforms(value[k], sub, f"{path}.{k}")
    elif isinstance(schema, list):
        assert isinstance(value, list), f"{path}: expected an array"
        for i, v in enumerate(value):
            conforms(v, schema[0], f"{path}[{i}]")
    elif isinstance(schema, tuple):
        errs = []
        for alt in schema:
            try:
                conforms(value, alt, path)
                return
            except AssertionError as e:
                errs.append(str(e))
        raise AssertionError(f"{path}: no alternative matched ({'; '.join(errs)})")
    elif isinstance(schema, type):
        ok = isinstance(value, schema) and not (schema is int and isinstance(value, bool))
        if schema is float:
            ok = isinstance(value, (int, float)) and not isinstance(value, bool)
        assert ok, f"{path}: expected {schema.__name__}, got {value!r}"
    else:
        assert schema(value), f"{path}: unexpected value {value!r}"


def test_response_objects_conform_to_the_published_schemas(srv):
    with pytest.raises(AssertionError):
        conforms({"id": "x"}, CHAT_COMPLETION)                  # the checker itself rejects a stub
    for provider in ("openai", "openrouter"):
        st, _, raw = call(srv, provider, "/v1/models")
        conforms(json.loads(raw), MODEL_LIST)
        st, _, raw = chat(srv, provider=provider, max_tokens=5)
        assert st == 200
        conforms(json.loads(raw), CHAT_COMPLETION)
        tools = [{"type": "function", "function": {"name": "get_weather", "parameters": {"type": "object"}}}]
        st, _, raw = chat(srv, TOOL_CALL_TRIGGER, provider=provider, tools=tools)
        d = json.loads(raw)
        conforms(d, CHAT_COMPLETION)
        assert d["choices"][0]["finish_reason"] == "tool_calls" and d["choices"][0]["message"]["tool_calls"]
        st, _, raw = chat(srv, provider=provider, stream=True, stream_options={"include_usage": True})
        events = [d for _, d in sse(raw)]
        assert events[-1] == "[DONE]"
        chunks = [json.loads(d) for d in events[:-1]]
        for c in chunks:
            conforms(c, CHAT_CHUNK)
        assert chunks[-1]["usage"] and chunks[0]["choices"][0]["delta"].get("role") == "assistant"
        # every error status carries the error object
        for st_want, (path, body, key) in {401: ("/v1/models", None, "bad"), 404: ("/v1/nope", None, "ok"),
                                           400: ("/v1/chat/completions", {"model": "brain/mock"}, "ok")}.items():
            st, _, raw = call(srv, provider, path, body, key=key)
            assert st == st_want
            conforms(json.loads(raw), OPENAI_ERROR)
    st, _, raw = call(srv, "openai", "/v1/embeddings", {"model": "brain/mock", "input": ["a", "b"]})
    conforms(json.loads(raw), EMBEDDINGS)
    st, _, raw = call(srv, "anthropic", "/v1/messages", {"model": "brain/mock", "max_tokens": 16,
                                                        "messages": [{"role": "user", "content": "hi"}]})
    assert st == 200
    conforms(json.loads(raw), ANTHROPIC_MESSAGE)
    st, _, raw = call(srv, "anthropic", "/v1/messages", {"model": "brain/mock"})
    assert st == 400
    conforms(json.loads(raw), ANTHROPIC_ERROR)
