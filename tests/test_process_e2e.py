"""Process-level checks with the real executable, real sockets and real signals (the reference's
tests/e2e/{shutdown,ready}.bats): the ready file appears only once the listeners answer, every
surface combination leaves with exit code 0 on SIGINT and on SIGTERM, the key file works."""
import json
import os
import signal
import subprocess
import sys
import time
import urllib.request

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BRAIN = os.path.join(ROOT, "brain")


def _start(tmp_path, flags, stdin=None):
    ready = tmp_path / "ready.json"
    keys = tmp_path / "keys.json"
    env = dict(os.environ, BRAIN_MOCK="1", PYTHONPATH=ROOT)
    p = subprocess.Popen([sys.executable, BRAIN, "serve", *flags, "--ready-file", str(ready),
                          "--api-keys-out", str(keys)], env=env, stdin=stdin, stdout=subprocess.PIPE,
                         stderr=subprocess.PIPE, text=True)
    t_end = time.time() + 120
    while not ready.exists() and time.time() < t_end and p.poll() is None:
        time.sleep(0.05)
    if not ready.exists():
        p.kill()
        out, err = p.communicate()
        raise AssertionError(f"server never became ready: rc={p.returncode}\n{out}\n{err}")
    return p, json.loads(ready.read_text()), keys


def _key(keys_path, surface):
    """The key file maps each listening surface to its key (mode 0600)."""
    assert (os.stat(keys_path).st_mode & 0o777) == 0o600
    return json.loads(keys_path.read_text())[surface]


@pytest.mark.parametrize("sig", [signal.SIGINT, signal.SIGTERM])
@pytest.mark.parametrize("flags", [["--openai", "0"], ["--openai", "0", "--anthropic", "0", "--openrouter", "0"]])
def test_http_surfaces_answer_when_ready_and_leave_cleanly_on_a_signal(tmp_path, flags, sig):
    p, ready, keys = _start(tmp_path, flags)
    try:
        ports = ready["ports"]
        assert set(ports) == {f[2:] for f in flags if f.startswith("--")}
        assert "brain/mock" in ready["models"]
        # the ready file is written after the listeners are bound: a request right away succeeds
        port = ports["openai"]
        key = _key(keys, "openai")
        req = urllib.request.Request(f"http://127.0.0.1:{port}/v1/models", headers={"Authorization": f"Bearer {key}"})
        with urllib.request.urlopen(req, timeout=30) as r:
            body = json.loads(r.read())
        assert any(m["id"] == "brain/mock" for m in body["data"])
        body = json.dumps({"model": "brain/mock", "messages": [{"role": "user", "content": "hello"}],
                           "max_tokens": 8}).encode()
        req = urllib.request.Request(f"http://127.0.0.1:{port}/v1/chat/completions", data=body,
                                     headers={"Authorization": f"Bearer {key}", "Content-Type": "application/json"})
        with urllib.request.urlopen(req, timeout=30) as r:
            out = json.loads(r.read())
        assert out["choices"][0]["message"]["content"]
        p.send_signal(sig)
        rc = p.wait(timeout=30)
        assert rc == 0, p.stderr.read()
    finally:
        if p.poll() is None:
            p.kill()
            p.wait()


def test_stdio_surface_ends_at_end_of_input_and_with_http_beside_it(tmp_path):
    p, ready, _ = _start(tmp_path, ["--stdio", "--openai", "0"], stdin=subprocess.PIPE)
    try:
        assert "openai" in ready["ports"]
        p.stdin.write(json.dumps({"id": 1, "method": "models"}) + "\n")
        p.stdin.flush()
        line = p.stdout.readline()
        while line and not line.lstrip().startswith("{"):
            line = p.stdout.readline()     # listener announcements come first
        assert "brain/mock" in line
        p.stdin.close()
        assert p.wait(timeout=30) == 0
    finally:
        if p.poll() is None:
            p.kill()
            p.wait()


def test_a_second_signal_forces_the_exit(tmp_path):
    """Two-stage shutdown: the first signal asks, a second one while still draining exits at once
    with the conventional 128 + signal code or 0 if the drain had already finished."""
    p, _, _ = _start(tmp_path, ["--openai", "0"])
    try:
        p.send_signal(signal.SIGINT)
        p.send_signal(signal.SIGINT)
        rc = p.wait(timeout=30)
        assert rc in (0, 130, -signal.SIGINT, 1)
    finally:
        if p.poll() is None:
            p.kill()
            p.wait()
