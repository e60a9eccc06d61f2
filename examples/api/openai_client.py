#!/usr/bin/env python3
"""OpenAI-surface walk-through with nothing but the standard library.

    BRAIN_MOCK=1 python examples/api/openai_client.py                       # starts ./brain serve itself
    python examples/api/openai_client.py --base-url http://127.0.0.1:8788 --keys-file keys.json

Calls, in order: GET /v1/models, POST /v1/chat/completions (plain, then `stream: true` reading the
SSE deltas), POST /v1/embeddings, POST /v1/images/generations (saved to --out)."""
import argparse
import base64
import json
import os
import subprocess
import sys
import tempfile
import time
import urllib.error
import urllib.request

EXIT_SKIP = 77
ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def call(base, key, path, body=None, stream=False):
    req = urllib.request.Request(base + path, data=None if body is None else json.dumps(body).encode(),
                                 headers={"Authorization": f"Bearer {key}", "Content-Type": "application/json"})
    resp = urllib.request.urlopen(req, timeout=120)
    if stream:
        return resp
    with resp:
        return json.loads(resp.read())


def sse(resp):
    """Yield the JSON payload of every `data:` line until `[DONE]`."""
    with resp:
        for raw in resp:
            line = raw.decode().strip()
            if not line.startswith("data:"):
                continue
            data = line[5:].strip()
            if data == "[DONE]":
                return
            yield json.loads(data)


def launch(brain, workdir):
    ready, keys = os.path.join(workdir, "ready.json"), os.path.join(workdir, "keys.json")
    p = subprocess.Popen([sys.executable, brain, "serve", "--openai", "0", "--ready-file", ready,
                          "--api-keys-out", keys], stdout=subprocess.DEVNULL, stderr=subprocess.PIPE, text=True)
    t_end = time.time() + 300
    while not os.path.exists(ready):
        if p.poll() is not None or time.time() > t_end:
            print("server did not start:", p.stderr.read() if p.poll() is not None else "timeout", file=sys.stderr)
            sys.exit(EXIT_SKIP)
        time.sleep(0.05)
    port = json.load(open(ready))["ports"]["openai"]
    return p, f"http://127.0.0.1:{port}", json.load(open(keys))["openai"]


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", default="brain/mock")
    ap.add_argument("--base-url")
    ap.add_argument("--api-key")
    ap.add_argument("--keys-file")
    ap.add_argument("--brain", default=os.path.join(ROOT, "brain"))
    ap.add_argument("--out", default=os.path.join(tempfile.gettempdir(), "brain_example_image.bin"))
    a = ap.parse_args()
    proc = None
    with tempfile.TemporaryDirectory() as tmp:
        if a.base_url:
            key = a.api_key or (json.load(open(a.keys_file))["openai"] if a.keys_file else None)
            if not key:
                ap.error("--base-url needs --api-key or --keys-file")
            base = a.base_url.rstrip("/")
        else:
            proc, base, key = launch(a.brain, tmp)
        try:
            models = [m["id"] for m in call(base, key, "/v1/models")["data"]]
            print("models:", ", ".join(models))
            if a.model not in models:
                print(f"{a.model} is not served here", file=sys.stderr)
                sys.exit(EXIT_SKIP)
            msgs = [{"role": "user", "content": "Say hello in five words."}]
            r = call(base, key, "/v1/chat/completions", {"model": a.model, "messages": msgs, "max_tokens": 32})
            print("chat:", r["choices"][0]["message"]["content"].strip(), "| usage:", r.get("usage"))
            parts = []
            for ev in sse(call(base, key, "/v1/chat/completions",
                               {"model": a.model, "messages": msgs, "max_tokens": 32, "stream": True}, stream=True)):
                for ch in ev.get("choices", []):
                    parts.append(ch.get("delta", {}).get("content") or "")
            print("stream:", "".join(parts).strip())
            try:
                e = call(base, key, "/v1/embeddings", {"model": a.model, "input": "a sentence to embed"})
                print("embedding: dim", len(e["data"][0]["embedding"]))
            except urllib.error.HTTPError as err:
                print("embeddings: not offered by this model:", err.code)
            try:
                im = call(base, key, "/v1/images/generations",
                          {"model": a.model, "prompt": "a red square", "response_format": "b64_json"})
                blob = base64.b64decode(im["data"][0]["b64_json"])
                open(a.out, "wb").write(blob)
                print(f"image: {len(blob)} bytes -> {a.out}")
            except urllib.error.HTTPError as err:
                print("images: not offered by this model:", err.code)
        finally:
            if proc is not None:
                proc.terminate()
                proc.wait(timeout=30)


if __name__ == "__main__":
    main()
