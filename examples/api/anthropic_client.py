#!/usr/bin/env python3
"""Anthropic Messages surface through `brain_py.BrainAnthropic`.

    BRAIN_MOCK=1 python examples/api/anthropic_client.py          # starts ./brain serve --anthropic itself
    python examples/api/anthropic_client.py --base-url http://127.0.0.1:8787 --api-key KEY"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from brain_py import BrainAnthropic  # noqa: E402
from brain_py.base import skip  # noqa: E402


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", default="brain/mock")
    ap.add_argument("--base-url")
    ap.add_argument("--api-key", default="")
    ap.add_argument("--brain", default=os.path.join(ROOT, "brain"))
    a = ap.parse_args()
    proc = None
    with tempfile.TemporaryDirectory() as tmp:
        base, key = a.base_url, a.api_key
        if not base:
            ready, keys = os.path.join(tmp, "ready.json"), os.path.join(tmp, "keys.json")
            proc = subprocess.Popen([sys.executable, a.brain, "serve", "--anthropic", "0", "--ready-file", ready,
                                     "--api-keys-out", keys], stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)
            t_end = time.time() + 300
            while not os.path.exists(ready):
                if proc.poll() is not None or time.time() > t_end:
                    skip("could not start ./brain serve --anthropic")
                time.sleep(0.05)
            base = f"http://127.0.0.1:{json.load(open(ready))['ports']['anthropic']}"
            key = json.load(open(keys))["anthropic"]
        try:
            with BrainAnthropic(base, key) as brain:
                if a.model not in brain.models():
                    skip(f"{a.model} is not served at {base}")
                msgs = [{"role": "user", "content": "Name three colours."}]
                print("count_tokens:", brain.count_tokens(msgs, system="Be brief."))
                print("message:", brain.generate(messages=msgs, model=a.model, max_new=32).text().strip())
                sys.stdout.write("streamed: ")
                out = brain.generate(messages=msgs, model=a.model, max_new=32,
                                     on_token=lambda t: (sys.stdout.write(t), sys.stdout.flush()))
                print("\nfinish:", out.get("finish_reason") or out.get("finish"))
        finally:
            if proc is not None:
                proc.terminate()
                proc.wait(timeout=30)


if __name__ == "__main__":
    main()
