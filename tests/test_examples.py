"""Every script under examples/ runs offline to exit code 0 (the reference's tests/e2e/examples.bats:
each example against the deterministic mock model)."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CASES = [
    ("api/openai_client.py", [], ["models: brain/mock", "chat:", "stream:"]),
    ("api/anthropic_client.py", [], ["count_tokens:", "message:", "streamed:"]),
    ("llm/chat_jsonl.py", [], ["brain/mock:", "chat:", "streamed:"]),
    ("serving/offline_batch.py", ["--requests", "8", "--max-batch", "3", "--max-new", "6"],
     ["cancelled request", "prefix cache served", "(one forward)"]),
    ("train/tiny_gpt2.py", ["--steps", "30", "--device", "cpu"], ["loss", "sample: the quick"]),
]


def test_every_example_file_has_a_case():
    found = set()
    for d, _, files in os.walk(os.path.join(ROOT, "examples")):
        for f in files:
            if f.endswith(".py"):
                found.add(os.path.relpath(os.path.join(d, f), os.path.join(ROOT, "examples")))
    assert found == {c[0] for c in CASES}


@pytest.mark.parametrize("script,args,expect", CASES, ids=[c[0] for c in CASES])
def test_example_runs_against_the_mock(script, args, expect):
    env = dict(os.environ, BRAIN_MOCK="1", PYTHONPATH=ROOT, CUDA_VISIBLE_DEVICES="")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "examples", script), *args], env=env,
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, f"{r.stdout}\n{r.stderr}"
    for e in expect:
        assert e in r.stdout, f"missing {e!r} in:\n{r.stdout}\n{r.stderr}"
