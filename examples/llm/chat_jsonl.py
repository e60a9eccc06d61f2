#!/usr/bin/env python3
"""`brain_py` over the JSONL stdio transport: the client starts `brain serve --stdio` as a child and
talks newline-delimited JSON over its pipes.

    BRAIN_MOCK=1 python examples/llm/chat_jsonl.py
    BRAIN_QWEN_WEIGHTS=model.safetensors BRAIN_QWEN_TOKENIZER=tok/ python examples/llm/chat_jsonl.py --model brain/qwen3"""
import argparse
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from brain_py import Brain  # noqa: E402
from brain_py.base import BrainError, skip  # noqa: E402


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", default=None, help="model id (default: the first one that offers generate)")
    ap.add_argument("--brain", default=os.path.join(ROOT, "brain"))
    a = ap.parse_args()
    try:
        brain = Brain(transport="jsonl", brain_bin=a.brain, env=dict(os.environ))
    except (BrainError, OSError) as e:
        skip(f"cannot start the server: {e}")
    with brain:
        for m in brain.manifests():
            print(f"{m['model']}: " + ", ".join(x["name"] for x in m["actions"]))
        model = a.model or brain.model_for("generate")
        print("chat:", brain.chat("What is the capital of Sweden?", model=model, max_new=32).strip())
        sys.stdout.write("streamed: ")
        out = brain.generate("Count from one to five.", model=model, max_new=32, seed=7, temp=0.7,
                             on_token=lambda t: (sys.stdout.write(t), sys.stdout.flush()))
        print("\ntokens:", out.get("completion_tokens"), "finish:", out.get("finish_reason"))


if __name__ == "__main__":
    main()
