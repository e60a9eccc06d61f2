"""``brain serve`` (reference: crates/cli/src/run_cli.rs:186-263 flag set: ``--stdio --gpt --yolo
--max-new --temp --top-k --seed --conf --dbus --dbus-system --dbus-name --reserve-gb --models-dir
--anthropic [8787] --openai [8788] --openrouter [8789] --api-keys-out FILE --ready-file PATH
-v/--verbose [0-3]``; HTTP binds localhost only, there is no ``--listen``)."""
from __future__ import annotations

import json
import sys
import time
from typing import List

from ..cli.args import Args
from ..utils import shutdown, trace
from . import auth
from .executor import Executor
from .resident import registry_from_env
from .server import DEFAULT_PORTS, Server


def _port_flag(args: List[str], name: str):
    """``--openai`` alone selects the default port; ``--openai 9000`` a specific one."""
    if name not in args:
        return None
    i = args.index(name)
    if i + 1 < len(args) and args[i + 1].isdigit():
        port = int(args[i + 1])
        del args[i:i + 2]
        return port
    del args[i]
    return DEFAULT_PORTS[name[2:]]


def store_residency(models_dir, reserve_gb, device: str, already: set):
    """Suppliers for every model in the on-disk store (``--models-dir`` / BRAIN_MODELS_DIR; the default
    root is only used when one of the two names it), loaded on first use.  Budget per device: its
    memory minus ``--reserve-gb`` (default 8) on a GPU, ``BRAIN_RESIDENCY_BUDGET_GB`` (default 64) on
    the CPU.  None when there is no store or it is empty."""
    import os
    from ..modelstore import Store
    from .residency import Residency, StoreSupplier
    root = models_dir or os.environ.get("BRAIN_MODELS_DIR")
    if not root or not os.path.isdir(root):
        return None
    sup = {}
    for lm in Store(root).scan():
        if lm.card is not None and getattr(lm.card, "family", "qwen") not in ("qwen", "qwen3"):
            continue
        s = StoreSupplier(lm, weights="int8" if os.environ.get("BRAIN_QWEN_INT8") == "1" else "bf16",
                          kv_dtype="int8" if os.environ.get("BRAIN_QWEN_KV_INT8") == "1" else "bf16")
        if s.id not in already:
            sup[s.id] = s
    if not sup:
        return None
    import torch
    from ..train import pick_device
    dev = pick_device(device)
    if dev.type == "cuda":
        reserve = float(reserve_gb) if reserve_gb else 8.0
        budgets = {}
        for i in range(torch.cuda.device_count()):
            total = torch.cuda.get_device_properties(i).total_memory
            budgets[f"cuda:{i}"] = max(int(total - reserve * 2**30), 0)
    else:
        budgets = {"cpu": int(float(os.environ.get("BRAIN_RESIDENCY_BUDGET_GB", "64")) * 2**30)}
    return Residency(sup, budgets, busy_wait_s=5.0)   # a load waits briefly for a busy victim before a 429


def run_serve(argv: List[str], device: str = "auto") -> int:
    args = list(argv)
    ports = {p: _port_flag(args, "--" + p) for p in ("anthropic", "openai", "openrouter")}
    ports = {k: v for k, v in ports.items() if v is not None}
    a = Args(args)
    stdio = a.take_flag("--stdio")
    keys_out = a.take_str("--api-keys-out")
    ready = a.take_str("--ready-file")
    verbose = a.int_or("--verbose", a.int_or("-v", 1))
    defaults = {}
    for flag, key, conv in (("--max-new", "max_new", int), ("--temp", "temp", float), ("--top-k", "top_k", int),
                            ("--seed", "seed", int)):
        v = a.take_str(flag)
        if v is not None:
            defaults[key] = conv(v)
    gpt_ckpt = a.take_str("--gpt")
    for f in ("--dbus", "--dbus-system"):
        if a.take_flag(f):
            print(f"serve: {f} is not available in this build (no D-Bus); ignoring", file=sys.stderr)
    if a.take_str("--yolo") is not None:
        print("serve: --yolo is not available in this build (no vision stack); ignoring", file=sys.stderr)
    models_dir = a.take_str("--models-dir")
    reserve_gb = a.take_str("--reserve-gb")
    for f in ("--dbus-name", "--conf"):
        a.take_str(f)
    a.finish()
    if not stdio and not ports:
        print("usage: brain serve [--stdio | --openai [PORT] --anthropic [PORT] --openrouter [PORT]] "
              "[--api-keys-out FILE --ready-file PATH --models-dir DIR --reserve-gb G -v N]   (models: BRAIN_MOCK=1, BRAIN_QWEN_WEIGHTS=FILE, BRAIN_MODEL=vendor/repo[:owner:name:tag])",
              file=sys.stderr)
        return 2
    models = registry_from_env(load=True, device=device)
    if gpt_ckpt:
        from .resident import load_gpt
        try:
            g = load_gpt(gpt_ckpt, device, defaults)
        except Exception as e:  # noqa: BLE001
            print(f"serve: --gpt {gpt_ckpt}: {e}", file=sys.stderr)
            return 1
        models[g.id] = g
    residency = store_residency(models_dir, reserve_gb, device, set(models))
    if not models and residency is None:
        print("serve: no model selected — set BRAIN_QWEN_WEIGHTS (and BRAIN_QWEN_TOKENIZER), BRAIN_MODEL (a model-store reference) or BRAIN_MOCK=1",
              file=sys.stderr)
        return 1
    ex = Executor(models, residency=residency)
    shutdown.install()
    server = None
    try:
        if ports:
            server = Server(ex, ports).start_background()
            server.announce(lambda s: print(s, flush=True))
            if keys_out:
                auth.write_keys(keys_out, server.keys)
        if ready:
            shutdown.write_ready_file(ready, json.dumps({"ports": server.bound if server else {},
                                                         "models": list(models)}) + "\n")
        if stdio:
            from .stdio import StdioServer
            StdioServer(ex, defaults=defaults).serve()
        else:
            last = time.time()
            while not shutdown.wait(0.5):
                if verbose >= 2 and time.time() - last > 10:
                    from ..utils.stats import snapshot
                    print("stats " + json.dumps(snapshot(ex)["executor"]), file=sys.stderr)
                    last = time.time()
    finally:
        if server is not None:
            server.shutdown()
        ex.close()
    return 0
