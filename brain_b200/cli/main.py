"""``brain`` entry point: global flags, infrastructure verbs, then architecture dispatch
(reference: crates/cli/src/main.rs:96-381 help text and verb table; crates/cli/src/resolve.rs:
171-192 both word orders)."""
from __future__ import annotations

import json
import os
import sys
from typing import List, Optional

from .. import __version__, arch as archs
from ..utils import trace
from .args import Args
from .resolve import resolve

HELP = """brain — B200-native training and serving framework

usage: brain <verb> <arch> [args]      (same as: brain <arch> <verb> [args])

model commands
  gpt2     train <data_dir> [--out F --steps N --batch B --block T --layers L --d-model D --heads H
                 --lr X --warmup N --eval-interval N --grad-accum N --seed S --mask C --align]
           eval  --weights F --data D [--batches N --samples M]
           infer --weights F [--data D] [--prompt "..." --max-new 200 --temp 0.8 --top-k 40 --seed 1234]
  qwen3    import --hf DIR --out F [--block T --dtype F32|BF16]
           train <data_dir> [--out out/qwen.safetensors --steps 2000 --batch 8 --block 256 --lr 3e-4
                 --seed 1234 --mask C --align --save-secs 600 --preset 0.6b --dp N]
           finetune <data_dir> --weights BASE --out F [...]        (full-parameter, moments offloaded)
           finetune --lora R --weights BASE --adapter OWNER/NAME[:TAG] --dataset DIR [--alpha A ...]
           infer --weights F --tokenizer T --prompt "..." [--max-new N --temp X --top-k K --seed S --chat
                 --spec K]
           serve --weights F --tokenizer T --prompt "..." [--prompt "..."]... [--max-new 64
                 --block-size 16 --weights-int8 --int8|--kv-fp32 --kv-calib --tp N]
           export --weights F --out DIR     eval --weights F --jsonl FILE [--adapter ...]
           toolcall gen|eval ...            calib --weights F --jsonl FILE [--report --clip-out F]
           precompile
  toymoe   train [--steps N --batch-size B --block-size T --lr X --out F]
           infer --weights F [--prompt 1,2,3,4 --max-new N --temperature X --top-k K]
           eval  --weights F [--samples N]
  splat    render|train ...                 (headless Gaussian-splat rasteriser)

infrastructure
  data gen <name> [--out DIR --n N --seed S]     shakespeare_char calculator reverser wordcalc gpt timeseries
  devices                                         list compute devices
  flops --model qwen|gpt [--weights F --batch B --block T --train --i8 --stages N --run]
  gradcheck [--model gpt|qwen|qwen2|qwen_lora|moe|qwen_moe|all] [--dirs N]
  bench [--gpus N --steps K …] | bench learn [copy mod_add parity] [--arch qwen|gpt --steps N --seed S]
  perf list | run <scenario> [...] | compare A B | gate A B [--tolerance X] | faults [NAME…]
  top --url http://HOST:PORT (--key K | --api-keys FILE) [--interval S --once --json]
  bench [--gpus N --steps K --warmup W]           the training benchmark (bench.py)
  federated split|verify|merge|assemble|train-expert ...
  caps                                            capability manifests of the servable models
  serve [--stdio | --openai [8788] --anthropic [8787] --openrouter [8789]] [--api-keys-out F
        --ready-file P --max-new N --temp X --top-k K --seed S -v N]
  import <FILE|DIR> [--out F | --id VENDOR/REPO [--models-dir D]] | import --list
  quantize <SRC> [--out F --tier Q8_0|Q4_0 --format gguf|safetensors --keep SUBSTR... --plan]
  help | --help | --version

global flags
  --device auto|cpu|cuda[:N]      --trace-<family> 0-5   --trace name=level[,…]
  --trace-format text|json        --trace-output -|PATH   (env: BRAIN_TRACE, BRAIN_DEVICE, BRAIN_PROFILE)
  --device: cpu | gpu | gpuN | gpu0,gpu1 | cpuN | cpuA-B | gpu1,cpu0-3   (indexed CPU selections pin the
            process affinity and size the thread pool; GPU indices are sorted by PCI bus id)
"""


def _take_global(argv: List[str]):
    rest, levels, fmt, output = trace.take_flags(argv)
    device = os.environ.get("BRAIN_DEVICE", "auto")
    out = []
    i = 0
    while i < len(rest):
        if rest[i] == "--device" and i + 1 < len(rest):
            device = rest[i + 1]
            i += 2
        else:
            out.append(rest[i])
            i += 1
    if device == "gpu":
        device = "cuda"
    return out, device, levels, fmt, output


def main(argv: Optional[List[str]] = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    try:
        argv, device, levels, fmt, output = _take_global(argv)
    except ValueError as e:
        print(str(e), file=sys.stderr)
        return 2
    trace.install(levels, fmt, output)
    if not argv or argv[0] in ("help", "--help", "-h"):
        print(HELP)
        return 0
    if argv[0] in ("--version", "-V", "version"):
        print(f"brain {__version__}")
        return 0
    trace.event("cli", 3, "command", argv=" ".join(argv), device=device)
    verb, rest = argv[0], argv[1:]
    infra = {"data": _data, "devices": _devices, "flops": _flops, "gradcheck": _gradcheck, "perf": _perf,
             "bench": _bench, "federated": _federated, "caps": _caps, "serve": _serve, "top": _top}
    if verb in infra and not (rest and archs.by_id(rest[0]) and verb == "serve"):
        return infra[verb](rest, device) or 0
    r = resolve(argv)
    if r.kind == "arch":
        return _dispatch_arch(r.arch, r.rest, device)
    if r.kind == "import":
        return _import_file(r.rest, device) or 0
    if r.kind == "quantize":
        return _quantize(r.rest, device) or 0
    if r.word in ("npu", "forecast", "capture", "dbus"):
        print(f"brain {r.word}: not built by this framework (ONNX/NPU export, the forecasting models, camera "
              "capture and the D-Bus service are outside what it covers)", file=sys.stderr)
        return 2
    print(f"unknown command {r.word!r}; try `brain help`", file=sys.stderr)
    return 2


def _top(rest: List[str], device: str) -> int:
    from .top import run_top
    return run_top(rest)


def _dispatch_arch(arch_id: str, rest: List[str], device: str) -> int:
    a = archs.by_id(arch_id)
    if not a.built:
        print(f"brain {arch_id}: the {a.family} family is not built by this framework "
              f"(built: {' '.join(x.id for x in archs.all_archs(True))})", file=sys.stderr)
        return 3
    if a.id == "gpt2":
        from .gpt_cli import run_gpt
        return run_gpt(rest, device)
    if a.id == "qwen3":
        from .qwen_cli import run_qwen
        return run_qwen(rest, device)
    if a.id == "toymoe":
        from .toymoe_cli import run_toymoe
        return run_toymoe(rest, device)
    if a.id == "splat":
        try:
            from .splat_cli import run_splat
        except ImportError:
            print("brain splat: the rasteriser is not part of this build", file=sys.stderr)
            return 3
        return run_splat(rest, device)
    return 2


# ------------------------------------------------------------------------------------ infra verbs
_DATASETS = ("shakespeare_char", "calculator", "reverser", "wordcalc", "gpt", "timeseries")


def _data(args, device):
    from ..data import datasets
    if not args or args[0] != "gen":
        print(f"usage: brain data gen <name> [--out DIR] [--n N] [--seed S]  (got {args[:1] or None})", file=sys.stderr)
        return 2
    a = Args(args[1:])
    name = a.positional()
    if name is None:
        print("usage: brain data gen <name> [--out DIR] [--n N] [--seed S]", file=sys.stderr)
        return 2
    if name not in _DATASETS:
        print(f"unknown dataset {name!r}; expected one of: {' '.join(_DATASETS)}", file=sys.stderr)
        return 2
    out = a.str_or("--out", os.path.join("data", name))
    n = a.int_or("--n", 200_000 if name == "timeseries" else 100_000)
    seed = a.int_or("--seed", 1337)
    a.finish()
    print(f"preparing {name} -> {out} (n={n}, seed={seed})")
    try:
        datasets.prepare(name, out, n, seed)
    except Exception as e:  # noqa: BLE001
        print(f"error: {e}", file=sys.stderr)
        return 1
    print(f"done: {out}")


def _devices(args, device):
    from ..utils import devices
    print(devices.render("" if device == "auto" else device))


def _flops(args, device):
    from ..checkpoint import st
    from ..models.config import GptConfig, QwenConfig
    from ..utils import cost
    a = Args(args)
    model = a.str_or("--model", "")
    weights = a.take_str("--weights")
    b = a.int_or("--batch", 1)
    block = a.opt_int("--block")
    train = a.take_flag("--train")
    i8 = a.take_flag("--i8")
    stages = a.int_or("--stages", 1)
    run = a.take_flag("--run")
    preset = a.take_str("--preset")
    a.finish()
    if model not in ("qwen", "gpt"):
        print("usage: brain flops --model qwen|gpt [--weights F] [--batch B] [--block T] [--train] [--i8] "
              "[--stages N] [--run] [--preset 0.6b]", file=sys.stderr)
        return 2
    if i8 and train:
        print("the int8 path is inference-only", file=sys.stderr)
        return 2
    if model == "qwen":
        if weights:
            with st.WeightReader(weights) as r:
                cfg = QwenConfig.from_json(r.config())
        elif preset:
            cfg = QwenConfig.preset(preset)
        else:
            cfg = QwenConfig(vocab=256, block_size=64, n_layers=2, d_model=64, n_heads=4, n_kv_heads=2,
                             head_dim=16, d_ff=128)
        costfn = lambda sh: cost.qwen_cost(cfg, b, t, train, i8, sh)
    else:
        cfg = GptConfig.gradcheck() if not weights else None
        if cfg is None:
            with st.WeightReader(weights) as r:
                cfg = GptConfig.from_json(r.config())
        costfn = lambda sh: cost.gpt_cost(cfg, b, t, train, sh)
    t = min(block or cfg.block_size, cfg.block_size)
    mode = "int8" if i8 else "train" if train else "infer"
    print(f"{model}: layers={cfg.n_layers} d_model={cfg.d_model} b={b} t={t} mode={mode}" +
          (f" stages={stages}" if stages > 1 else ""))
    for si, sh in enumerate(cost.even_shards(cfg.n_layers, stages)):
        label = f"stage {si} (layers {sh[0]}..{sh[1]})" if stages > 1 else model
        fwd, bwd = costfn(sh)
        print(f"---- {label}: forward (offline) ----\n{fwd}\n")
        if bwd is not None:
            print(f"---- {label}: backward (offline) ----\n{bwd}\n")
        if run:
            _flops_online(model, cfg, b, t, train, fwd, bwd, device, label)


def _flops_online(model, cfg, b, t, train, fwd, bwd, device, label):
    """Execute one pass with kernel timing on and print the measured per-kernel table."""
    import torch
    from ..models import build_from_config
    from ..train import pick_device
    from ..utils import profile
    dev = pick_device(device)
    if dev.type != "cuda":
        print(f"{label}: --run needs a CUDA device (the CPU backend has no kernel counters)\n")
        return
    m = build_from_config(cfg.to_json())
    m.init_weights(3)
    m = m.to(dev, torch.bfloat16)
    x = (torch.arange(b * t, device=dev) % cfg.vocab).reshape(b, t).to(torch.int32)

    def step():
        if train:
            m.loss(x, x.long()).backward()
        else:
            with torch.no_grad():
                m(x)
    print(profile.profile(f"{label}: online counters", step, steps=1, warmup=1))


def _gradcheck(args, device):
    from .. import gradcheck
    a = Args(args)
    which = a.str_or("--model", "gpt")
    dirs = a.int_or("--dirs", 4)
    a.finish()
    names = ("gpt", "qwen", "qwen2", "qwen_lora", "qwen3_weighted", "moe", "qwen_moe") if which == "all" else tuple(which.split(","))
    fails = gradcheck.run_gate(names, n_dirs=dirs)
    return 1 if fails else 0


def _perf(args, device):
    from ..perf.cli import run_perf
    return run_perf(args, device)


def _bench(args, device):
    """``brain bench learn [task…]``: the learnability battery (CPU or GPU); ``brain bench [flags]``:
    the training-throughput benchmark at the repository root (needs a GPU)."""
    if args and args[0] == "learn":
        from .. import learnbench
        from ..train import pick_device
        a = Args(args[1:])
        arch = a.str_or("--arch", "qwen")
        steps = a.int_or("--steps", 400)
        seed = a.int_or("--seed", 0)
        names = []
        while True:
            n = a.positional()
            if n is None:
                break
            names.append(n)
        a.finish()
        if arch not in ("qwen", "gpt"):
            print("--arch: qwen | gpt", file=sys.stderr)
            return 2
        try:
            res = learnbench.run_battery(names, arch, steps, seed, str(pick_device(device)))
        except ValueError as e:
            print(str(e), file=sys.stderr)
            return 2
        return 0 if all(r["passed"] for r in res) else 1
    import runpy
    import torch
    if not torch.cuda.is_available():
        print("brain bench: the throughput benchmark needs a CUDA device; `brain bench learn` runs the "
              "learnability battery on the CPU", file=sys.stderr)
        return 1
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    sys.argv = [os.path.join(root, "bench.py")] + list(args)
    runpy.run_path(sys.argv[0], run_name="__main__")


def _federated(args, device):
    from ..federated.cli import run_federated
    return run_federated(args, device)


def _caps(args, device):
    from ..api.capability import all_manifests
    print(json.dumps([m.to_json() for m in all_manifests()], indent=1))


def _serve(args, device):
    from ..api.run import run_serve
    return run_serve(args, device)


def _import_file(rest, device):
    """``brain import <FILE|DIR>``: a Hugging Face directory (or one safetensors file inside one)."""
    from .qwen_cli import run_qwen
    a = Args(rest)
    if a.take_flag("--list"):
        for arch in archs.all_archs():
            print(f"{arch.id:<14} {'importable (Hugging Face safetensors directory)' if arch.id == 'qwen3' else 'no importer in this build'}")
        return 0
    src = a.positional()
    if src is None:
        print("usage: brain import <hf_dir|model.safetensors> [--out F | --id VENDOR/REPO] | brain import --list",
              file=sys.stderr)
        return 2
    d = src if os.path.isdir(src) else os.path.dirname(src) or "."
    return run_qwen(["import", "--hf", d] + a.leftover(), device)


def _quantize(rest, device):
    from ..serve.quantize import quantize_checkpoint
    a = Args(rest)
    src = a.positional()
    out = a.take_str("--out")
    tier = (a.take_str("--tier") or "Q8_0").upper()
    keep = a.take_all("--keep")
    plan_only = a.take_flag("--plan")
    fmt = (a.take_str("--format") or "").lower()
    a.finish()
    if src is None:
        print("usage: brain quantize <SRC.safetensors|.gguf|.pt> [--out F --tier Q8_0|Q4_0 --format gguf|safetensors "
              "--keep SUBSTR... --plan]", file=sys.stderr)
        return 2
    if not fmt:
        fmt = "gguf" if (out or "").lower().endswith(".gguf") or not src.lower().endswith(".safetensors") \
            or tier == "Q4_0" else "safetensors"
    if fmt == "gguf":
        # any container in, GGUF out: block quantisers Q8_0 / Q4_0, every kept tensor with its reason
        from ..checkpoint.convert import quantize_to_gguf
        if tier not in ("Q8_0", "Q4_0"):
            print(f"--tier {tier}: the GGUF writer encodes Q8_0 and Q4_0 (the k-quant tiers are decode-only)", file=sys.stderr)
            return 2
        out = out or os.path.splitext(src)[0] + f".{tier.lower()}.gguf"
        info = quantize_to_gguf(src, out, tier, keep=keep, plan_only=plan_only)
        if plan_only:
            for n, shape, d in info["plan"]:
                print(f"{d:<48}  {n} {list(shape)}")
            return 0
        print(f"ok: wrote {out} ({info['quantized']} {tier} tensors, {info['bytes_in'] / 2**20:.1f} MiB fp32 -> "
              f"{info['bytes_out'] / 2**20:.1f} MiB)")
        return 0
    if tier not in ("Q8_0", "W8", "INT8"):
        print(f"--tier {tier}: the safetensors output is per-row symmetric int8 (Q8_0-class); use --format gguf for Q4_0",
              file=sys.stderr)
        return 2
    if plan_only:
        from ..checkpoint import st as _st
        from ..serve.quantize import _rows, plan as _plan
        with _st.WeightReader(src) as r:
            rows = _rows(r.config())
            sizes = []
            for n in r.names():
                k = 1
                for dim in r.shape(n):
                    k *= dim
                sizes.append((n, k))
        for n, d in _plan(sizes, rows, keep):
            print(f"{d:>5}  {n}")
        return 0
    out = out or src.replace(".safetensors", "") + ".w8.safetensors"
    info = quantize_checkpoint(src, out, keep=keep)
    print(f"ok: wrote {out} ({info['tensors']} int8 tensors, {info['bytes_in'] / 2**20:.1f} MiB -> "
          f"{info['bytes_out'] / 2**20:.1f} MiB)")
