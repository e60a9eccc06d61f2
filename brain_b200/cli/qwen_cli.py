"""``brain qwen3 <import|infer|serve|export|precompile|train|finetune|toolcall|eval|calib>``
(reference: crates/cli/src/qwen_cli.rs:26-43 verb table; :84-116 import, :158-267 serve,
:269-365 infer, :368-475 train, :477-512 finetune, :562-750 LoRA finetune, :751-832 toolcall,
:833-1003 chat eval, :1004-1100 KV calibration).  ``--dp/--tp`` are additive flags of this
framework (the reference CLI has no multi-GPU training flag)."""
from __future__ import annotations

import json
import os
import shutil
import sys
import time
from typing import List, Optional

from .args import Args, canon_verb

_USAGE = "usage: brain qwen3 <import|infer|serve|export|precompile|train|finetune|toolcall|eval|calib> ..."


def run_qwen(argv: List[str], device: str = "auto") -> int:
    verb = canon_verb(argv[0]) if argv else None
    rest = argv[1:]
    table = {"import": _import, "infer": _infer, "serve": _serve, "export": _export,
             "precompile": _precompile, "train": lambda a, d: _train(a, d, None), "finetune": _finetune,
             "toolcall": _toolcall, "eval": _eval_chat, "calib": _calib}
    fn = table.get(verb)
    if fn is None:
        print(f"{_USAGE}  (got {verb!r})", file=sys.stderr)
        return 2
    return fn(rest, device) or 0


# ------------------------------------------------------------------------------------ helpers
def _load(weights: str, device: str, dtype=None):
    import torch
    from ..checkpoint import st
    from ..train import pick_device
    dev = pick_device(device)
    if dtype is None:
        dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
    model, cfg, card = st.load_model(weights, device=dev, dtype=dtype)
    model.eval()
    return model, cfg, card, dev


def _tok(path: str):
    from ..data.tokenizer import load_tokenizer
    try:
        return load_tokenizer(path)   # tokenizer.json, or a dataset directory (character level)
    except Exception as e:  # noqa: BLE001
        print(f"tokenizer load failed: {e}", file=sys.stderr)
        return None


def _eos(tok) -> Optional[int]:
    try:
        ids = tok.encode("<|im_end|>")
    except ValueError:   # a character-level vocabulary without the marker's characters
        ids = []
    return ids[0] if len(ids) == 1 else tok.eos_id


# ------------------------------------------------------------------------------------ import/export
def _import(args, device):
    from ..checkpoint.hf_import import import_hf
    a = Args(args)
    hf = a.str_or("--hf", "")
    out = a.take_str("--out")
    block = a.opt_int("--block")
    dtype = a.str_or("--dtype", "F32").upper()
    model_id = a.take_str("--id")
    mdir = a.take_str("--models-dir")
    gguf_src = a.take_str("--gguf")
    if not hf and not gguf_src:
        hf = a.positional() or ""
        if hf.lower().endswith(".gguf"):
            gguf_src, hf = hf, ""
        elif hf and os.path.isfile(hf):
            hf = os.path.dirname(hf) or "."
    a.finish()
    if gguf_src:
        # a llama.cpp-style GGUF of a dense Qwen2 / Qwen3 model, any block type this build decodes
        from ..checkpoint.convert import import_gguf_qwen
        dst = out or "qwen.safetensors"
        try:
            cfg = import_gguf_qwen(gguf_src, dst, block, dtype, model_id=model_id)
        except Exception as e:  # noqa: BLE001
            print(f"import failed: {e}", file=sys.stderr)
            return 1
        print(f"ok: wrote {dst} ({cfg.n_layers} layers, d_model {cfg.d_model}, vocab {cfg.vocab})")
        return 0
    if not hf:
        print("usage: brain qwen3 import <hf_dir|model.safetensors|model.gguf> [--out F | --id VENDOR/REPO [--models-dir D]] "
              "[--block T --dtype F32|BF16]", file=sys.stderr)
        return 2
    ref = None
    if model_id:
        from ..modelref import ModelRef, RefError
        try:
            ref = ModelRef.parse(model_id).base()
        except RefError as e:
            print(f"--id: {e}", file=sys.stderr)
            return 2
    tmp_out = out or ("qwen.safetensors" if ref is None else os.path.join(hf, ".brain_import.safetensors"))
    try:
        import_hf(hf, tmp_out, block, dtype, model_id=str(ref) if ref else None)   # dense or Qwen3-MoE by model_type
    except Exception as e:  # noqa: BLE001
        print(f"import failed: {e}", file=sys.stderr)
        return 1
    if ref is not None:
        # place the converted weights (and the tokenizer files next to the source) in the model store
        import shutil
        from ..modelstore import Store
        root = models_dir(mdir)
        if not root:
            print("no models directory resolved (set --models-dir, BRAIN_MODELS_DIR, or HOME)", file=sys.stderr)
            return 1
        tok = os.path.join(hf, "tokenizer.json")
        lm = Store(root).install(ref, tmp_out, tok if os.path.exists(tok) else None)
        for extra in ("tokenizer_config.json", "chat_template.jinja"):
            if os.path.exists(os.path.join(hf, extra)):
                shutil.copyfile(os.path.join(hf, extra), os.path.join(lm.dir, extra))
        if out is None:
            os.remove(tmp_out)
        print(f"ok: installed {ref} -> {lm.weights}")
    else:
        print(f"ok: wrote {tmp_out}")


def _export(args, device):
    from ..checkpoint.hf_import import export_hf
    a = Args(args)
    weights = a.str_or("--weights", "")
    out = a.str_or("--out", "qwen-hf")
    dtype = a.str_or("--dtype", "BF16").upper()
    tier = a.take_str("--tier")
    a.finish()
    if weights and out.lower().endswith(".gguf"):
        from ..checkpoint.convert import export_gguf
        info = export_gguf(weights, out, tier.upper() if tier else None)
        print(f"ok: wrote {out} ({info['bytes_out'] / 2**20:.1f} MiB, {info.get('quantized', 0)} quantised tensors)")
        return 0
    if not weights:
        print("usage: brain qwen3 export --weights F --out DIR [--dtype BF16|F32]", file=sys.stderr)
        return 2
    try:
        export_hf(weights, out, dtype)
    except Exception as e:  # noqa: BLE001
        print(f"export failed: {e}", file=sys.stderr)
        return 1
    print(f"ok: wrote {out}/model.safetensors + config.json")


def _precompile(args, device):
    """Build the native libraries ahead of time and, on a GPU box, run one tiny forward so tensor
    maps and the CUDA context are warm (the reference's verb compiles its NPU graph cache)."""
    from .. import _build
    a = Args(args)
    a.take_str("--weights"); a.take_str("--seq"); a.take_str("--npu-cache"); a.take_flag("--allow-fallback")
    a.finish()
    t0 = time.time()
    _build.build_all()
    print(f"precompiled native libraries in {time.time() - t0:.1f}s -> {_build.LIBDIR}")


# ------------------------------------------------------------------------------------ serve / infer
def _serve(args, device):
    from ..serve.offline import serve_prompts
    a = Args(args)
    weights = a.str_or("--weights", "")
    tokenizer = a.str_or("--tokenizer", "")
    prompts = a.take_all("--prompt")
    max_new = a.int_or("--max-new", 64)
    block_size = a.int_or("--block-size", 16)
    kv_int8 = a.take_flag("--int8")
    if a.take_flag("--kv-fp32"):
        kv_int8 = False
    weights_int8 = a.take_flag("--weights-int8")
    kv_calib = a.take_flag("--kv-calib")
    tp_n = a.int_or("--tp", 1)
    a.finish()
    if not weights or not tokenizer or not prompts:
        print('usage: brain qwen3 serve --weights F --tokenizer T --prompt "..." [--prompt "..."]... '
              "[--max-new N --block-size B --weights-int8 --int8 | --kv-fp32  --kv-calib  --tp N]", file=sys.stderr)
        return 2
    tok = _tok(tokenizer)
    if tok is None:
        return 1
    if tp_n > 1:
        return _relaunch(tp_n, ["qwen3", "serve"] + args)
    tp = _tp_from_env(device)
    model, cfg, _, dev = _load(weights, device)
    chatml = hasattr(tok, "apply_chat_template")
    toks = [tok.encode(tok.apply_chat_template([("user", p)], True) if chatml else p) for p in prompts]
    mode = "int8" if weights_int8 and dev.type == "cuda" else "bf16"
    clip = None
    if kv_int8 and kv_calib:
        from ..serve.calib import load_kv_clip
        clip = load_kv_clip(weights)
        if clip is None:
            print("note: --kv-calib given but no kv_calib.json beside the weights; using uncapped row scales",
                  file=sys.stderr)
    r = serve_prompts(model, toks, max_new, block_size, mode, _eos(tok), tp=tp,
                      kv_dtype="int8" if kv_int8 else "bf16", kv_clip=clip)
    if tp is None or tp.rank == 0:
        for i, out in enumerate(r["outputs"]):
            print(f"=== prompt {i}: {prompts[i]!r}")
            print(tok.decode(out) + "\n")
        kv = "int8 KV" if kv_int8 else ("bf16 KV" if dev.type == "cuda" else "fp32 KV")
        print(f"served {len(prompts)} prompts, {r['tokens']} tokens in {r['secs']:.2f}s "
              f"({r['tok_s']:.1f} tok/s aggregate) [{kv}]" + (" [int8 weights]" if mode == "int8" else ""),
              file=sys.stderr)


def _tp_from_env(device):
    """Inside a multi-process launch (WORLD_SIZE > 1) every rank builds the tensor-parallel group."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world <= 1:
        return None
    import torch
    import torch.distributed as dist
    from ..parallel.tp import TensorParallel
    cuda = torch.cuda.is_available() and device != "cpu"
    if cuda:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    if not dist.is_initialized():
        dist.init_process_group("nccl" if cuda else "gloo")
    return TensorParallel(impl="fused" if cuda else "nccl")


def _relaunch(n: int, argv: List[str]) -> int:
    """Re-run this command as ``n`` ranks on one node (one process per GPU)."""
    import subprocess
    argv = [a for i, a in enumerate(argv) if a not in ("--tp", "--dp") and (i == 0 or argv[i - 1] not in ("--tp", "--dp"))]
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", os.environ.get("MASTER_PORT", "29531"),
           "-m", "brain_b200.cli"] + argv
    return subprocess.call(cmd)


def _infer(args, device):
    from ..serve.offline import serve_prompts
    from ..serve.sampling import SampleParams
    a = Args(args)
    weights = a.str_or("--weights", "")
    tokenizer = a.str_or("--tokenizer", "")
    prompt = a.str_or("--prompt", "")
    max_new = a.int_or("--max-new", 32)
    temp = a.float_or("--temp", 0.0)
    top_k = a.int_or("--top-k", 0)
    seed = a.int_or("--seed", 0)
    chat = a.take_flag("--chat")
    spec_k = a.int_or("--spec", 0)
    for f in ("--npu-cache", "--seq"):
        a.take_str(f)
    a.take_flag("--allow-fallback")
    a.finish()
    if not weights or not tokenizer:
        print('usage: brain qwen3 infer --weights F --tokenizer tokenizer.json --prompt "..." '
              "[--max-new N --temp X --top-k K --chat --spec K]", file=sys.stderr)
        return 2
    tok = _tok(tokenizer)
    if tok is None:
        return 1
    text = tok.apply_chat_template([("user", prompt)], True) if chat and hasattr(tok, "apply_chat_template") else prompt
    ids = tok.encode(text)
    if not ids:
        print("empty prompt", file=sys.stderr)
        return 1
    t0 = time.time()
    model, _, _, _ = _load(weights, device)
    load_ms = (time.time() - t0) * 1e3
    t1 = time.time()
    if spec_k > 0 and temp == 0.0:
        # greedy speculative decoding with a prompt-lookup draft: same text, fewer target forwards
        from ..serve.engine import QwenEngine
        from ..serve.spec import ngram_draft, spec_decode
        ctx = -(-(len(ids) + max_new + 8) // 16) * 16
        eng = QwenEngine(model, block_size=16, num_blocks=ctx // 16 + 1, max_seq_len=ctx,
                         max_prefill=max(len(ids), 1), cuda_graphs=False)
        gen, fwd = spec_decode(eng, ids, max_new, spec_k, ngram_draft(3))
        eos = _eos(tok)
        if eos is not None and eos in gen:
            gen = gen[:gen.index(eos)]
        print(f"qwen-spec k={spec_k} target_forwards={fwd} tokens={len(gen)}", file=sys.stderr)
    else:
        r = serve_prompts(model, [ids], max_new, 16, "bf16", _eos(tok), SampleParams(temp, top_k, 1.0), seed)
        gen = r["outputs"][0]
    print(f"qwen-timing load_ms={load_ms:.1f} gen_ms={(time.time() - t1) * 1e3:.1f} tokens={len(gen)}",
          file=sys.stderr)
    print(prompt + tok.decode(gen))


# ------------------------------------------------------------------------------------ train / finetune
def _train(args, device, base: Optional[str]):
    from ..models.config import QwenConfig
    from ..models.qwen3 import Qwen3
    from ..train import FitOpts, fit
    a = Args(args)
    data_dir = a.positional()
    out = a.str_or("--out", "out/qwen.safetensors")
    steps = a.int_or("--steps", 2000)
    batch = a.int_or("--batch", 8)
    block = a.int_or("--block", 256)
    lr = a.float_or("--lr", 1e-5 if base else 3e-4)
    seed = a.int_or("--seed", 1234)
    mask = a.char_opt("--mask")
    align = a.take_flag("--align")
    save_secs = a.int_or("--save-secs", 600)
    dp_n = a.int_or("--dp", 1)
    preset = a.take_str("--preset")
    weighted = a.take_flag("--weighted")
    recompute = a.take_flag("--recompute")
    a.finish()
    if data_dir is None:
        print("usage: brain qwen3 {train|finetune} <data_dir> --out F [--steps N --batch B --block T --lr X "
              "--mask = --align --dp N --preset 0.6b --weighted --recompute]", file=sys.stderr)
        return 2
    if dp_n > 1:
        return _relaunch(dp_n, ["qwen3", "finetune" if base else "train"] + args +
                         (["--weights", base] if base else []))
    o = FitOpts(steps=steps, batch_size=batch, block_size=block, lr=lr, warmup=50, decay_iters=steps,
                min_lr=lr * 0.1, weight_decay=0.1, grad_clip=1.0, grad_accum=1,
                eval_interval=max(steps // 10, 1), eval_batches=20, checkpoint_secs=save_secs,
                mask_before=mask, mask_per_line=mask is not None, align_to_lines=align, seed=seed,
                device=device, weighted=weighted)
    if weighted and not os.path.exists(os.path.join(data_dir, "train.weight.bin")):
        print(f"--weighted: {data_dir}/train.weight.bin not found", file=sys.stderr)
        return 1

    def build(vocab, blk):
        m = _build(vocab, blk)
        m.recompute_blocks = recompute      # keep block inputs only; re-run the blocks in backward
        return m

    def _build(vocab, blk):
        if preset:
            c = QwenConfig.preset(preset, blk)
            c.vocab = vocab
            return Qwen3(c)
        return Qwen3(QwenConfig(vocab=vocab, block_size=blk, n_layers=6, d_model=384, n_heads=6, n_kv_heads=2,
                                head_dim=64, d_ff=1024, rope_theta=1.0e6, rms_eps=1e-6,
                                max_position_embeddings=blk, tie_embeddings=True))
    os.makedirs(os.path.dirname(out) or ".", exist_ok=True)
    prev = os.environ.get("BRAIN_OFFLOAD_ADAM")
    if base:
        if not os.path.exists(out):
            shutil.copyfile(base, out)       # fit() resumes from `out`: the base seeds the run
        os.environ["BRAIN_OFFLOAD_ADAM"] = "1"
    dp = _dp_from_env(device)
    try:
        l0, l1 = fit(data_dir, build, o, out, dp=dp,
                     log=print if dp is None or dp.rank == 0 else (lambda s: None))
    except Exception as e:  # noqa: BLE001
        print(f"train error: {e}", file=sys.stderr)
        return 1
    finally:
        if base:
            if prev is None:
                os.environ.pop("BRAIN_OFFLOAD_ADAM", None)
            else:
                os.environ["BRAIN_OFFLOAD_ADAM"] = prev
    if dp is None or dp.rank == 0:
        print(f"trained: loss {l0:.4f} -> {l1:.4f}; saved {out}")


def _dp_from_env(device):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world <= 1:
        return None
    import torch
    import torch.distributed as dist
    from ..parallel.zero import ZeroDP
    cuda = torch.cuda.is_available() and device != "cpu"
    if cuda:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    if not dist.is_initialized():
        dist.init_process_group("nccl" if cuda else "gloo")
    return ZeroDP(impl="fused" if cuda else "nccl")


def _finetune(args, device):
    if "--lora" in args:
        return _finetune_lora(args, device)
    a = Args(args)
    base = a.take_str("--weights")
    if not base:
        print("usage: brain qwen3 finetune <data_dir> --weights BASE --out F [...]", file=sys.stderr)
        return 2
    return _train(a.leftover(), device, base)


def parse_adapter_spec(spec: str):
    """``OWNER/NAME[:TAG]`` -> (owner, name, tag); tag defaults to ``latest``."""
    body, _, tag = spec.partition(":")
    owner, sep, name = body.partition("/")
    ok = lambda s: bool(s) and all(c.isalnum() or c in "-_." for c in s)
    if not sep or not ok(owner) or not ok(name) or (tag and not ok(tag)):
        raise ValueError("expected OWNER/NAME[:TAG] with [A-Za-z0-9-_.] components")
    return owner, name, tag or "latest"


def models_dir(flag: Optional[str] = None) -> Optional[str]:
    from ..modelstore import default_root
    return default_root(flag)


def adapter_path(root: str, base_id: str, owner: str, name: str, tag: str) -> str:
    """``<root>/<vendor>/<repo>/adapters/<owner>/<name>/<tag>/adapter.brain.safetensors``."""
    from ..modelref import ModelRef
    from ..modelstore import Store
    ref = ModelRef.parse(base_id if "/" in base_id else f"local/{base_id}").base()
    return Store(root).adapter_weights_path(ref.with_adapter(owner, name, tag))


def _finetune_lora(args, device):
    from ..checkpoint import st
    from ..models.config import LoraCfg
    from ..models.lora import attach_lora, save_adapter
    from ..train import FitOpts, fit, pick_device
    a = Args(args)
    base = a.str_or("--weights", "")
    spec = a.str_or("--adapter", "")
    dataset = a.str_or("--dataset", "") or (a.positional() or "")
    rank = a.int_or("--lora", 0)
    alpha = a.float_or("--alpha", 0.0)
    steps = a.int_or("--steps", 500)
    lr = a.float_or("--lr", 5e-5)
    batch = a.int_or("--batch", 4)
    block = a.int_or("--block", 1024)
    seed = a.int_or("--seed", 1234)
    mdir = a.take_str("--models-dir")
    dataset_id = a.take_str("--dataset-id")
    targets = a.str_or("--targets", "wq,wk,wv,wo")
    a.finish()
    if not base or not spec or not dataset:
        print("usage: brain qwen3 finetune --lora RANK --weights BASE --adapter OWNER/NAME[:TAG] --dataset DIR "
              "[--alpha A --steps N --lr X --batch B --block T --seed S --models-dir DIR --dataset-id ID]",
              file=sys.stderr)
        return 2
    if rank <= 0:
        print("--lora RANK must be > 0", file=sys.stderr)
        return 2
    alpha = alpha or 2.0 * rank
    try:
        owner, name, tag = parse_adapter_spec(spec)
    except ValueError as e:
        print(f"--adapter {spec!r}: {e}", file=sys.stderr)
        return 2
    root = models_dir(mdir)
    if root is None:
        print("no models directory resolved (set --models-dir, BRAIN_MODELS_DIR, or HOME)", file=sys.stderr)
        return 1
    model, cfg, card = st.load_model(base)
    base_id = card.id if card is not None else "brain/qwen3"
    out = adapter_path(root, base_id, owner, name, tag)
    os.makedirs(os.path.dirname(out), exist_ok=True)
    block = min(block, model.cfg.block_size)
    attach_lora(model, LoraCfg(rank=rank, alpha=alpha, targets=tuple(targets.split(","))), seed)
    o = FitOpts(steps=steps, batch_size=batch, block_size=block, lr=lr, warmup=min(20, steps), decay_iters=steps,
                min_lr=lr * 0.1, weight_decay=0.0, grad_clip=1.0, eval_interval=max(steps // 10, 1),
                eval_batches=8, checkpoint_secs=0, seed=seed, device=device)
    adapter_id = f"{base_id}:{owner}:{name}:{tag}"
    try:
        l0, l1 = fit(dataset, None, o, out, model=model,
                     save=lambda p, m: save_adapter(p, m, base_id, dataset_id, adapter_id))
    except Exception as e:  # noqa: BLE001
        print(f"finetune error: {e}", file=sys.stderr)
        return 1
    print(f"trained adapter {adapter_id}: loss {l0:.4f} -> {l1:.4f}; saved {out}")


# ------------------------------------------------------------------------------------ toolcall / eval / calib
def _toolcall(args, device):
    sub = args[0] if args else None
    if sub == "gen":
        return _toolcall_gen(args[1:])
    if sub == "eval":
        return _toolcall_eval(args[1:], device)
    print(f"usage: brain qwen3 toolcall <gen|eval> ...  (got {sub!r})", file=sys.stderr)
    return 2


def _toolcall_gen(args):
    from ..data import chat, toolcall
    a = Args(args)
    out = a.str_or("--out", "data/toolcall")
    tokenizer = a.str_or("--tokenizer", "")
    n, held = a.int_or("--n", 400), a.int_or("--held", 40)
    tools, vocab, seed = a.int_or("--tools", 3), a.int_or("--vocab", 151936), a.int_or("--seed", 1)
    a.finish()
    if not tokenizer:
        print("usage: brain qwen3 toolcall gen --tokenizer tokenizer.json --out DIR [--n --held --tools --vocab --seed]",
              file=sys.stderr)
        return 2
    tok = _tok(tokenizer)
    if tok is None:
        return 1
    train = [c.to_chat_example() for c in toolcall.generate(n, tools, seed)]
    val = [c.to_chat_example() for c in toolcall.generate(held, tools, seed ^ 0xDEAD)]
    chat.prepare_chat(train, val, tok, max(vocab, tok.vocab_size), out)
    print(f"ok: wrote {n} train + {held} val tool-call examples -> {out}")


def _generate_text(model, tok, prompt_ids, max_new, eos):
    from ..serve.offline import serve_prompts
    r = serve_prompts(model, [prompt_ids], max_new, 16, "bf16", eos)
    return r["outputs"][0]


def _toolcall_eval(args, device):
    from ..data import toolcall
    a = Args(args)
    weights, tokenizer = a.str_or("--weights", ""), a.str_or("--tokenizer", "")
    n, tools, seq, seed = a.int_or("--n", 40), a.int_or("--tools", 3), a.int_or("--seq", 512), a.int_or("--seed", 999)
    a.finish()
    if not weights or not tokenizer:
        print("usage: brain qwen3 toolcall eval --weights F --tokenizer T [--n --tools --seq --seed]", file=sys.stderr)
        return 2
    tok = _tok(tokenizer)
    if tok is None:
        return 1
    model, _, _, _ = _load(weights, device)
    exact = tok_hits = tok_total = 0
    for case in toolcall.generate(n, tools, seed):
        ex = case.to_chat_example()
        ids = tok.encode(tok.apply_chat_template(ex.messages(), True))[-(seq - 64):]
        want = tok.encode(case.response_str())
        got = _generate_text(model, tok, ids, len(want) + 8, _eos(tok))
        exact += int(toolcall.calls_match(case.name, case.arguments, toolcall.first_tool_call(tok.decode(got))))
        tok_hits += sum(int(x == y) for x, y in zip(want, got))
        tok_total += len(want)
    print(f"tool-call eval: exact-match {100.0 * exact / max(n, 1):.1f}%  token-acc "
          f"{100.0 * tok_hits / max(tok_total, 1):.1f}%  ({n} held-out cases)")


def _eval_chat(args, device):
    """Masked next-token loss / perplexity of the assistant turns of a chat JSONL file, optionally
    with a LoRA adapter folded in."""
    import math
    import torch
    from ..checkpoint import st
    from ..data import chat
    from ..models.lora import fold_adapter_into
    a = Args(args)
    base, jsonl = a.str_or("--weights", ""), a.str_or("--jsonl", "")
    tokenizer = a.str_or("--tokenizer", "")
    adapter = a.take_str("--adapter")
    block = a.int_or("--block", 1024)
    mdir = a.take_str("--models-dir")
    a.take_str("--kv")
    a.finish()
    if not base or not jsonl:
        print("usage: brain qwen3 eval --weights BASE --jsonl FILE [--tokenizer T --adapter OWNER/NAME[:TAG] "
              "--block T --models-dir DIR]", file=sys.stderr)
        return 2
    tokenizer = tokenizer or os.path.join(os.path.dirname(base) or ".", "tokenizer.json")
    tok = _tok(tokenizer)
    if tok is None:
        return 1
    model, _, card, dev = _load(base, device)
    if adapter:
        owner, name, tag = parse_adapter_spec(adapter)
        p = adapter if os.path.exists(adapter) else adapter_path(models_dir(mdir) or ".", card.id if card else "brain/qwen3", owner, name, tag)
        tensors, acfg, _ = st.load(p)
        n = fold_adapter_into(model, {k: v.to(dev) for k, v in tensors.items()}, int(acfg["rank"]), float(acfg["alpha"]))
        print(f"folded adapter {adapter} ({n} projections)")
    exs = chat.examples_from_records(chat.load_jsonl(jsonl))
    tot, cnt = 0.0, 0
    with torch.no_grad():
        for ex in exs:
            ids, mask = ex.encode(tok)
            ids, mask = ids[:block + 1], mask[:block + 1]
            x = torch.tensor([ids[:-1]], dtype=torch.int32, device=dev)
            y = torch.tensor([[t if m else -1 for t, m in zip(ids[1:], mask[1:])]], dtype=torch.int64, device=dev)
            k = int((y >= 0).sum())
            if k == 0:
                continue
            tot += float(model.loss(x, y)) * k
            cnt += k
    loss = tot / max(cnt, 1)
    print(f"chat eval: {len(exs)} examples, {cnt} supervised tokens, loss {loss:.4f}, perplexity {math.exp(min(loss, 50)):.3f}")


def _calib(args, device):
    """Per-layer, per-KV-head absolute-max / percentile statistics of K and V over a chat JSONL
    file: the scales a quantised KV cache would clip to."""
    import torch
    from ..data import chat
    from ..serve.calib import collect_kv_stats
    a = Args(args)
    weights, jsonl = a.str_or("--weights", ""), a.str_or("--jsonl", "")
    tokenizer = a.str_or("--tokenizer", "")
    out, clip_out = a.take_str("--out"), a.take_str("--clip-out")
    pct = a.float_or("--percentile", 0.999)
    report = a.take_flag("--report")
    a.take_str("--models-dir")
    a.finish()
    if not weights or not jsonl:
        print("usage: brain qwen3 calib --weights BASE --jsonl FILE [--report] [--out kv_calib_report.json] "
              "[--clip-out kv_calib.json --percentile Q]", file=sys.stderr)
        return 2
    if not report and out is None and clip_out is None:
        clip_out = os.path.join(os.path.dirname(weights) or ".", "kv_calib.json")
    tok = _tok(tokenizer or os.path.join(os.path.dirname(weights) or ".", "tokenizer.json"))
    if tok is None:
        return 1
    model, _, _, dev = _load(weights, device)
    exs = chat.examples_from_records(chat.load_jsonl(jsonl))
    seqs = [ex.encode(tok)[0][:model.cfg.block_size] for ex in exs]
    stats = collect_kv_stats(model, seqs, pct)
    if report or out:
        body = json.dumps(stats, indent=1)
        if out:
            open(out, "w").write(body)
            print(f"ok: wrote {out}")
        else:
            print(body)
    if clip_out:
        open(clip_out, "w").write(json.dumps({"percentile": pct, "k": stats["k_clip"], "v": stats["v_clip"]}))
        print(f"ok: wrote {clip_out}")
