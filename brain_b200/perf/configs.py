"""The benchmark configurations beside the flagship one that ``bench.py`` runs.

    python -m brain_b200.perf.configs cpu-dp      # GPT-2 small, fp32, CPU backend, 2 data-parallel
                                                  # thread workers, 20 steps + the d64 gradcheck gate

Each prints one JSON line.  Synthetic data (uniform-random token ids) and random-init weights."""
from __future__ import annotations

import argparse
import json
import sys
import time

import torch


def cpu_dp(args) -> dict:
    """GPT-2 small (12 layers, d 768, 12 heads, ff 3072, vocab 50257, ctx 1024) fp32 on the CPU
    backend with 2 data-parallel thread workers, per-worker batch 4 x 128, AdamW lr 3e-4 betas
    0.9/0.95 wd 0.1, 20 steps; then the finite-difference gradcheck on a 2-layer d64 variant.  The
    timed oracle is the same model through plain PyTorch autograd ops on one worker."""
    from .. import gradcheck
    from ..data.rng import Rng
    from ..models.config import GptConfig
    from ..models.gpt2 import Gpt2
    from ..parallel.dp import DataParallel
    torch.manual_seed(0)
    # the native GEMM of csrc/cpu is the CPU backend's linear layer in this configuration unless the
    # caller chose (BRAIN_CPU_NATIVE=0 runs the PyTorch ops, the oracle, for comparison)
    import os
    os.environ.setdefault("BRAIN_CPU_NATIVE", "1")
    from ..ops import cpu_native
    cfg = GptConfig(vocab=50257, block_size=1024, n_layers=args.layers, d_model=768, n_heads=12, d_ff=3072)
    workers, B, T = 2, 4, 128

    def make():
        return Gpt2(cfg).init_weights(0)
    t0 = time.perf_counter()
    dp = DataParallel(make, workers, betas=(0.9, 0.95))
    build_s = time.perf_counter() - t0
    rng = Rng(0)
    losses, times = [], []
    mbs = []          # one fixed batch per worker, drawn once with seed 0
    for _ in range(workers):
        toks = torch.from_numpy(rng.tokens(B * (T + 1), cfg.vocab).astype("int64")).view(B, T + 1)
        mbs.append((toks[:, :-1].to(torch.int32).contiguous(), toks[:, 1:].contiguous()))
    opt_times = []
    for step in range(args.steps):
        t1 = time.perf_counter()
        losses.append(dp.forward_backward(mbs))
        t2 = time.perf_counter()
        dp.adamw_step(3e-4, 0.1, 1.0)       # all-reduce over the replicas, clip, AdamW, weights to every replica
        t3 = time.perf_counter()
        times.append(t3 - t1)
        opt_times.append(t3 - t2)
    steady = times[2:] if len(times) > 4 else times
    ms = 1e3 * sum(steady) / len(steady)
    opt_steady = opt_times[2:] if len(opt_times) > 4 else opt_times
    opt_ms = 1e3 * sum(opt_steady) / len(opt_steady)
    report = gradcheck.check_gpt(n_dirs=4, d_model=64)
    fails = report.failures()
    worst = report.worst()
    return {"config": "cpu-dp", "metric": "train tok/s (GPT-2 small fp32, CPU backend, 2 DP thread workers)",
            "value": workers * B * T / (ms / 1e3), "unit": "tokens/s", "ms_per_step": ms,
            "forward_backward_ms": ms - opt_ms, "reduce_and_optimiser_ms": opt_ms, "steps": args.steps,
            "loss_first": losses[0], "loss_last": losses[-1], "loss_decreased": losses[-1] < losses[0],
            "build_s": build_s, "threads": torch.get_num_threads(),
            "linear": "native csrc/cpu GEMM" if cpu_native.enabled() else "PyTorch ops",
            "gradcheck": {"model": "gpt 2-layer d64", "tensors": len(report.entries), "failures": len(fails),
                          "worst_rel": worst.rel if worst else None, "worst_name": worst.name if worst else None},
            "dtype": "fp32", "data": "synthetic"}


def _dist_init():
    import os
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    return rank, world, torch.device("cuda", local)


def _random_qwen(cfg, dev, seed=1234):
    """Random-init model built directly on the device in bf16 (normal std 0.02, gains 1); every
    rank draws the same values from the same seed."""
    from ..models.qwen3 import Qwen3
    prev = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    try:
        with torch.device(dev):
            m = Qwen3(cfg)
    finally:
        torch.set_default_dtype(prev)
    g = torch.Generator(device=dev).manual_seed(seed)
    with torch.no_grad():
        for name, p in m.named_parameters():
            if p.dim() == 1:
                p.fill_(1.0)
            else:
                p.normal_(0.0, 0.02, generator=g)
    return m.eval()


def serve_tp(args) -> dict:
    """Qwen3-8B-architecture serving, tensor parallel over all ranks, W8A8 int8, paged KV with
    16-token blocks, continuous batching: 512 requests at 256 concurrent (closed loop), prompts
    uniform 128..2048 random token ids, 256 greedy output tokens each (stop ignored)."""
    import torch.distributed as dist
    from ..models.config import QwenConfig
    from ..ops import _cuda
    from ..parallel.tp import TensorParallel
    from ..serve.engine import QwenEngine
    from .driver import drive
    from .metrics import Summary
    from .targets import SchedulerTarget
    from .workload import Arrival, standard
    rank, world, dev = _dist_init()
    import faulthandler
    tp = TensorParallel(impl=args.impl, device=dev, arena_mb=1024, wait_seconds=5.0) if world > 1 else None
    cfg = QwenConfig.preset(args.model, 4096)
    if args.layers:
        cfg.n_layers = args.layers
    ctx = 2048 + args.out_tokens + 16
    conc, nreq = args.concurrency, args.requests
    t0 = time.perf_counter()
    model = _random_qwen(cfg, dev)
    per_seq = -(-ctx // 16)
    eng = QwenEngine(model, block_size=16, num_blocks=per_seq * conc + conc, max_seq_len=per_seq * 16,
                     max_prefill=2048, weights=args.weights, tp=tp, cuda_graphs=not args.no_graphs)
    del model
    torch.cuda.empty_cache()
    build_s = time.perf_counter() - t0
    wl = standard("serving_mix", Arrival.closed_loop(conc), nreq, seed=0, vocab=cfg.vocab)
    wl.classes[0].output.n = args.out_tokens
    # warm-up: a few short requests so graphs for small buckets and all lazy setup exist
    warm = standard("serving_mix", Arrival.closed_loop(min(conc, 8)), 8, seed=1, vocab=cfg.vocab)
    warm.classes[0].output.n = 8
    target = SchedulerTarget(None, max_batch=conc, ctx=per_seq * 16, engine=eng, name=f"qwen3-{args.model}",
                             admit_batch=args.admit_batch, prefill_budget=args.prefill_budget,
                             admit_max_wait=args.admit_wait, mixed=not args.no_mixed,
                             prefix_cache=False)   # random prompts share no prefix
    drive(target, warm)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    launches0 = _cuda.launch_count
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for k in eng.acct:
        eng.acct[k] = type(eng.acct[k])(0)
    run = drive(target, wl)
    ev1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([ev0.elapsed_time(ev1)], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    _cuda.check_error()
    faulthandler.cancel_dump_traceback_later()
    s = Summary.build(run.records, float(ms.item()) / 1e3, wl.classes[0].slo)
    j = s.to_json()
    return {"config": "serve-tp", "metric": f"serve out tok/s + p50 TTFT (Qwen3-{args.model} TP{world} {args.weights})",
            "value": s.output_per_s, "unit": "output tokens/s", "n_gpus": world, "ttft_ms_p50": j["ttfa_ms"].get("p50"),
            "ttft_ms_p99": j["ttfa_ms"].get("p99"), "tpot_ms_p50": j["tpoa_ms"].get("p50"),
            "e2e_ms_p50": j["e2e_ms"].get("p50"), "requests": s.requests, "completed": s.completed,
            "input_tokens": s.input_artifacts, "output_tokens": s.output_artifacts, "wall_s": s.wall_s,
            "nvls_all_reduce": bool(tp is not None and getattr(tp, "nvls", False)), "concurrency": conc, "admit_batch": args.admit_batch, "admit_wait": args.admit_wait, "mixed": not args.no_mixed, "prefill_budget": args.prefill_budget, "weights": args.weights, "impl": args.impl, "layers": cfg.n_layers,
            "kv_pool_gb": eng.kv_pool_bytes() / 2**30, "weight_gb_per_rank": eng.weight_bytes() / 2**30,
            "cuda_graph_replays": eng.graph_replays, "engine_steps": eng.steps, "build_s": build_s,
            "engine_time": {k: (round(v, 3) if isinstance(v, float) else v) for k, v in eng.acct.items()},
            "gpu_launches": _cuda.launch_count - launches0, "dtype": "int8 weights+activations, bf16 KV" if args.weights == "int8" else "bf16",
            "data": "synthetic", "timing": "CUDA events around the whole run, max over ranks"}


def _timed_steps(step_fn, steps, warmup, dev, world):
    import torch.distributed as dist
    for _ in range(warmup):
        step_fn()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    loss = None
    for _ in range(steps):
        loss = step_fn()
    ev1.record()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ms = torch.tensor([ev0.elapsed_time(ev1)], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return float(ms.item()) / steps, loss


def train_3d(args) -> dict:
    """Qwen3-14B architecture, bf16, tensor parallel x pipeline parallel (default TP4 x PP2 on 8
    GPUs), 1F1B over 16 micro-batches of 1 x 4096 uniform-random tokens; fused all-gather->GEMM and
    GEMM->reduce-scatter inside every block, pipeline send/recv on NCCL p2p."""
    from ..models.config import QwenConfig
    from ..ops import _cuda
    from ..parallel.grid import Grid
    from ..parallel.trainer3d import Trainer3D
    rank, world, dev = _dist_init()
    tp = args.tp or (4 if world >= 8 else max(world // 2, 1))
    pp = world // tp
    cfg = QwenConfig.preset(args.model, args.seq)
    if args.layers:
        cfg.n_layers = args.layers
    tr = Trainer3D(cfg, Grid(tp=tp, pp=pp, dp=1), dev, impl=args.impl, schedule=args.schedule, seed=1234,
                   recompute=args.recompute)
    gd = torch.Generator(device=dev).manual_seed(0)     # same seed on every rank: same batches
    n_micro, T = args.micro, args.seq
    count = n_micro * T

    def step():
        # fresh uniform-random tokens every step (drawn on the device, no host traffic)
        toks = [torch.randint(0, cfg.vocab, (1, T), generator=gd, device=dev, dtype=torch.int32) for _ in range(n_micro)]
        tgts = [torch.randint(0, cfg.vocab, (1, T), generator=gd, device=dev) for _ in range(n_micro)]
        return tr.train_step(toks, tgts, 1e-4, count)
    launches0 = _cuda.launch_count
    ms, loss = _timed_steps(step, args.steps, args.warmup, dev, world)
    _cuda.check_error()
    flops = tr.model.flops_per_token(T) if hasattr(tr.model, "flops_per_token") else 0.0
    return {"config": "train-3d", "metric": f"train tok/s (Qwen3-{args.model} bf16 TP{tp}xPP{pp} {args.schedule})",
            "value": count / (ms / 1e3), "unit": "tokens/s", "n_gpus": world, "ms_per_step": ms, "steps": args.steps,
            "warmup": args.warmup, "micro_batches": n_micro, "seq_len": T, "impl": args.impl, "layers": cfg.n_layers,
            "final_loss": float(loss), "params_per_rank_b": tr.store.n_train / 1e9,
            "mem_gb": torch.cuda.max_memory_allocated() / 2**30, "gpu_launches": _cuda.launch_count - launches0,
            "dtype": "bf16", "data": "synthetic", "timing": "CUDA events, max over ranks"}


def train_ep(args) -> dict:
    """Qwen3-30B-A3B-style MoE (48 layers, hidden 2048, 32 Q / 4 KV heads, 128 experts of FFN 768,
    softmax router top-8, aux loss 0.001), bf16, expert parallel over all ranks, 8 sequences of
    4096 uniform-random tokens per GPU; fused peer-memory dispatch/combine + grouped tcgen05 GEMM."""
    from ..models.config import MoeConfig
    from ..models.moe import MoeModel
    from ..ops import _cuda
    from ..parallel.ep import ExpertParallel
    from ..parallel.trainer_ep import TrainerEP
    rank, world, dev = _dist_init()
    cfg = MoeConfig.qwen3_30b_a3b(args.seq)
    if args.layers:
        cfg.n_layers = args.layers
    if args.experts:
        cfg.n_experts = args.experts
    ep = ExpertParallel(impl=args.impl, device=dev, arena_mb=args.arena_mb) if world > 1 else None
    prev = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    try:
        with torch.device(dev):
            model = MoeModel(cfg, ep=ep)
    finally:
        torch.set_default_dtype(prev)
    gen = torch.Generator(device=dev).manual_seed(1234)
    gen_local = torch.Generator(device=dev).manual_seed(99 + rank)
    with torch.no_grad():
        for name, p in model.named_parameters():
            if p.dim() == 1:
                p.fill_(1.0)
            else:
                p.normal_(0.0, 0.02, generator=gen_local if ".moe.w_" in name else gen)
    model.recompute_blocks = not (args.no_recompute or args.recompute_experts)
    model.recompute_experts = args.recompute_experts
    tr = TrainerEP(model, dev, dtype=torch.bfloat16)
    g = torch.Generator().manual_seed(rank)
    B, T = args.seqs_per_gpu, args.seq
    toks = torch.randint(0, cfg.vocab, (B, T), generator=g, dtype=torch.int32).pin_memory()
    tgts = torch.randint(0, cfg.vocab, (B, T), generator=g).pin_memory()
    count = B * T * world
    launches0 = _cuda.launch_count
    ms, loss = _timed_steps(lambda: tr.train_step(toks, tgts, 1e-4, args.micro_batch, count), args.steps, args.warmup,
                            dev, world)
    _cuda.check_error()
    loss_t = loss.detach().float().reshape(1).clone()
    if world > 1:
        import torch.distributed as dist
        dist.all_reduce(loss_t)
    return {"config": "train-ep", "metric": f"train tok/s (Qwen3-MoE {cfg.n_experts} experts top-{cfg.top_k} bf16 EP{world})",
            "value": count / (ms / 1e3), "unit": "tokens/s", "n_gpus": world, "ms_per_step": ms, "steps": args.steps,
            "warmup": args.warmup, "seqs_per_gpu": B, "seq_len": T, "micro_batch": args.micro_batch, "impl": args.impl,
            "layers": cfg.n_layers, "experts": cfg.n_experts, "final_loss": float(loss_t),
            "recompute_blocks": bool(model.recompute_blocks), "recompute_experts": bool(model.recompute_experts), "shared_params_b": tr.shared.n_train / 1e9, "expert_params_per_rank_b": tr.expert.n_train / 1e9,
            "mem_gb": torch.cuda.max_memory_allocated() / 2**30, "gpu_launches": _cuda.launch_count - launches0,
            "dtype": "bf16", "data": "synthetic", "timing": "CUDA events, max over ranks"}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("which", choices=["cpu-dp", "serve-tp", "train-3d", "train-ep"])
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--tp", type=int, default=0)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--micro", type=int, default=16, help="train-3d: micro-batches per step")
    ap.add_argument("--schedule", default="1f1b", choices=["1f1b", "gpipe"])
    ap.add_argument("--seqs-per-gpu", type=int, default=8)
    ap.add_argument("--micro-batch", type=int, default=1, help="train-ep: sequences per forward/backward")
    ap.add_argument("--experts", type=int, default=0)
    ap.add_argument("--arena-mb", type=int, default=4096)
    ap.add_argument("--recompute", action="store_true",
                    help="train-3d: keep block inputs only and re-run the blocks in backward")
    ap.add_argument("--no-recompute", action="store_true", help="train-ep: keep all block activations (more memory)")
    ap.add_argument("--recompute-experts", action="store_true",
                    help="train-ep: re-run only the expert layers in backward (attention keeps its activations)")
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--layers", type=int, default=0, help="override depth (debug; invalidates the number)")
    ap.add_argument("--model", default="8b")
    ap.add_argument("--weights", default="int8", choices=["int8", "bf16"])
    ap.add_argument("--impl", default="fused", choices=["fused", "nccl"])
    ap.add_argument("--requests", type=int, default=512)
    ap.add_argument("--concurrency", type=int, default=256)
    ap.add_argument("--out-tokens", type=int, default=256)
    ap.add_argument("--no-graphs", action="store_true")
    ap.add_argument("--mixed", action="store_true",
                    help="serve-tp: accepted for old command lines; mixed steps are the default")
    ap.add_argument("--no-mixed", action="store_true",
                    help="serve-tp: run a step's prompt chunks and its decode batch as two forwards (the product "
                         "default, as in the resident server, is one forward: +4 % out tok/s at TP=4)")
    ap.add_argument("--admit-batch", type=int, default=1, help="serve-tp: admit new requests in groups of this many")
    ap.add_argument("--admit-wait", type=int, default=64,
                    help="serve-tp: with --admit-batch > 1, admit at the latest after this many scheduler steps")
    ap.add_argument("--prefill-budget", type=int, default=0, help="serve-tp: prompt tokens per scheduler step")
    ap.add_argument("--stuck-after", type=int, default=600, help="seconds before a stuck rank dumps its stack and exits")
    a = ap.parse_args(argv)
    if a.which == "cpu-dp" and not a.layers:
        a.layers = 12
    if a.which in ("train-3d", "train-ep") and a.steps == 20:
        a.steps = 3
    if a.which == "train-3d" and a.model == "8b":
        a.model = "14b"
    if a.which != "cpu-dp":
        import faulthandler
        faulthandler.dump_traceback_later(a.stuck_after, exit=True)   # a stuck rank prints its stack and exits
    out = {"cpu-dp": cpu_dp, "serve-tp": serve_tp, "train-3d": train_3d, "train-ep": train_ep}[a.which](a)
    import os
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
