"""``brain perf {list,run,compare,gate}`` (reference: crates/cli/src/perf_cli.rs — workloads and
targets by name, one JSON row per run, compare/gate between saved rows)."""
from __future__ import annotations

import json
import sys
import time
from typing import List

from ..cli.args import Args
from . import fidelity, gate
from .driver import drive
from .metrics import Summary
from .targets import FakeTarget, HttpTarget, SchedulerTarget, synth_qwen
from .workload import Arrival, standard, standard_names


def _arrival(a: Args) -> Arrival:
    rate = a.float_or("--rate", 0.0)
    if a.take_flag("--saturated"):
        return Arrival.saturated()
    if rate > 0:
        return Arrival.rate(rate, a.float_or("--burstiness", 1.0))
    return Arrival.closed_loop(a.int_or("--concurrency", 8))


def _make_target(spec: str, device: str, a_conc: int, ctx: int, weights: str, **sched_kw):
    """(factory of fresh targets, vocabulary size); ``sched_kw`` reaches the in-process scheduler
    targets (prefix_cache=, policy=, policy_arg=, ...)."""
    if spec == "fake":
        return (lambda: FakeTarget(max(a_conc, 1), 2)), 32000
    if spec.startswith("qwen-synth:"):
        from ..train import pick_device
        dev = pick_device(device)
        model = synth_qwen(spec.split(":", 1)[1], dev)
        return (lambda: SchedulerTarget(model, max_batch=max(a_conc, 1), ctx=ctx, weights=weights, name=spec,
                                        **sched_kw)), model.cfg.vocab
    if spec.startswith("qwen:"):
        spec = "weights:" + spec[5:]
    if spec.startswith("weights:"):
        import torch
        from ..checkpoint import st
        from ..train import pick_device
        dev = pick_device(device)
        model, _, _ = st.load_model(spec.split(":", 1)[1], device=dev,
                                    dtype=torch.bfloat16 if dev.type == "cuda" else torch.float32)
        model.eval()
        return (lambda: SchedulerTarget(model, max_batch=max(a_conc, 1), ctx=ctx, weights=weights, name=spec,
                                        **sched_kw)), model.cfg.vocab
    if spec.startswith("http:"):
        # http:<base_url>|<api_key>|<model>
        base, key, model = spec[5:].split("|")
        return (lambda: HttpTarget(base, key, model)), 32000
    raise ValueError(f"unknown target {spec!r}: fake | qwen-synth:LxDxH[xV] | weights:FILE | http:URL|KEY|MODEL")


def run_perf(argv: List[str], device: str = "auto") -> int:
    sub = argv[0] if argv else None
    if sub == "list":
        print("workloads: " + " ".join(standard_names()))
        print("targets:   fake | qwen-synth:LxDxH[xV] | weights:FILE | http:URL|KEY|MODEL")
        print("arrivals:  --concurrency N (closed loop) | --saturated | --rate R [--burstiness K]")
        print("tools:     brain perf tool {kernels|launches|comm|serve-micro|mixed-ab|configs|fa-timeline|mma-probe} [args]")
        return 0
    if sub == "tool":
        # measurement tools that are not workloads: each is a module with its own argument parser
        tools = {"kernels": "kernel_bench", "launches": "launch_list", "comm": "comm_bench",
                 "serve-micro": "serve_micro", "mixed-ab": "mixed_ab", "configs": "configs",
                 "fa-timeline": "fa_timeline", "mma-probe": "mma_probe"}
        name = argv[1] if len(argv) > 1 else None
        if name not in tools:
            print("tools: " + " ".join(sorted(tools)), file=sys.stderr)
            return 2
        import importlib
        mod = importlib.import_module(f"brain_b200.perf.{tools[name]}")
        return int(mod.main(argv[2:]) or 0)
    if sub == "run" and len(argv) > 1 and argv[1] in ("latency", "throughput", "serve", "sweep", "startup", "mixed",
                                                      "overload", "cancel", "kvcache", "soak", "faults",
                                                      "residency", "placement", "frontend"):
        return run_perf(["scenario"] + argv[1:], device)     # `perf run <scenario>` as the reference spells it
    if sub == "run":
        a = Args(argv[1:])
        name = a.positional() or "interactive"
        target = a.str_or("--target", "fake")
        n = a.int_or("--requests", 32)
        seed = a.int_or("--seed", 0)
        ctx = a.int_or("--ctx", 4096)
        weights = a.str_or("--weights-dtype", "bf16")
        out = a.take_str("--out")
        skip_fid = a.take_flag("--no-fidelity")
        mixed = a.take_flag("--mixed")      # prompt chunks and the decode batch of a step in one forward
        arrival = _arrival(a)
        a.finish()
        wl = standard(name, arrival, n, seed)
        if wl is None:
            print(f"unknown workload {name!r}; have: {' '.join(standard_names())}", file=sys.stderr)
            return 2
        try:
            make, vocab = _make_target(target, device, arrival.concurrency if arrival.kind == "closed_loop" else 256, ctx, weights,
                                       **({"mixed": True} if mixed and target != "fake" else {}))
            wl.vocab = vocab
        except ValueError as e:
            print(str(e), file=sys.stderr)
            return 2
        fid = None
        if not skip_fid and not target.startswith("http:"):
            fid = fidelity.serial_vs_concurrent(make, wl, n=min(4, n))
            if not fid.passed:
                print(f"fidelity FAILED: serial and concurrent outputs differ ({fid.matching}/{fid.compared} exact)",
                      file=sys.stderr)
        t = make()
        try:
            run = drive(t, wl)
        finally:
            t.close()
        s = Summary.build(run.records, run.wall_s, wl.classes[0].slo)
        row = {"workload": wl.to_json(), "target": dict(t.info, spec=target), "summary": s.to_json(),
               "fidelity": fid.to_json() if fid else None, "when": time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime())}
        text = json.dumps(row)
        if out:
            open(out, "w").write(text + "\n")
        j = s.to_json()
        print(f"{name} on {target}: {s.completed}/{s.requests} done in {s.wall_s:.2f}s  out {s.output_per_s:.1f}/s  "
              f"goodput {s.goodput_per_s:.1f}/s  TTFA p50 {j['ttfa_ms'].get('p50', 0) or 0:.1f} ms p99 "
              f"{j['ttfa_ms'].get('p99', 0) or 0:.1f} ms  TPOA p50 {j['tpoa_ms'].get('p50', 0) or 0:.2f} ms  "
              f"SLO {100 * s.slo_attainment:.0f}%")
        if not out:
            print(text)
        return 0 if (fid is None or fid.passed) else 1
    if sub in ("compare", "gate"):
        a = Args(argv[1:])
        ca, ba = a.positional(), a.positional()
        floor = 1.0 - a.float_or("--tolerance", 0.1)
        a.finish()
        if not ca or not ba:
            print(f"usage: brain perf {sub} CANDIDATE.json BASELINE.json [--tolerance 0.1]", file=sys.stderr)
            return 2
        c = json.loads(open(ca).read())["summary"]
        b = json.loads(open(ba).read())["summary"]
        checks = gate.compare(c, b, floor)
        print(gate.render(checks, floor))
        return 0 if (sub == "compare" or gate.passed(checks)) else 1
    if sub == "scenario":
        from . import scenarios as sc
        a = Args(argv[1:])
        name = a.positional() or ""
        target = a.str_or("--target", "fake")
        n = a.int_or("--requests", 32)
        seed = a.int_or("--seed", 0)
        ctx = a.int_or("--ctx", 4096)
        conc = a.int_or("--concurrency", 8)
        weights = a.str_or("--weights-dtype", "bf16")
        rate = a.float_or("--rate", 0.0)
        seconds = a.float_or("--seconds", 10.0)
        inp = a.int_or("--input", 0) or None
        out = a.take_str("--out")
        a.finish()
        if name not in sc.TIER1 + sc.TIER2:
            print(f"usage: brain perf scenario <{'|'.join(sc.TIER1 + sc.TIER2)}> [--target T --requests N "
                  "--concurrency C --rate R --seconds S --input L --out F]", file=sys.stderr)
            return 2
        if name == "faults":
            return run_perf(["faults"], device)
        if name in ("residency", "placement", "frontend"):
            # the layers around the engine: residency manager, placer, host-side front end (no target)
            from . import scenarios2 as s2
            res = (s2.residency(requests=max(n, 120), concurrency=conc, seed=seed) if name == "residency"
                   else s2.placement(requests=max(n, 60), seed=seed) if name == "placement"
                   else s2.frontend(requests=max(n, 20), device_rate_per_s=rate or 200.0, seed=seed))
            text = json.dumps(res)
            if out:
                open(out, "w").write(text + "\n")
            else:
                print(text)
            return 0 if res.get("passed", True) else 1
        try:
            mk, vocab = _make_target(target, device, conc, ctx, weights)
            if name == "latency":
                res = sc.latency(mk, n=n, seed=seed, vocab=vocab, input_override=inp)
            elif name == "throughput":
                res = sc.throughput(mk, n=n, seed=seed, vocab=vocab, input_override=inp)
            elif name == "serve":
                if rate <= 0:
                    print("serve needs --rate R (requests per second)", file=sys.stderr)
                    return 2
                res = sc.serve(mk, rate, n=n, seed=seed, vocab=vocab, input_override=inp)
            elif name == "sweep":
                ladder = [c for c in (1, 2, 4, 8, 16, 32, 64, 128, 256) if c <= max(conc, 1)]
                mk_big, _ = _make_target(target, device, ladder[-1], ctx, weights)
                res = sc.sweep(mk_big, ladder, n=n, seed=seed, vocab=vocab, input_override=inp)
            elif name == "startup":
                res = sc.startup(mk, vocab=vocab, seed=seed)
            elif name == "mixed":
                res = sc.mixed(mk, n=n, concurrency=conc, seed=seed, vocab=vocab)
            elif name == "soak":
                res = sc.soak(mk, seconds=seconds, concurrency=conc, seed=seed, vocab=vocab)
            elif name == "cancel":
                mk_nc, _ = _make_target(target, device, conc, ctx, weights, **({} if target == "fake" else {"prefix_cache": False}))
                res = sc.cancel(mk_nc, n=n, seed=seed, vocab=vocab)
            elif name == "kvcache":
                if target == "fake" or target.startswith("http:"):
                    print("kvcache needs an in-process engine target (qwen-synth: or weights:)", file=sys.stderr)
                    return 2
                mk_c, _ = _make_target(target, device, conc, ctx, weights, prefix_cache=True)
                mk_u, _ = _make_target(target, device, conc, ctx, weights, prefix_cache=False)
                res = sc.kvcache(mk_c, mk_u, n=n, seed=seed, vocab=vocab)
            else:   # overload
                if target == "fake" or target.startswith("http:"):
                    print("overload needs an in-process engine target (qwen-synth: or weights:)", file=sys.stderr)
                    return 2
                cap = sc.throughput(mk, n=max(n // 2, 8), seed=seed, vocab=vocab, input_override=inp)
                per_s = max(cap["summary"]["requests_per_s"], 1e-3)
                mk_b, _ = _make_target(target, device, conc, ctx, weights, policy="max_queue_depth",
                                       policy_arg=float(2 * conc))
                res = sc.overload(mk_b, per_s, n=n, seed=seed, vocab=vocab, input_override=inp)
        except ValueError as e:
            print(str(e), file=sys.stderr)
            return 2
        text = json.dumps(res)
        if out:
            open(out, "w").write(text + "\n")
        else:
            print(text)
        return 0 if res.get("passed", True) else 1
    if sub == "faults":
        from . import faults
        names = [n for n in argv[1:] if not n.startswith("-")] or None
        bad = [n for n in (names or []) if n not in faults.SCENARIOS]
        if bad:
            print(f"unknown fault {bad[0]!r}; one of: {' '.join(faults.SCENARIOS)}", file=sys.stderr)
            return 2
        res = faults.run_all(names)
        for r in res:
            print(f"{r.fault:<22} reported {str(r.reported):<5} clean {str(r.clean):<5} survived "
                  f"{str(r.survived):<5} {'PASS' if r.passed else 'FAIL'}  {r.detail}")
        return 0 if all(r.passed for r in res) else 1
    print("usage: brain perf list | run <workload> [--target T --requests N --concurrency C --mixed --out F] | "
          "compare A B | gate A B [--tolerance X] | scenario <name> [...] | faults [NAME…]", file=sys.stderr)
    return 2
