"""Auxiliary tools that run without a GPU: profile table (roof percentages and the impossible-rate
flag), ncu launch-list aggregation, KV calibration and its use by the int8 KV cache, model
evaluation helpers."""
import json
import os

import numpy as np
import pytest
import torch


def test_profile_table_flags_rates_above_the_roof():
    from brain_b200.utils import profile
    from brain_b200.utils.roof import Roof
    roof = Roof(hbm_gbs=6000.0, bf16_tflops=1600.0, bf16_tflops_sustained=1400.0, i8_tops=3000.0, source="test")
    agg = {
        "gemm_bf16": {"n": 4, "ms": 4.0, "flops": 4 * 1.2e12, "int_ops": 0.0, "bytes": 4 * 2e8, "uncosted": 0},
        "rmsnorm_fwd": {"n": 8, "ms": 0.4, "flops": 0.0, "int_ops": 0.0, "bytes": 8 * 2.0e8, "uncosted": 0},
        "bogus": {"n": 1, "ms": 0.001, "flops": 1e13, "int_ops": 0.0, "bytes": 0.0, "uncosted": 0},
    }
    text = profile.render(agg, "unit", roof)
    lines = {l.split()[0]: l for l in text.splitlines() if l and not l.startswith("-")}
    assert "compute" in lines["gemm_bf16"] and "memory" in lines["rmsnorm_fwd"]
    gemm_pct = float(lines["gemm_bf16"].split()[-1])
    assert gemm_pct == pytest.approx(100 * (1.2e12 / 1600e12) / 1e-3, rel=1e-3)      # 75 % of the roof
    assert "above the measured roof" in lines["bogus"] and "above" not in lines["gemm_bf16"]
    assert "roof: HBM 6000 GB/s" in text


def test_launch_list_aggregation(tmp_path):
    from brain_b200.perf import launch_list
    p = tmp_path / "l.csv"
    p.write_text("==PROF== header line\n"
                 '"ID","Process ID","Process Name","Host Name","Kernel Name","Context","Stream","Block Size","Grid Size",'
                 '"Device","CC","Section Name","Metric Name","Metric Unit","Metric Value"\n'
                 '"0","1","python","h","void bb::gemm_kernel<256, 0>(CUtensorMap_st)","1","7","(256, 1, 1)","(148, 1, 1)","0","10.0","Command line profiler metrics","gpu__time_duration.sum","ns","150,000"\n'
                 '"1","1","python","h","void bb::gemm_kernel<256, 0>(CUtensorMap_st)","1","7","(256, 1, 1)","(148, 1, 1)","0","10.0","Command line profiler metrics","gpu__time_duration.sum","ns","50,000"\n'
                 '"2","1","python","h","bb::adamw_kernel(float*)","1","7","(256, 1, 1)","(148, 1, 1)","0","10.0","Command line profiler metrics","gpu__time_duration.sum","us","100"\n')
    agg, total, n = launch_list.aggregate(str(p))
    assert n == 3 and total == pytest.approx(300.0)
    assert agg["void bb::gemm_kernel<256, 0>"] == [2, pytest.approx(200.0)]
    text = launch_list.render(agg, total, n)
    assert text.splitlines()[2].split()[1] == "66.7%" and "adamw_kernel" in text


def test_kv_calibration_feeds_the_int8_cache(tmp_path):
    from brain_b200.models.config import QwenConfig
    from brain_b200.models.qwen3 import Qwen3
    from brain_b200.serve.calib import collect_kv_stats, load_kv_clip
    from brain_b200.serve.engine import QwenEngine
    cfg = QwenConfig(vocab=61, block_size=64, n_layers=2, d_model=32, n_heads=4, n_kv_heads=2, head_dim=8, d_ff=64)
    m = Qwen3(cfg).init_weights(5).eval()
    rng = np.random.RandomState(0)
    seqs = [rng.randint(0, 61, n).tolist() for n in (20, 33, 7)]
    stats = collect_kv_stats(m, seqs, percentile=0.99, block_size=8)
    assert stats["tokens"] == 60 and len(stats["k_clip"]) == 2 and len(stats["k_clip"][0]) == 2
    for li in range(2):
        for h in range(2):
            assert 0 < stats["k_clip"][li][h] <= stats["layers"][li]["k_absmax"][h]
            assert 0 < stats["v_clip"][li][h] <= stats["layers"][li]["v_absmax"][h]
    w = tmp_path / "model" / "w.safetensors"
    w.parent.mkdir()
    w.write_bytes(b"")
    assert load_kv_clip(str(w)) is None
    (w.parent / "kv_calib.json").write_text(json.dumps({"percentile": 0.99, "k": stats["k_clip"], "v": stats["v_clip"]}))
    clip = load_kv_clip(str(w))
    eng = QwenEngine(m, block_size=8, num_blocks=16, max_seq_len=64, max_prefill=64, kv_dtype="int8", kv_clip=clip)
    bt = np.arange(8, dtype=np.int32)
    eng.prefill_chunk(np.asarray(seqs[1], dtype=np.int32), 0, bt, True)
    for li in range(2):        # no stored row scale exceeds its head's ceiling / 127
        for h in range(2):
            assert float(eng.ks[li][:, h].max()) <= stats["k_clip"][li][h] / 127 + 1e-9
            assert float(eng.vs[li][:, h].max()) <= stats["v_clip"][li][h] / 127 + 1e-9


def test_eval_helpers(tmp_path):
    from brain_b200.cli.main import main
    from brain_b200.eval import exact_match, val_perplexity
    d, w = str(tmp_path / "calc"), str(tmp_path / "g.safetensors")
    assert main(["data", "gen", "calculator", "--out", d, "--n", "300", "--seed", "2"]) == 0
    assert main(["gpt2", "train", d, "--out", w, "--steps", "4", "--batch", "4", "--block", "16", "--layers", "1",
                 "--d-model", "16", "--heads", "2", "--mask", "=", "--align", "--device", "cpu"]) == 0
    ppl = val_perplexity(w, d, batches=2)
    assert ppl == ppl and 1.0 < ppl < 1e4
    em = exact_match(w, d, samples=4)
    assert 0.0 <= (em if isinstance(em, float) else em[0]) <= 1.0


def test_actstats_collector_keeps_a_uniform_strided_subsample():
    from brain_b200.utils.actstats import Collector
    c = Collector(cap=64)
    x = torch.arange(1000, dtype=torch.float32)
    for lo, hi in ((0, 7), (7, 130), (130, 131), (131, 1000)):      # ragged chunks, one stream
        c.observe("ramp", -x[lo:hi])                                 # magnitudes are recorded
    st = c.streams["ramp"]
    assert st.seen == 1000 and st.absmax == 999.0 and st.stride == 16
    kept = st.sample[:st.fill]
    assert torch.equal(kept, torch.arange(0, 1000, 16, dtype=torch.float32))
    assert c.quantile("ramp", 0.5) == pytest.approx(496.0, abs=16)
    assert c.quantile("nope", 0.5) is None
    c.observe("spiky", torch.cat([torch.ones(500), torch.tensor([100.0])]))
    rep = c.report()
    assert rep[0].name == "spiky" and rep[0].outlier_ratio == pytest.approx(100.0) and rep[0].seen == 501


def test_hsm_bubbling_lca_ordering_and_run_to_completion():
    """A controller in the shape of a serving session: Idle and Busy{Generating, Cancelling} under
    Root.  Unhandled events bubble; a transition exits up to the least common ancestor and enters
    down to the target; self-posted reminders are handled after the current event."""
    from brain_b200.utils.hsm import Handled, Hsm, Super, Tran, Unhandled

    class M:
        parents = {"root": None, "idle": "root", "busy": "root", "generating": "busy", "cancelling": "busy"}

        def __init__(self):
            self.log, self.tokens, self.hsm = [], 0, None

        def parent(self, s):
            return self.parents[s]

        def on_entry(self, s):
            self.log.append("+" + s)

        def on_exit(self, s):
            self.log.append("-" + s)

        def dispatch(self, s, ev):
            if s == "idle" and ev == "user_text":
                return Tran("generating")
            if s == "generating" and ev == "tick":
                self.tokens += 1
                if self.tokens < 3:
                    self.hsm.post("tick")          # reminder: one token per self-posted event
                    return Handled
                return Tran("idle")
            if s == "generating" and ev == "cancel":
                return Tran("cancelling")
            if s == "cancelling" and ev == "ack":
                return Tran("idle")
            if s == "busy" and ev == "status":
                self.log.append("busy!")
                return Handled
            if s == "cancelling" and ev == "status":
                return Super("busy")
            if s == "root" and ev == "status":
                self.log.append("root!")
                return Handled
            return Unhandled
    m = M()
    h = m.hsm = Hsm(m, "idle")
    h.init()
    assert m.log == ["+root", "+idle"] and h.in_state("root") and not h.in_state("busy")
    m.log.clear()
    h.send("status")                                   # idle does not handle it: root does
    assert m.log == ["root!"]
    m.log.clear()
    h.post("user_text")
    h.post("tick")
    h.run()                                            # the tick posts two more ticks to itself
    assert m.tokens == 3 and h.state == "idle"
    assert m.log == ["-idle", "+busy", "+generating", "-generating", "-busy", "+idle"]
    m.log.clear()
    m.tokens = 0
    h.send("user_text")
    h.send("cancel")                                   # sibling transition: busy is neither left nor re-entered
    assert m.log == ["-idle", "+busy", "+generating", "-generating", "+cancelling"]
    m.log.clear()
    h.send("status")                                   # explicit Super("busy")
    assert m.log == ["busy!"]
    h.send("nonsense")                                 # unhandled everywhere: ignored
    h.send("ack")
    assert h.state == "idle" and m.log[-3:] == ["-cancelling", "-busy", "+idle"]


def test_torchlib_arm_trains_on_cpu():
    """The stock-PyTorch arm of the benchmarks (same architecture, none of this repository's
    kernels) takes the native trainer's call and learns."""
    import torch
    from brain_b200.models.config import QwenConfig
    from brain_b200.perf.torchlib_ref import TorchlibTrainer
    cfg = QwenConfig(vocab=128, block_size=32, n_layers=2, d_model=64, n_heads=4, n_kv_heads=2, head_dim=16, d_ff=128)
    tr = TorchlibTrainer(cfg, torch.device("cpu"))
    ids = torch.randint(0, 128, (4, 33), dtype=torch.int32)
    losses = [float(tr.train_step(ids[:, :-1].contiguous(), ids[:, 1:].contiguous(), 1e-2, 2)) for _ in range(5)]
    assert abs(losses[0] - 4.85) < 0.3 and losses[-1] < losses[0] - 0.5


def test_native_cpu_gemm_and_linear_autograd():
    """csrc/cpu: the AVX2 GEMM in all three products of a linear layer (odd sizes, strided rows,
    alpha / beta) and the autograd wrapper against the PyTorch restatement."""
    import torch
    from brain_b200.ops import cpu_native, reference as ref
    torch.manual_seed(0)
    for M, N, K in ((1, 1, 1), (7, 19, 33), (130, 257, 300), (64, 1030, 520)):
        a, b = torch.randn(M, K), torch.randn(N, K)
        want = a @ b.t()
        assert torch.allclose(cpu_native.gemm(a, b, tb=True), want, rtol=1e-4, atol=1e-3)
        assert torch.allclose(cpu_native.gemm(a, b.t().contiguous()), want, rtol=1e-4, atol=1e-3)
        assert torch.allclose(cpu_native.gemm(a.t().contiguous(), b, ta=True, tb=True), want, rtol=1e-4, atol=1e-3)
    big = torch.randn(40, 100)
    a = big[:, 10:74]                                            # strided rows
    b = torch.randn(24, 64)
    c0 = torch.randn(40, 24)
    got = cpu_native.gemm(a, b, tb=True, out=c0.clone(), alpha=0.5, beta=2.0)
    assert torch.allclose(got, 0.5 * (a @ b.t()) + 2.0 * c0, rtol=1e-4, atol=1e-3)
    x = torch.randn(3, 17, 48, requires_grad=True)
    w = torch.randn(80, 48, requires_grad=True)
    bias = torch.randn(80, requires_grad=True)
    dy = torch.randn(3, 17, 80)
    y = cpu_native.linear(x, w, bias)
    y.backward(dy)
    xr, wr, br = (t.detach().clone().requires_grad_() for t in (x, w, bias))
    yr = ref.linear(xr, wr, br)
    yr.backward(dy)
    for g, r in ((y, yr), (x.grad, xr.grad), (w.grad, wr.grad), (bias.grad, br.grad)):
        assert torch.allclose(g, r, rtol=1e-4, atol=1e-3)
    xn, wn = torch.randn(37, 100), torch.randn(100)
    assert torch.allclose(cpu_native.rmsnorm(xn, wn, 1e-6), ref.rmsnorm(xn, wn, 1e-6), rtol=1e-4, atol=1e-5)


def test_native_cpu_attention_matches_the_materialised_reference(monkeypatch):
    """csrc/cpu/attention.cpp against the fp64 materialised-scores reference: causal and full, grouped
    KV heads, more keys than queries, lengths that are not multiples of 8 and that cross the 64-key and
    32-row tile edges; forward and all three
    gradients.  With BRAIN_CPU_NATIVE=1 the CPU path of flash_attention runs on it."""
    import math
    from brain_b200.ops import cpu_native, reference as ref
    from brain_b200.ops.attention import flash_attention
    torch.manual_seed(0)
    for B, T, S, hq, hk, hd, causal in ((2, 37, 37, 4, 2, 16, True), (1, 16, 40, 6, 3, 8, True),
                                        (2, 33, 33, 4, 4, 64, False), (1, 70, 70, 2, 1, 24, True),
                                        (1, 150, 150, 2, 1, 16, True), (1, 65, 129, 3, 1, 40, True),
                                        (1, 130, 67, 2, 2, 32, False)):
        q = torch.randn(B * T, hq * hd, requires_grad=True)
        k = torch.randn(B * S, hk * hd, requires_grad=True)
        v = torch.randn(B * S, hk * hd, requires_grad=True)
        o = cpu_native.attention(q, k, v, B, T, S, hq, hk, hd, causal)
        g = torch.randn_like(o)
        got = torch.autograd.grad(o, (q, k, v), g)
        q64, k64, v64 = (t.detach().double().requires_grad_() for t in (q, k, v))
        want = ref.attention(q64.reshape(B, T, hq, hd), k64.reshape(B, S, hk, hd), v64.reshape(B, S, hk, hd),
                             causal, 1 / math.sqrt(hd)).reshape(B * T, hq * hd)
        wgrads = torch.autograd.grad(want, (q64, k64, v64), g.double())
        assert float((o.detach() - want.detach()).abs().max()) < 5e-6
        for a, b in zip(got, wgrads):
            assert float((a - b).abs().max()) < 2e-5
    # routing: the public op takes the native kernels only when the CPU backend's native part is on
    q = torch.randn(2 * 16, 4 * 8)
    k = torch.randn(2 * 16, 2 * 8)
    v = torch.randn(2 * 16, 2 * 8)
    monkeypatch.setenv("BRAIN_CPU_NATIVE", "0")
    base = flash_attention(q, k, v, 2, 16, 4, 2, 8)
    monkeypatch.setenv("BRAIN_CPU_NATIVE", "1")
    calls = []
    real = cpu_native.attention
    monkeypatch.setattr(cpu_native, "attention", lambda *a, **kw: (calls.append(1), real(*a, **kw))[1])
    nat = flash_attention(q, k, v, 2, 16, 4, 2, 8)
    assert calls and torch.allclose(nat, base, atol=1e-5)
    assert cpu_native.attention_supported(q, 128, 4096) and not cpu_native.attention_supported(q, 12, 16)


def test_bench_reference_arm_reports_unavailable_and_exits_zero():
    """``bench.py --impl reference`` cannot run the reference here (a Rust / graphics-API workspace): it
    must say so in one JSON line and exit 0, whatever the other flags are."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference", "--gpus", "2",
                        "--steps", "3", "--warmup", "3"], capture_output=True, text=True, timeout=120)
    assert p.returncode == 0, p.stderr[-2000:]
    lines = [l for l in p.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and isinstance(d.get("unavailable"), str) and d["unavailable"]


def test_native_cpu_gemm_on_the_avx2_micro_kernel():
    """On a CPU with AVX-512 the GEMM picks its 12 x 32 tile at run time; ``BRAIN_CPU_ISA=avx2`` (read once per
    process, hence the child process) keeps the 6 x 16 AVX2 tile, which must give the same products."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = (
        "import sys, torch\n"
        f"sys.path.insert(0, {root!r})\n"
        "from brain_b200.ops import cpu_native\n"
        "torch.manual_seed(1)\n"
        "for M, N, K in ((5, 17, 9), (97, 130, 300), (256, 515, 257)):\n"
        "    a, b = torch.randn(M, K), torch.randn(N, K)\n"
        "    want = a @ b.t()\n"
        "    assert torch.allclose(cpu_native.gemm(a, b, tb=True), want, rtol=1e-4, atol=1e-3)\n"
        "    assert torch.allclose(cpu_native.gemm(a.t().contiguous(), b.t().contiguous(), ta=True), want, rtol=1e-4, atol=1e-3)\n"
        "print('ok')\n")
    p = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300,
                       env=dict(os.environ, BRAIN_CPU_ISA="avx2"))
    assert p.returncode == 0 and "ok" in p.stdout, p.stderr[-2000:]
