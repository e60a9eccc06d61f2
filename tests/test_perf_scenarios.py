"""Named perf scenarios on a tiny synthetic Qwen behind the real engine + scheduler (CPU) and on
the deterministic fake target."""
import pytest
import torch

from brain_b200.perf import scenarios as sc
from brain_b200.perf.targets import FakeTarget, SchedulerTarget, synth_qwen

VOCAB = 64


@pytest.fixture(scope="module")
def model():
    return synth_qwen("1x32x4x64").eval()


def _make(model, **kw):
    return lambda: SchedulerTarget(model, max_batch=kw.pop("max_batch", 4), ctx=512, block_size=8, **kw)


def test_tier1_on_fake_target():
    mk = lambda: FakeTarget(max_concurrent=4, prefill_steps=2)
    lat = sc.latency(mk, n=4, vocab=VOCAB, input_override=16)
    thr = sc.throughput(mk, n=8, vocab=VOCAB, input_override=16)
    assert lat["summary"]["completed"] == 4 and thr["summary"]["completed"] == 8
    sw = sc.sweep(mk, ladder=(1, 2, 4, 8), n=8, vocab=VOCAB, input_override=16)
    assert [r["concurrency"] for r in sw["rows"]] == [1, 2, 4, 8] and sw["knee"] in (1, 2, 4, 8)
    st = sc.startup(mk, vocab=VOCAB)
    assert st["build_s"] >= 0 and st["first_artifact_s"] is not None
    sv = sc.serve(mk, per_s=2000.0, n=8, vocab=VOCAB, input_override=16)
    assert sv["summary"]["completed"] == 8


def test_mixed_and_soak(model):
    r = sc.mixed(_make(model), n=12, concurrency=4, vocab=VOCAB, short=8, long=96, out_tokens=4)
    assert r["passed"] and r["classes"]["short"]["requests"] + r["classes"]["long"]["requests"] == 12
    s = sc.soak(_make(model), seconds=1.0, concurrency=2, vocab=VOCAB, input_len=16, out_tokens=4)
    assert s["rounds"] >= 1 and s["blocks_before"] == s["blocks_after"] and s["completed"] > 0


def test_cancel_frees_blocks_and_leaves_survivors_untouched(model):
    r = sc.cancel(_make(model, prefix_cache=False), n=8, cancel_every=2, after_artifacts=2, vocab=VOCAB, input_len=24,
                  out_tokens=12)
    assert r["passed"], r
    assert r["cancelled"] == 4 and r["late_artifacts"] == 0 and r["blocks_before"] == r["blocks_after"]


def test_kvcache_saves_prefill_and_keeps_outputs(model):
    r = sc.kvcache(_make(model, prefix_cache=True), _make(model, prefix_cache=False), n=6, prefix=96, tail=16,
                   out_tokens=4, vocab=VOCAB)
    assert r["outputs_equal"] and r["passed"], r
    assert r["cached"]["prefill_tokens"] < r["uncached"]["prefill_tokens"]


def test_overload_rejects_the_excess(model):
    mk = _make(model, max_batch=2, policy="max_queue_depth", policy_arg=2.0)
    r = sc.overload(mk, capacity_per_s=50.0, factor=40.0, n=24, vocab=VOCAB, input_override=16)
    assert r["passed"], r
    assert 0 < r["rejected_fraction"] < 1


def test_residency_placement_and_frontend_scenarios():
    """The scenarios around the engine: many models over one budget through the real residency
    manager (nothing fails or starves under a 4x oversubscribed catalogue with a popularity shift),
    the placer's mix against the best single device, and the host-side cost per request."""
    from brain_b200.perf import scenarios2 as s2
    r = s2.residency(requests=160, seed=1)
    assert r["passed"], r
    assert r["oversubscription"] >= 3 and r["evictions"] > 0 and r["hit_rate"] > 0.2
    assert r["ttfa_warm_p50_ms"] < r["ttfa_cold_p50_ms"]
    p = s2.placement(requests=80)
    assert p["passed"] and p["placement_efficiency"] > 1.2, p
    f = s2.frontend(requests=10)
    assert f["passed"] and f["host_cores_per_saturated_device"] > 0 and f["dominant_stage"] in f["stage_us_per_request"]
    from brain_b200.perf.cli import run_perf
    assert run_perf(["scenario", "frontend", "--requests", "5"]) == 0
