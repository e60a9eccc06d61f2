"""Autotune cache: the fastest candidate wins, failing candidates are skipped, winners persist
across instances and are keyed by device name."""
import json

from brain_b200.utils.tune import AutoTuner


def test_autotuner_picks_caches_and_persists(tmp_path):
    path = str(tmp_path / "t" / "tune.json")
    cost = {0: 3.0, 64: 2.0, 128: 1.0}
    ran = []

    def timer(fn):
        fn()
        return cost[ran[-1]]

    def run(c):
        if c == 256:
            raise RuntimeError("unsupported tile")
        ran.append(c)

    t = AutoTuner(path, "B200", timer)
    k = t.key("gemm_bf16", 4096, 1024, 1024, 0, 0, 0)
    assert t.pick(k, (0, 64, 128, 256), run) == 128 and t.trials == 3
    assert t.pick(k, (0, 64, 128, 256), run) == 128 and t.trials == 3      # cached: nothing re-timed
    assert json.loads(open(path).read()) == {k: 128}
    t2 = AutoTuner(path, "B200", timer)
    assert t2.pick(k, (0,), run) == 128 and t2.trials == 0                  # persisted
    t3 = AutoTuner(path, "H100", timer)
    assert t3.key("gemm_bf16", 4096, 1024, 1024, 0, 0, 0) != k             # other device: other key
