"""Fault scenarios (host-side injection only): every scenario must report the failure, leave the
surviving answers uncorrupted and keep unrelated work running."""
import pytest

from brain_b200.perf import faults


@pytest.mark.parametrize("name", list(faults.SCENARIOS))
def test_fault_scenario(name):
    r = faults.SCENARIOS[name]()
    assert r.reported, r
    assert r.clean, r
    assert r.survived, r


def test_device_error_word_raises_in_training_and_serving(monkeypatch):
    """A bounded wait that ran out inside a kernel leaves a code in the device error word.  The
    trainer reads it once per optimiser step and the scheduler once per step before it commits;
    here the native read is replaced by a fake that returns 'peer flag never arrived'."""
    import torch
    from brain_b200.ops import _cuda
    from brain_b200.engine import Trainer
    from brain_b200.models.config import QwenConfig
    from brain_b200.models.qwen3 import Qwen3
    from brain_b200.serve.scheduler import Scheduler
    from tests.test_serving import FakeDecoder

    codes = iter([0, 6])
    monkeypatch.setattr(_cuda, "_error_source", lambda: next(codes))
    # serving: the first step passes, the second raises before any token of it is committed
    dec = FakeDecoder()
    dec.check_device = _cuda.check_error
    s = Scheduler(dec, max_batch=2, window=1)
    rid = s.submit([1, 2, 3], 4)
    s.step()
    before = list(s.tokens_of(rid))
    with pytest.raises(_cuda.NativeError, match="peer flag never arrived"):
        s.step()
    assert s.tokens_of(rid) == before

    # training: poll_error raises from optimizer_step (forced onto the CUDA branch of the check)
    cfg = QwenConfig(vocab=64, block_size=16, n_layers=1, d_model=32, n_heads=2, n_kv_heads=1,
                     head_dim=16, d_ff=64)
    tr = Trainer(Qwen3(cfg).init_weights(seed=0), device=torch.device("cpu"))
    ids = torch.randint(0, 64, (2, 17), dtype=torch.int32)
    tr.train_step(ids[:, :-1].contiguous(), ids[:, 1:].contiguous(), 1e-3)     # CPU: no check
    tr.cuda = True
    monkeypatch.setattr(tr, "_to_device", lambda t: t)
    monkeypatch.setattr(_cuda, "_error_source", lambda: 6)
    with pytest.raises(_cuda.NativeError, match="device error 6"):
        tr.optimizer_step(1e-3)
