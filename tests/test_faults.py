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
