"""Fused expert-parallel MoE (peer-load dispatch/combine) == single-rank MoE, on 2 GPUs."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fused_ep_matches_single_rank():
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    p = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
                        "--nproc-per-node=2", "--master-addr", "127.0.0.1", "--master-port", "29545",
                        os.path.join(here, "ep_worker.py")], capture_output=True, text=True,
                       timeout=600, env=env)
    assert p.returncode == 0, p.stdout[-3000:] + p.stderr[-3000:]
    assert "ok=1" in p.stdout
