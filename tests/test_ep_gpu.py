"""Fused expert-parallel MoE (peer-load dispatch/combine) == single-rank MoE, on 2 GPUs."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("inside_gemm", ["1", "0"])
def test_fused_ep_matches_single_rank(inside_gemm):
    """Both forms of the row transfers: inside the grouped GEMMs (mover CTAs / combine epilogue) and as
    separate full-width peer-load kernels (what ``auto`` picks for the small experts of this test)."""
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", BRAIN_EP_FUSED_DISPATCH=inside_gemm,
               BRAIN_EP_FUSED_COMBINE=inside_gemm)
    p = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
                        "--nproc-per-node=2", "--master-addr", "127.0.0.1", "--master-port", "29545",
                        os.path.join(here, "ep_worker.py")], capture_output=True, text=True,
                       timeout=600, env=env)
    assert p.returncode == 0, p.stdout[-3000:] + p.stderr[-3000:]
    assert "ok=1" in p.stdout
