"""Fused tensor-parallel GEMM kernels == NCCL baseline, on 2 GPUs (skipped when fewer)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fused_tp_matches_nccl_two_ranks():
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    p = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
                        "--nproc-per-node=2", "--master-addr", "127.0.0.1", "--master-port", "29543",
                        os.path.join(here, "tp_worker.py")], capture_output=True, text=True,
                       timeout=600, env=env)
    assert p.returncode == 0, p.stdout[-3000:] + p.stderr[-3000:]
    assert "ok=1" in p.stdout


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_nvls_multimem_allreduce_two_ranks():
    """The same worker with the all-reduce routed through NVLink multicast (multimem.ld_reduce /
    multimem.st).  Where the fabric offers no multicast binding the worker reports nvls off and the
    plain peer-memory path is what ran."""
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, BRAIN_TP_NVLS="1")
    p = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
                        "--nproc-per-node=2", "--master-addr", "127.0.0.1", "--master-port", "29544",
                        os.path.join(here, "tp_worker.py")], capture_output=True, text=True,
                       timeout=600, env=env)
    assert p.returncode == 0, p.stdout[-3000:] + p.stderr[-3000:]
    assert "ok=1" in p.stdout
