"""The fused o_proj all-reduce + residual add + RMSNorm kernel against NCCL + torch, on 2 ranks.

The check itself is ``multi_gpu_allreduce_check.py`` (one process per GPU under torchrun); this
wrapper launches it when the machine has at least two GPUs.
"""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_fused_allreduce_matches_nccl():
    script = Path(__file__).with_name("multi_gpu_allreduce_check.py")
    env = dict(os.environ)
    env.pop("KTK_TIME_ALLREDUCE", None)
    r = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
         "--master-addr", "127.0.0.1", "--master-port", "29541", str(script)],
        capture_output=True, text=True, timeout=240, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "fused all-reduce ok on 2 ranks" in r.stdout
