"""Multi-GPU checks, run as one process per GPU under torchrun when the machine has at least two GPUs:

* ``multi_gpu_allreduce_check.py``: the fused NVLink exchange kernels against an fp32 all-reduce + torch;
* ``multi_gpu_layer_check.py``: the KV-head-sharded decoder layer (both exchanges) against the TP=1 layer, and a
  sharded decoder stack (prefill + decode) against the unsharded one.
"""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu

needs_two = pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs two GPUs")


def _torchrun(script: str, nproc: int, port: int):
    env = dict(os.environ)
    return subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(nproc),
         "--master-addr", "127.0.0.1", "--master-port", str(port), str(Path(__file__).with_name(script))],
        capture_output=True, text=True, timeout=420, env=env)


@needs_two
def test_fused_exchange_matches_fp32_allreduce():
    r = _torchrun("multi_gpu_allreduce_check.py", 2, 29541)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "fused exchange ok on 2 ranks" in r.stdout


@needs_two
def test_sharded_layer_equals_tp1_layer():
    r = _torchrun("multi_gpu_layer_check.py", 2, 29543)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert r.stdout.count("tp layer ok on 2 ranks") == 5
    assert "tp decoder stack ok on 2 ranks" in r.stdout
