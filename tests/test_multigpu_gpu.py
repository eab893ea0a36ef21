"""Runs tests/multigpu_check.py on two GPUs when the box has them (skipped on a single GPU)."""
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sharded_equals_single_gpu():
    script = Path(__file__).resolve().parent / "multigpu_check.py"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", "29533", str(script)]
    env = {"NCCL_NVLS_ENABLE": "0"}
    import os

    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env={**os.environ, **env})
    assert res.returncode == 0 and "multigpu ok" in res.stdout, res.stdout[-2000:] + res.stderr[-4000:]
