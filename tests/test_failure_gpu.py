"""Device half of failure detection: a bounded wait that runs out reports through the status word."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_barrier_wait_runs_out_cleanly(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least 2 GPUs")
    out = str(tmp_path / "res.json")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29725", os.path.join(ROOT, "tests", "barrier_timeout_worker.py"), out]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    r = json.load(open(out))
    assert r["raised"] and "flag wait" in r["message"] and r["usable"], r
