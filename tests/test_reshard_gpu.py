"""Trainer -> rollout weight transfer over NVLink peer memory (LoRA merged on the way)."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_p2p_reshard_two_gpus(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least 2 GPUs")
    out = str(tmp_path / "res.json")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29723", os.path.join(ROOT, "tests", "reshard_worker.py"), out]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    r = json.load(open(out))
    assert r[0]["fused"] and r[1]["fused"]
    assert r[0]["max_abs_diff"] < 2e-2, r       # bf16 rounding of the merged LoRA weight
