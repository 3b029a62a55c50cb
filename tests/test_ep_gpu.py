"""Expert parallelism over NVLink peer memory: dispatch / combine pulls around the grouped GEMM."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_expert_parallel_layer_matches_single_gpu(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least 2 GPUs")
    out = str(tmp_path / "res.json")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29721", os.path.join(ROOT, "tests", "ep_worker.py"), out]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    for r in json.load(open(out)):
        assert r["fused"], "symmetric memory unavailable: the peer-memory path did not run"
        for k, v in r.items():
            if k != "fused":
                assert v < 2.5e-2, (k, v)
