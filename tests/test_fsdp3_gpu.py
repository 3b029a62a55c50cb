"""Weight-sharded data parallelism: GEMMs that all-gather their weights over NVLink peer memory as they run."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_weight_gathering_gemms_and_sharded_model(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least 2 GPUs")
    out = str(tmp_path / "res.json")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29719", os.path.join(ROOT, "tests", "fsdp3_worker.py"), out]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    for r in json.load(open(out)):
        assert r["fused"], "symmetric memory unavailable: the fused kernels did not run"
        for k, v in r.items():
            if k.startswith(("fwd_", "dgrad_", "wgrad_")):
                assert v < 1.5e-2, (k, v)
        assert r["model_loss_rel"] < 2e-2 and r["model_grad_sharded"] < 5e-2 and r["model_grad_embed"] < 5e-2, r
