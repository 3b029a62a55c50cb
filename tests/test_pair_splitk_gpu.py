"""The CTA-pair split-K GEMM for a few hundred rows (csrc/gemm_pair_splitk.cu) against fp32 PyTorch. The kernel is
selected by an environment variable that the library reads once, so the checks run in a child process."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r"""
import json, sys, torch
sys.path.insert(0, %r)
from tunix_b200 import _lib
from tunix_b200.ops import kernels as K
torch.manual_seed(0)
out = []
for (M, N, Kd) in [(256, 4096, 4096), (256, 6144, 4096), (200, 4096, 12288), (512, 4096, 4096), (384, 2048, 2048), (129, 264, 1032)]:
    A = torch.randn(M, Kd, device="cuda", dtype=torch.bfloat16)
    B = (torch.randn(N, Kd, device="cuda") * 0.05).to(torch.bfloat16)
    bias = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    res = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    ref = A.float() @ B.float().t()
    n0 = K.launch_count
    y = K.gemm(A, B)
    y2 = K.gemm(A, B, bias=bias, residual=res, alpha=0.5)
    acc = torch.ones(M, N, device="cuda")
    K.gemm(A, B, out=acc, accumulate=True)
    _lib.raise_if_kernel_error()
    rel = lambda a, b: float((a.float() - b).norm() / b.norm())
    full = 0.5 * ref + bias.float() + res.float()
    out.append({"shape": [M, N, Kd], "rel": rel(y, ref), "rel_epi": rel(y2, full), "rel_acc": rel(acc, ref + 1.0),
                "maxabs": float((y.float() - ref).abs().max()), "scale": float(ref.abs().max())})
print("RESULT " + json.dumps(out))
"""


def test_pair_splitk_gemm_matches_fp32():
    env = dict(os.environ, TUNIX_B200_PAIR_SPLITK="1")
    p = subprocess.run([sys.executable, "-c", CHILD % ROOT], env=env, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    line = [l for l in p.stdout.splitlines() if l.startswith("RESULT ")][-1]
    for r in json.loads(line[7:]):
        assert r["rel"] < 1e-2 and r["rel_epi"] < 1e-2 and r["rel_acc"] < 2e-3, r
        assert r["maxabs"] < 0.02 * r["scale"], r
