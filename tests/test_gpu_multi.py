"""Multi-GPU checks (2 ranks, one per GPU): peer-memory collectives, fused GEMM+all-reduce, tensor-parallel engine."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_selftest_two_ranks():
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", "29541", "-m", "atlas_b200.parallel.selftest", "--engine"]
    r = subprocess.run(cmd, cwd=ROOT, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600)
    checks = [json.loads(l) for l in r.stdout.splitlines() if l.startswith("{") and '"check"' in l]
    assert r.returncode == 0, r.stdout[-3000:]
    assert checks and all(c["ok"] for c in checks), checks
