"""Sharded execution on real GPUs: needs at least two (skipped otherwise; the same partition and
gather logic runs on CPU ranks in tests/test_multi_gloo.py)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_two_rank_shard_and_nccl_gather(hb_lib, oracle_libs):
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs two GPUs; this box has %d" % n)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", str(29600 + os.getpid() % 300),
           os.path.join(ROOT, "tests", "multi_rank_check.py")]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    assert "MULTI_RANK_CHECK PASS" in res.stdout
