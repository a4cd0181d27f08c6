"""Fused GEMM + all-gather and the K-sharded reduce-scatter across GPUs: needs at least two GPUs on the box;
skipped otherwise."""
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.gpu
def test_fused_gather_matches_unsharded_kernel_on_two_gpus():
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", "29561", os.path.join(ROOT, "tests", "fused_gather_worker.py")]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert res.stdout.count("bit-equal to the unsharded kernel = True") == 4, res.stdout[-3000:]
    assert res.stdout.count("bit-equal to the single-GPU sum = True") == 6, res.stdout[-3000:]   # NCCL form + 2 fused calls, per rank
