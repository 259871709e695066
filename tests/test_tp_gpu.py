"""Fused GEMM->reduce-scatter and all-gather->GEMM on two B200s against fp32 math.

Needs two GPUs; the ranks are child processes started with torch.distributed.run. NVLS is
switched off for NCCL in this test."""

import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_fused_tp_kernels_two_ranks():
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", "29517", os.path.join(ROOT, "benchmarks", "bench_fused_tp.py"), "--check-only"]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert '"kernel": "gemm_rs"' in res.stdout and '"kernel": "gemm_ag"' in res.stdout
