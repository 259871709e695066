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


def _run_dist(mode, tmp_path, port):
    import json

    out = tmp_path / f"{mode}.json"
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1",
               PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(ROOT, "tests", "helpers", "dist_engine_gpu_rank.py"), mode, str(out)]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=240)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    return json.loads(out.read_text())


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_dist_engine_tensor_parallel_fused(tmp_path):
    """tp=2 over the fused kernels: logits of a mixed step within bf16 noise of one GPU."""
    r = _run_dist("tp", tmp_path, 29519)
    assert r["logit_rel_err"] < 3e-2, r
    assert r["token_agreement"] > 0.7, r


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_dist_engine_pipeline_two_stages(tmp_path):
    """pp=2 over NCCL send/recv with two micro-batches in flight: same tokens as one GPU."""
    r = _run_dist("pp", tmp_path, 29521)
    assert r["token_agreement"] > 0.95, r


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_expert_parallel_moe_two_ranks():
    """Dispatch / grouped GEMMs / combine-in-epilogue over peer memory against fp32 math."""
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", "29523", os.path.join(ROOT, "benchmarks", "bench_fused_ep.py"), "--check-only"]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert '"kernel": "ep_moe_ffn"' in res.stdout


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_dist_engine_expert_parallel_fused(tmp_path):
    """Attention tp=2 + experts ep=2 (peer-memory dispatch/combine) against one GPU."""
    r = _run_dist("ep", tmp_path, 29525)
    assert r["logit_rel_err"] < 3e-2, r
    assert r["token_agreement"] > 0.7, r
