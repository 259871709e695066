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


def _run_dist(mode, tmp_path, port, nproc=2):
    import json

    out = tmp_path / f"{mode}.json"
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1",
               PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nproc-per-node", str(nproc), "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(ROOT, "tests", "helpers", "dist_engine_gpu_rank.py"), mode, str(out)]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=420)
    if res.returncode != 0:
        import glob

        errs = "".join(f"\n--- {p}\n" + open(p).read()[-2500:] for p in sorted(glob.glob(f"{out}.rank*.err")))
        raise AssertionError(errs + res.stderr[-1500:])
    return json.loads(out.read_text())


# layout, GPUs it needs. The 4- and 8-GPU rows run when the box has that many devices.
LAYOUTS = [("tp2", 2), ("pp2", 2), ("ep2", 2), ("dpep2", 2),
           ("tp4", 4), ("pp4", 4), ("pp2tp2", 4), ("dpep4", 4), ("pp2dpep2", 4),
           ("tp8", 8), ("pp8", 8), ("pp2tp4", 8), ("dpep8", 8), ("pp2dpep4", 8),
           # tensor-parallel stages of the other families (heads split, sequence-sharded residual stream)
           ("tp2@small-mla", 2), ("tp2@small-dsa", 2), ("tp2@small-hybrid", 2), ("tp2@small-msa", 2),
           # e4m3 KV pages under pipeline and tensor parallelism
           ("pp2#fp8kv", 2), ("tp2#fp8kv", 2),
           # per-request LoRA adapters on tensor-parallel ranks (sliced adapters) and on pipeline stages
           ("tp2%lora", 2), ("pp2%lora", 2)]


@pytest.mark.parametrize("mode,n", LAYOUTS)
def test_dist_engine_layout_matches_one_gpu(mode, n, tmp_path):
    """Every layout of the multi-GPU engine (pipeline stages, fused tensor-parallel kernels, expert
    parallelism over peer memory with data-parallel attention, and combinations) against a single-GPU
    engine: all tokens whose single-GPU logit margin exceeds bf16 summation noise must be equal."""
    if torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")
    r = _run_dist(mode, tmp_path, 29600 + LAYOUTS.index((mode, n)) * 2, nproc=n)
    import json

    brief = json.dumps({k: r.get(k) for k in ("mode", "compared", "equal", "noise", "logit_rel_err", "logit_abs_err",
                                              "mismatches", "token_agreement")})
    # random-init weights leave few tokens with a clear margin; what counts is that none of them differs
    assert r["compared"] >= (2 if "#fp8kv" in mode else 4), brief
    assert r["equal"] == r["compared"], brief
    if "logit_rel_err" in r:
        assert r["logit_rel_err"] < 3e-2, r
    if mode.startswith("pp") and "tp" not in mode and "ep" not in mode and "#" not in mode:
        # same kernels in the same order on every stage: only the hand-off differs
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
