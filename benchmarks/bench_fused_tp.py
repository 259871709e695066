"""Fused tensor-parallel kernels vs their unfused NCCL baselines (numerics + device timing).

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29511 \\
        benchmarks/bench_fused_tp.py [--check-only] [--out FILE]

Shapes are the Qwen3-8B / Qwen3-32B projections under TP. Timing: CUDA events on the launching
stream, 3 warm-up iterations, barrier + synchronise on both sides, max over ranks. Roofline of
a fused kernel = the slower of (FLOPs / measured cuBLAS bf16 peak) and (bytes that must cross
NVLink per GPU / 770 GB/s measured peer-copy bandwidth).
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from parallax_b200.ops import cuda as cu  # noqa: E402
from parallax_b200.ops import reference as ref  # noqa: E402
from parallax_b200.parallel import fused  # noqa: E402
from parallax_b200.parallel.symm import TPWorkspace  # noqa: E402

NVLINK_GBS = 770.0


def peaks():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return json.load(open(p))["bf16_tflops"], "of measured"
    return 1590.0, "of fallback"


def rel(a, b):
    return float((a.float() - b.float()).norm() / (b.float().norm() + 1e-12))


def timed(fn, group, iters=10, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier(group)
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    dist.barrier(group)
    t = torch.tensor([s.elapsed_time(e) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t)


def check_rs(ws, group, rank, tp, Rp, N, Kl, residual=True):
    g = torch.Generator(device="cuda").manual_seed(100 + rank)
    a = torch.randn(tp * Rp, Kl, device="cuda", dtype=torch.bfloat16, generator=g)
    w = torch.randn(N, Kl, device="cuda", dtype=torch.bfloat16, generator=g) * 0.05
    res = torch.randn(Rp, N, device="cuda", dtype=torch.bfloat16, generator=g) if residual else None
    want = a.float() @ w.float().t()
    dist.all_reduce(want, group=group)
    want = want[rank * Rp:(rank + 1) * Rp]
    if residual:
        want = want + res.float()
    errs = []
    for _ in range(3):  # repeated calls exercise the alternating buffer sets and epochs
        got = fused.gemm_rs(ws, a, w, residual=res)
        torch.cuda.synchronize()
        errs.append(rel(got, want))
    cu.check_status(torch.device("cuda", torch.cuda.current_device()))
    return max(errs), (a, w, res)


def check_ag(ws, group, rank, tp, Rp, N, K, epi):
    g = torch.Generator(device="cuda").manual_seed(200 + rank)
    xs = torch.randn(Rp, K, device="cuda", dtype=torch.bfloat16, generator=g)
    gw = torch.Generator(device="cuda").manual_seed(7)
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16, generator=gw) * 0.05
    full = torch.empty(tp * Rp, K, device="cuda", dtype=torch.bfloat16)
    dist.all_gather_into_tensor(full, xs, group=group)
    want = ref.linear(full, w, epi=epi).float()
    errs = []
    for _ in range(3):
        token, shard = fused.gemm_ag_begin(ws, Rp, K)
        shard.copy_(xs)
        got = fused.gemm_ag(ws, token, w, epi=epi)
        torch.cuda.synchronize()
        errs.append(rel(got, want))
    cu.check_status(torch.device("cuda", torch.cuda.current_device()))
    return max(errs), (xs, w)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--check-only", action="store_true")
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl", device_id=dev)
    group = dist.group.WORLD
    tp = world
    tf, tag = peaks()
    rows = []
    # (name, tokens, N_total, K_total): o_proj/down_proj are row-parallel (K split), qkv/gate_up column-parallel (N split)
    T_list = [512, 2560] if not args.check_only else [256]
    ws = TPWorkspace(group, dev, tp, rank, max_rows_per_rank=(max(T_list) // tp + 127) // 128 * 128,
                     max_k=5120, max_n=5120)
    for T in T_list:
        Rp = (T // tp + 127) // 128 * 128
        for name, N, K in [("o_proj", 4096, 4096), ("down_proj", 4096, 12288)]:
            Kl = K // tp
            err, (a, w, res) = check_rs(ws, group, rank, tp, Rp, N, Kl)
            row = {"kernel": "gemm_rs", "layer": name, "tp": tp, "tokens": tp * Rp, "N": N, "K_local": Kl,
                   "rel_err": round(err, 5)}
            assert err < 2e-2, row
            if not args.check_only:
                ms = timed(lambda: fused.gemm_rs(ws, a, w, residual=res), group)
                ms_nccl = timed(lambda: fused.gemm_rs_nccl(group, a, w, res), group)
                flops = 2.0 * tp * Rp * N * Kl
                link_bytes = (tp - 1) * Rp * N * 2.0
                ideal = max(flops / (tf * 1e12), link_bytes / (NVLINK_GBS * 1e9)) * 1e3
                row.update(ms=round(ms, 4), nccl_baseline_ms=round(ms_nccl, 4), roofline_frac=round(ideal / ms, 3),
                           tag=tag)
            rows.append(row)
            if rank == 0:
                print(json.dumps(row), flush=True)
        for name, N, K, epi in [("qkv_proj", 6144, 4096, ref.EPI_NONE), ("gate_up", 24576, 4096, ref.EPI_SILU_MUL)]:
            Nl = N // tp
            err, (xs, w) = check_ag(ws, group, rank, tp, Rp, Nl, K, epi)
            row = {"kernel": "gemm_ag", "layer": name, "tp": tp, "tokens": tp * Rp, "N_local": Nl, "K": K,
                   "rel_err": round(err, 5)}
            assert err < 2e-2, row
            if not args.check_only:
                def run():
                    # both buffer sets already hold xs from the check above; in the model the
                    # shard is written in place by the RMSNorm kernel that precedes the GEMM
                    token, _shard = fused.gemm_ag_begin(ws, Rp, K)
                    fused.gemm_ag(ws, token, w, epi=epi)

                ms = timed(run, group)
                ms_nccl = timed(lambda: fused.gemm_ag_nccl(group, xs, w, silu_mul=False), group)   # baseline without the activation
                flops = 2.0 * tp * Rp * Nl * K
                link_bytes = (tp - 1) * Rp * K * 2.0
                ideal = max(flops / (tf * 1e12), link_bytes / (NVLINK_GBS * 1e9)) * 1e3
                row.update(ms=round(ms, 4), nccl_baseline_ms=round(ms_nccl, 4), roofline_frac=round(ideal / ms, 3),
                           tag=tag)
            rows.append(row)
            if rank == 0:
                print(json.dumps(row), flush=True)
    if rank == 0 and args.out:
        os.makedirs(os.path.dirname(args.out) or ".", exist_ok=True)
        json.dump(rows, open(args.out, "w"), indent=1)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
