"""Expert-parallel MoE layer over peer memory vs its NCCL baseline (numerics + device timing).

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29513 \\
        benchmarks/bench_fused_ep.py [--check-only] [--out FILE]

Shape: the Qwen3-30B-A3B MoE layer (hidden 2048, 128 experts, top-8, expert FFN 768) with the token
rows split evenly over the ranks. Timing: CUDA events, 3 warm-up iterations, barrier + synchronise
on both sides, max over ranks. Roofline = the slower of (expert FLOPs on this rank / measured cuBLAS
bf16 peak) and (bytes this rank must send or receive over NVLink / 770 GB/s).
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
from parallax_b200.parallel.ep import EPWorkspace, ep_moe_ffn, ep_moe_ffn_nccl  # noqa: E402

NVLINK_GBS = 770.0


def peaks():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return json.load(open(p))["bf16_tflops"], "of measured"
    return 1590.0, "of fallback"


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
    ep = world
    tf, tag = peaks()
    H, E, k, I = 2048, 128, 8, 768
    epr = E // ep
    rows_list = [96] if args.check_only else [256, 2048]
    ws = EPWorkspace(group, dev, ep, rank, max(rows_list), k, H)
    gw = torch.Generator(device="cuda").manual_seed(5)          # same expert weights on every rank
    w1_all = torch.randn(E * 2 * I, H, device="cuda", generator=gw) * 0.03
    w2_all = torch.randn(E * H, I, device="cuda", generator=gw) * 0.03
    w1 = w1_all[rank * epr * 2 * I:(rank + 1) * epr * 2 * I].to(torch.bfloat16).contiguous()
    w2 = w2_all[rank * epr * H:(rank + 1) * epr * H].to(torch.bfloat16).contiguous()
    out_rows = []
    for rows in rows_list:
        n_valid = rows - 5 if rank == world - 1 else rows          # a ragged tail on the last rank
        g = torch.Generator(device="cuda").manual_seed(100 + rank)
        x = (torch.randn(rows, H, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
        logits = torch.randn(rows, E, device="cuda", generator=g)
        wts, ids = torch.topk(torch.softmax(logits, -1), k)
        wts = (wts / wts.sum(-1, keepdim=True)).float().contiguous()
        ids = ids.int().contiguous()
        base = (torch.randn(rows, H, device="cuda", generator=g) * 0.1).to(torch.bfloat16)
        # fp32 reference on this rank's rows with all experts
        want = ref.moe_ffn(x[:n_valid].float().cpu(), ids[:n_valid].cpu(), wts[:n_valid].cpu(),
                           w1_all.to(torch.bfloat16).float().cpu(), w2_all.to(torch.bfloat16).float().cpu(), E,
                           base=base[:n_valid].float().cpu())
        errs = []
        for _ in range(3):
            got = ep_moe_ffn(ws, x, n_valid, ids, wts, w1, w2, epr, base=base)
            torch.cuda.synchronize()
            errs.append(float((got[:n_valid].float().cpu() - want).norm() / want.norm()))
        cu.check_status(dev)
        base_out = ep_moe_ffn_nccl(group, x, n_valid, ids, wts, w1, w2, epr, base=base)
        err_nccl = float((base_out[:n_valid].float().cpu() - want).norm() / want.norm())
        row = {"kernel": "ep_moe_ffn", "ep": ep, "rows_per_rank": rows, "hidden": H, "experts": E, "top_k": k,
               "expert_ffn": I, "rel_err": round(max(errs), 5), "rel_err_nccl_baseline": round(err_nccl, 5)}
        assert max(errs) < 2e-2 and err_nccl < 2e-2, row
        if not args.check_only:
            ms = timed(lambda: ep_moe_ffn(ws, x, n_valid, ids, wts, w1, w2, epr, base=base), group)
            ms_nccl = timed(lambda: ep_moe_ffn_nccl(group, x, n_valid, ids, wts, w1, w2, epr, base=base), group)
            pairs = rows * k                                        # balanced routing: pairs served per rank
            flops = pairs * 6.0 * H * I
            link_bytes = pairs * (ep - 1) / ep * H * 2.0            # sent (dispatch) = received (combine)
            ideal = max(flops / (tf * 1e12), link_bytes / (NVLINK_GBS * 1e9)) * 1e3
            row.update(ms=round(ms, 4), nccl_baseline_ms=round(ms_nccl, 4), roofline_frac=round(ideal / ms, 3), tag=tag)
        out_rows.append(row)
        if rank == 0:
            print(json.dumps(row), flush=True)
    if rank == 0 and args.out:
        os.makedirs(os.path.dirname(args.out) or ".", exist_ok=True)
        json.dump(out_rows, open(args.out, "w"), indent=1)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
