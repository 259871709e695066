"""Micro-benchmarks of the hot kernels against the measured roofline denominators.

Usage:  python benchmarks/bench_kernels.py [--which gemm,gemm_small,gemm_mid,attn,norm] [--out FILE]

Timing: CUDA events on the launching stream, 5 warm-up launches, an L2 flush (a 256 MB
memset) before every timed launch, median of the timed launches. Fractions are reported
against ``MEASURED_PEAKS.json`` when present ("of measured"), else against the stated
fallback figures ("of fallback").
"""

from __future__ import annotations

import argparse
import json
import math
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from parallax_b200.ops import cuda as cu  # noqa: E402
from parallax_b200.ops import reference as ref  # noqa: E402


def peaks():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return p["hbm_gbs"], p["bf16_tflops"], "of measured"
    return 6650.0, 1590.0, "of fallback"


_flush = None


def time_fn(fn, iters=10, warmup=5):
    global _flush
    if _flush is None:
        _flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        _flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e))
    ts.sort()
    return ts[len(ts) // 2]


def bench_gemm(rows):
    hbm, tf, tag = peaks()
    shapes = [
        (2560, 6144, 4096), (2560, 4096, 4096), (2560, 24576, 4096), (2560, 4096, 12288),
        (512, 6144, 4096), (512, 24576, 4096), (512, 4096, 12288),
        (8192, 8192, 8192), (4096, 151936, 4096), (64, 4096, 4096),
    ]
    for M, N, K in shapes:
        x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.02
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        flops = 2.0 * M * N * K
        byts = 2.0 * (M * K + N * K + M * N)
        best, per_bn = None, {}
        for bn in (64, 128, 192, 256):
            ms = time_fn(lambda: cu.linear(x, w, out=out, bn=bn))
            per_bn[bn] = round(ms, 4)
            if best is None or ms < best[1]:
                best = (bn, ms)
        picked = cu.gemm_pick_bn(M, N)
        ms_lib = time_fn(lambda: torch.matmul(x, w.t(), out=out))
        cu.check_status(x.device)
        bn, ms = best
        ideal = max(flops / (tf * 1e12), byts / (hbm * 1e9)) * 1e3
        rows.append({
            "kernel": "gemm_bf16_tcgen05", "M": M, "N": N, "K": K, "bn": bn, "ms": round(ms, 4), "ms_per_bn": per_bn,
            "bn_picked": picked,
            "tflops": round(flops / ms / 1e9, 1), "roofline_frac": round(ideal / ms, 3),
            "tag": tag, "torch_matmul_ms": round(ms_lib, 4),
        })
        print(rows[-1], flush=True)
        del x, w, out


def bench_gemm_small(rows):
    """Decode-sized GEMMs (M <= 128): memory-bound, so the figure of merit is weight bytes per second.
    Eight weight matrices are cycled so that no launch finds its weights in L2; the launches of one
    variant run back to back between one pair of events (a short kernel timed alone would mostly
    measure the launch)."""
    hbm, _tf, tag = peaks()
    reps = 8
    for M in (8, 64, 128):
        for N, K in [(4096, 4096), (6144, 4096), (4096, 12288)]:
            x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
            ws = [torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.02 for _ in range(reps)]
            out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)

            def run(fn):
                for w in ws:
                    fn(w)
                torch.cuda.synchronize()
                s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s.record()
                for _ in range(4):
                    for w in ws:
                        fn(w)
                e.record()
                torch.cuda.synchronize()
                return s.elapsed_time(e) / (4 * reps)

            ms_small = run(lambda w: cu.linear_small_m(x, w, out=out))
            ms_scratch = run(lambda w: cu.linear_small_m(x, w, out=out, mode=1))
            ms_cluster = run(lambda w: cu.linear_small_m(x, w, out=out, mode=2))
            ms_tile = min(run(lambda w: cu.linear(x, w, out=out, bn=64)), run(lambda w: cu.linear(x, w, out=out, bn=128)))
            ms_lib = run(lambda w: torch.matmul(x, w.t(), out=out))
            cu.check_status(x.device)
            byts = 2.0 * N * K
            rows.append({"kernel": "gemm_bf16_small_m", "M": M, "N": N, "K": K, "us": round(ms_small * 1e3, 2),
                         "us_scratch": round(ms_scratch * 1e3, 2), "us_cluster": round(ms_cluster * 1e3, 2),
                         "us_plain_tiles": round(ms_tile * 1e3, 2), "us_torch_matmul": round(ms_lib * 1e3, 2),
                         "weight_gbs": round(byts / ms_small / 1e6, 1),
                         "roofline_frac": round(byts / (hbm * 1e9) * 1e3 / ms_small, 3), "tag": tag})
            print(rows[-1], flush=True)
            del ws


def bench_gemm_mid(rows):
    """Pipeline-stage micro-batches (129 to 512 rows): both weight streaming and tensor throughput matter.
    Eight weight matrices are cycled so that no launch finds its weights in L2; launches run back to
    back between one pair of events."""
    hbm, tf, tag = peaks()
    reps = 8
    for M in (192, 320, 512):
        for N, K in [(6144, 4096), (4096, 4096), (24576, 4096), (4096, 12288)]:
            x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
            ws = [torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.02 for _ in range(reps)]
            out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)

            def run(fn):
                for w in ws:
                    fn(w)
                torch.cuda.synchronize()
                s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s.record()
                for _ in range(4):
                    for w in ws:
                        fn(w)
                e.record()
                torch.cuda.synchronize()
                return s.elapsed_time(e) / (4 * reps)

            ms_auto = run(lambda w: cu.linear(x, w, out=out))
            ms_plain = min(run(lambda w: cu.linear(x, w, out=out, bn=128)), run(lambda w: cu.linear(x, w, out=out, bn=256)))
            ms_lib = run(lambda w: torch.matmul(x, w.t(), out=out))
            sweep = {}
            for bn in (128, 256):
                for sk in (2, 3, 4, 6, 8):
                    if (K // 64) // sk < 4:
                        continue
                    sweep[f"{bn}x{sk}"] = round(run(lambda w: cu.linear_mid_m(x, w, bn=bn, splitk=sk, out=out)) * 1e3, 2)
            cu.check_status(x.device)
            flops = 2.0 * M * N * K
            byts = 2.0 * (M * K + N * K + M * N)
            ideal = max(flops / (tf * 1e12), byts / (hbm * 1e9)) * 1e3
            rows.append({"kernel": "gemm_bf16_mid_m", "M": M, "N": N, "K": K, "plan_bn_splitk": cu.gemm_mid_m_plan(M, N, K),
                         "us_cluster_bn_x_splitk": sweep,
                         "us": round(ms_auto * 1e3, 2), "us_plain_tiles": round(ms_plain * 1e3, 2),
                         "us_torch_matmul": round(ms_lib * 1e3, 2), "vs_torch": round(ms_lib / ms_auto, 3),
                         "roofline_frac": round(ideal / ms_auto, 3), "tag": tag})
            print(rows[-1], flush=True)
            del ws


def bench_attn(rows):
    hbm, tf, tag = peaks()
    Hq, Hkv, D, page = 32, 8, 128, 16
    for B, ctx in [(512, 1152), (64, 1152), (8, 32768), (256, 4096)]:
        nb = (ctx + page - 1) // page
        total = B * nb
        kc = torch.randn(total, Hkv, page, D, device="cuda", dtype=torch.bfloat16)
        vc = torch.randn(total, Hkv, page, D, device="cuda", dtype=torch.bfloat16)
        bt = torch.randperm(total, device="cuda").to(torch.int32).view(B, nb)
        cl = torch.full((B,), ctx, dtype=torch.int32, device="cuda")
        q = torch.randn(B, Hq, D, device="cuda", dtype=torch.bfloat16)
        out = torch.empty_like(q)
        sc = 1.0 / math.sqrt(D)
        ms = time_fn(lambda: cu.attn_decode(q, kc, vc, bt, cl, sc, max_ctx=ctx, out=out))
        byts = 2.0 * B * ctx * Hkv * D * 2
        rows.append({"kernel": "attn_decode", "B": B, "ctx": ctx, "ms": round(ms, 4),
                     "gbs": round(byts / ms / 1e6, 1), "roofline_frac": round(byts / (hbm * 1e9) * 1e3 / ms, 3),
                     "tag": tag})
        print(rows[-1], flush=True)
        del kc, vc
    for B, L, prefix in [(2, 1024, 0), (8, 1024, 0), (1, 8192, 0), (1, 8192, 24576)]:
        ctx = L + prefix
        nb = (ctx + page - 1) // page
        total = B * nb
        kc = torch.randn(total, Hkv, page, D, device="cuda", dtype=torch.bfloat16)
        vc = torch.randn(total, Hkv, page, D, device="cuda", dtype=torch.bfloat16)
        bt = torch.randperm(total, device="cuda").to(torch.int32).view(B, nb)
        cl = torch.full((B,), ctx, dtype=torch.int32, device="cuda")
        cu_q = (torch.arange(B + 1, device="cuda") * L).to(torch.int32)
        q = torch.randn(B * L, Hq, D, device="cuda", dtype=torch.bfloat16)
        out = torch.empty_like(q)
        sc = 1.0 / math.sqrt(D)
        ms = time_fn(lambda: cu.attn_prefill(q, kc, vc, bt, cu_q, cl, L, sc, out=out), iters=5)
        flops = 4.0 * B * Hq * D * (L * prefix + L * (L + 1) / 2)
        rows.append({"kernel": "attn_prefill", "B": B, "L": L, "prefix": prefix, "ms": round(ms, 4),
                     "tflops": round(flops / ms / 1e9, 1),
                     "roofline_frac": round(flops / (tf * 1e12) * 1e3 / ms, 3), "tag": tag})
        print(rows[-1], flush=True)
        del kc, vc


def bench_attn_small(rows):
    """Decode attention at pipeline micro-batch sizes (tens of sequences): how the split-KV factor trades
    a fuller machine against the extra partial results. Context lengths vary per sequence as in serving."""
    hbm, _tf, tag = peaks()
    Hq, Hkv, D, page = 32, 8, 128, 16
    for B in (57, 102, 128, 256):
        ctx_max = 1280
        nb = (ctx_max + page - 1) // page
        total = B * nb
        kc = torch.randn(total, Hkv, page, D, device="cuda", dtype=torch.bfloat16)
        vc = torch.randn(total, Hkv, page, D, device="cuda", dtype=torch.bfloat16)
        bt = torch.randperm(total, device="cuda").to(torch.int32).view(B, nb)
        cl = torch.randint(1024, ctx_max + 1, (B,), device="cuda").to(torch.int32)
        q = torch.randn(B, Hq, D, device="cuda", dtype=torch.bfloat16)
        out = torch.empty_like(q)
        sc = 1.0 / math.sqrt(D)
        byts = 2.0 * float(cl.sum()) * Hkv * D * 2
        per = {}
        for s in (0, 1, 2, 3, 4, 6):
            ms = time_fn(lambda: cu.attn_decode(q, kc, vc, bt, cl, sc, max_ctx=ctx_max, num_splits=s, out=out))
            per["auto" if s == 0 else s] = round(ms * 1e3, 1)
        best = min(per.values())
        rows.append({"kernel": "attn_decode (micro-batch sizes)", "B": B, "ctx": "1024..1280", "us_per_splits": per,
                     "ideal_us": round(byts / (hbm * 1e9) * 1e6, 1), "best_frac": round(byts / (hbm * 1e9) * 1e6 / best, 3),
                     "auto_frac": round(byts / (hbm * 1e9) * 1e6 / per["auto"], 3), "tag": tag})
        print(rows[-1], flush=True)
        del kc, vc


def bench_norm(rows):
    hbm, tf, tag = peaks()
    T, H = 65536, 4096
    x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(H, device="cuda", dtype=torch.bfloat16)
    out = torch.empty_like(x)
    ms = time_fn(lambda: cu.rmsnorm(x, w, 1e-6, out=out))
    byts = 2.0 * T * H * 2
    rows.append({"kernel": "rmsnorm", "T": T, "H": H, "ms": round(ms, 4), "gbs": round(byts / ms / 1e6, 1),
                 "roofline_frac": round(byts / (hbm * 1e9) * 1e3 / ms, 3), "tag": tag})
    print(rows[-1], flush=True)
    # engine-sized launches (one step of the headline workload has about 2500 rows)
    T = 2560
    x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    out = torch.empty_like(x)
    ms = time_fn(lambda: cu.rmsnorm(x, w, 1e-6, out=out))
    byts = 2.0 * T * H * 2
    rows.append({"kernel": "rmsnorm", "T": T, "H": H, "ms": round(ms, 4), "gbs": round(byts / ms / 1e6, 1),
                 "roofline_frac": round(byts / (hbm * 1e9) * 1e3 / ms, 3), "tag": tag})
    print(rows[-1], flush=True)
    Hq, Hkv, D, page = 32, 8, 128, 16
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device="cuda", dtype=torch.bfloat16)
    qn = torch.randn(D, device="cuda", dtype=torch.bfloat16)
    kn = torch.randn(D, device="cuda", dtype=torch.bfloat16)
    cs = ref.build_cos_sin(4096, D, 1e6, device="cuda")
    pos = torch.randint(0, 4096, (T,), device="cuda", dtype=torch.int32)
    blocks = 4096
    slots = torch.randperm(blocks * page, device="cuda")[:T].to(torch.int64)
    kc = torch.zeros(blocks, Hkv, page, D, device="cuda", dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    ms = time_fn(lambda: cu.qk_norm_rope_cache(qkv, qn, kn, cs, pos, slots, kc, vc, Hq, Hkv, D, D))
    byts = 2.0 * T * D * ((Hq + Hkv) * 2 + Hkv + 2 * Hkv)   # q, k read + written, v read, k and v cache writes
    rows.append({"kernel": "qk_norm_rope_cache", "T": T, "ms": round(ms, 4), "gbs": round(byts / ms / 1e6, 1),
                 "roofline_frac": round(byts / (hbm * 1e9) * 1e3 / ms, 3), "tag": tag})
    print(rows[-1], flush=True)
    logits = torch.randn(512, 151936, device="cuda").to(torch.bfloat16)
    ms = time_fn(lambda: cu.argmax(logits))
    byts = logits.numel() * 2.0
    rows.append({"kernel": "argmax", "B": 512, "V": 151936, "ms": round(ms, 4),
                 "gbs": round(byts / ms / 1e6, 1), "roofline_frac": round(byts / (hbm * 1e9) * 1e3 / ms, 3),
                 "tag": tag})
    print(rows[-1], flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--which", default="gemm,gemm_small,gemm_mid,attn,norm")
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    rows = []
    which = args.which.split(",")
    if "gemm" in which:
        bench_gemm(rows)
    if "gemm_small" in which:
        bench_gemm_small(rows)
    if "gemm_mid" in which:
        bench_gemm_mid(rows)
    if "attn" in which:
        bench_attn(rows)
    if "attn_small" in which:
        bench_attn_small(rows)
    if "norm" in which:
        bench_norm(rows)
    if args.out:
        os.makedirs(os.path.dirname(args.out) or ".", exist_ok=True)
        with open(args.out, "w") as f:
            json.dump(rows, f, indent=1)


if __name__ == "__main__":
    main()
