"""Small, self-terminating cases for `ncu` captures (one kernel, a few launches, < 2 GB).

    python benchmarks/profile_case.py gemm         # bf16 tcgen05 GEMM, 4096 x 8192 x 8192
    python benchmarks/profile_case.py gemm_small   # split-K small-M GEMM, 64 x 4096 x 4096
    python benchmarks/profile_case.py gemm_mid     # mid-M cluster split-K GEMM, 320 x 4096 x 12288
    python benchmarks/profile_case.py attn_decode  # paged GQA decode, 256 seqs x 2048 ctx
    python benchmarks/profile_case.py attn_prefill # ragged prefill, 4 x 2048
    python benchmarks/profile_case.py step         # 2 engine steps of a 4-layer Qwen3-8B-shaped
                                                   # model at 64 concurrent (launch list)
    python benchmarks/profile_case.py decode_step  # same, decode rows only (small-M GEMMs); decode_step_8: 8 rows

Each case uses inputs larger than the 126 MB L2 so that DRAM counters are meaningful, warms
up once, and brackets the launches of interest with cudaProfilerStart/Stop so that
`ncu --profile-from-start off` sees only those.
"""

from __future__ import annotations

import math
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from parallax_b200.ops import cuda as cu  # noqa: E402


def case_gemm(iters: int = 3):
    M, N, K = 4096, 8192, 8192
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.02
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    cu.linear(x, w, out=out, bn=256)
    torch.cuda.synchronize()
    torch.cuda.cudart().cudaProfilerStart()
    for _ in range(iters):
        cu.linear(x, w, out=out, bn=256)
    torch.cuda.synchronize()
    torch.cuda.cudart().cudaProfilerStop()
    cu.check_status(x.device)


def case_gemm_small(iters: int = 3, M: int = 64, N: int = 4096, K: int = 4096):
    """Decode-sized GEMM on the split-K path; a fresh weight matrix per launch (8 x 33 MB > L2)."""
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    ws = [torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.02 for _ in range(8)]
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    for w in ws:
        cu.linear_small_m(x, w, out=out)
    torch.cuda.synchronize()
    torch.cuda.cudart().cudaProfilerStart()
    for i in range(iters):
        cu.linear_small_m(x, ws[i % 8], out=out)
    torch.cuda.synchronize()
    torch.cuda.cudart().cudaProfilerStop()
    cu.check_status(x.device)


def case_gemm_mid(iters: int = 3, M: int = 320, N: int = 4096, K: int = 12288):
    """Pipeline-stage micro-batch GEMM on the cluster split-K path (what ``linear`` picks for this shape);
    a fresh weight matrix per launch (8 x 100 MB > L2)."""
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    ws = [torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.02 for _ in range(8)]
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    print("plan (tile width, K ranges):", cu.gemm_mid_m_plan(M, N, K))
    for w in ws:
        cu.linear(x, w, out=out)
    torch.cuda.synchronize()
    torch.cuda.cudart().cudaProfilerStart()
    for i in range(iters):
        cu.linear(x, ws[i % 8], out=out)
    torch.cuda.synchronize()
    torch.cuda.cudart().cudaProfilerStop()
    cu.check_status(x.device)


def _paged(B, ctx, Hkv=8, D=128, page=16):
    nb = (ctx + page - 1) // page
    total = B * nb
    kc = torch.randn(total, Hkv, page, D, device="cuda", dtype=torch.bfloat16)
    vc = torch.randn(total, Hkv, page, D, device="cuda", dtype=torch.bfloat16)
    bt = torch.randperm(total, device="cuda").to(torch.int32).view(B, nb)
    cl = torch.full((B,), ctx, dtype=torch.int32, device="cuda")
    return kc, vc, bt, cl


def case_attn_decode(iters: int = 3):
    B, ctx, Hq, D = 256, 2048, 32, 128
    kc, vc, bt, cl = _paged(B, ctx)
    q = torch.randn(B, Hq, D, device="cuda", dtype=torch.bfloat16)
    out = torch.empty_like(q)
    sc = 1.0 / math.sqrt(D)
    cu.attn_decode(q, kc, vc, bt, cl, sc, max_ctx=ctx, out=out)
    torch.cuda.synchronize()
    torch.cuda.cudart().cudaProfilerStart()
    for _ in range(iters):
        cu.attn_decode(q, kc, vc, bt, cl, sc, max_ctx=ctx, out=out)
    torch.cuda.synchronize()
    torch.cuda.cudart().cudaProfilerStop()
    cu.check_status(q.device)


def case_attn_prefill(iters: int = 3):
    B, L, Hq, D = 4, 2048, 32, 128
    kc, vc, bt, cl = _paged(B, L)
    q = torch.randn(B * L, Hq, D, device="cuda", dtype=torch.bfloat16)
    cu_q = (torch.arange(B + 1, device="cuda") * L).to(torch.int32)
    out = torch.empty_like(q)
    sc = 1.0 / math.sqrt(D)
    cu.attn_prefill(q, kc, vc, bt, cu_q, cl, L, sc, out=out)
    torch.cuda.synchronize()
    torch.cuda.cudart().cudaProfilerStart()
    for _ in range(iters):
        cu.attn_prefill(q, kc, vc, bt, cu_q, cl, L, sc, out=out)
    torch.cuda.synchronize()
    torch.cuda.cudart().cudaProfilerStop()
    cu.check_status(q.device)


def case_step(steps: int = 2, conc: int = 64, with_prefill: bool = True):
    from parallax_b200.engine.engine import Engine
    from parallax_b200.engine.request import Request, SamplingParams
    from parallax_b200.models.config import named_config

    cfg = named_config("qwen3-8b")
    cfg.num_hidden_layers = 4
    eng = Engine(cfg, device="cuda:0", max_batch_size=conc, max_num_tokens_per_batch=4096 + conc,
                 chunked_prefill_size=2048, max_total_length=1400, max_kv_tokens=conc * 1400,
                 request_timeout_s=None)
    g = torch.Generator().manual_seed(0)

    def admit(n_in, n_out):
        eng.add_request(Request(input_ids=torch.randint(0, cfg.vocab_size, (n_in,), generator=g).tolist(),
                                sampling_params=SamplingParams(max_new_tokens=n_out, temperature=0.0,
                                                               ignore_eos=True)))

    for i in range(conc):
        admit(1024 + (i * 4) % 256, 256 - (i * 4) % 256)
    eng.step()                                     # admits and starts prefilling
    for _ in range(40):
        if not any(r.is_prefill for r in eng.scheduler.running_requests()):
            break
        eng.step()
    if with_prefill:
        admit(1024, 256)                           # one prompt joins the decode batch in the captured steps
    torch.cuda.synchronize()
    torch.cuda.cudart().cudaProfilerStart()
    for _ in range(steps):
        eng.step()
    torch.cuda.synchronize()
    torch.cuda.cudart().cudaProfilerStop()
    cu.check_status(torch.device("cuda:0"))


if __name__ == "__main__":
    which = sys.argv[1] if len(sys.argv) > 1 else "gemm"
    {"gemm": case_gemm, "attn_decode": case_attn_decode, "attn_prefill": case_attn_prefill,
     "gemm_small": case_gemm_small, "gemm_mid": case_gemm_mid, "step": case_step, "decode_step": lambda: case_step(conc=64, with_prefill=False),
     "decode_step_8": lambda: case_step(conc=8, with_prefill=False)}[which]()
    print(f"profile case {which}: ok")
