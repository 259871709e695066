"""Block-scaled e4m3 tcgen05 GEMM against the fp32 restatement of the same quantised contraction."""

import pytest
import torch

from parallax_b200.loader.quant import quantize_fp8_block
from parallax_b200.ops import reference as ref

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return float((a.float().cpu() - b.float().cpu()).norm() / (b.float().cpu().norm() + 1e-12))


def _weights(N, K, seed):
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(N, K, generator=g) * 0.05
    wq, ws = quantize_fp8_block(w)
    return wq, ws.repeat_interleave(2, dim=0).contiguous()


@pytest.mark.parametrize("T,N,K", [(1, 256, 512), (200, 1024, 7168), (777, 2048, 1536)])
def test_fp8_dense(T, N, K):
    from parallax_b200.ops import cuda as cu

    dev = torch.device("cuda", 0)
    wq, ws64 = _weights(N, K, 1)
    x = (torch.randn(T, K) * 0.7).to(torch.bfloat16)
    xq, xs = cu.quant_fp8_rows(x.to(dev))
    rq, rs = ref.quant_fp8_rows(x)
    assert _rel(xs, rs) < 1e-3
    assert _rel(xq.float(), rq.float()) < 2e-2       # rounding of exact ties may differ by one code
    res = torch.randn(T, N).to(torch.bfloat16)
    for epi, r in ((ref.EPI_NONE, None), (ref.EPI_NONE, res), (ref.EPI_SILU_MUL, None)):
        want = ref.linear_fp8(x, wq, ws64, residual=r, epi=epi)
        got = cu.linear_fp8(x.to(dev), wq.to(dev), ws64.to(dev), residual=None if r is None else r.to(dev), epi=epi)
        torch.cuda.synchronize()
        assert got.shape == want.shape and _rel(got, want) < 2e-2, (epi, _rel(got, want))
    cu.check_status(dev)


def test_fp8_grouped_experts():
    from parallax_b200.ops import cuda as cu

    dev = torch.device("cuda", 0)
    E, N, K, T, k = 8, 256, 512, 300, 2
    g = torch.Generator().manual_seed(3)
    ids = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).int()
    plan = cu.moe_align(ids.to(dev), E)
    x = (torch.randn(T, K, generator=g) * 0.5).to(torch.bfloat16)
    xp = cu.moe_gather(x.to(dev), plan)
    ws, ss = zip(*[_weights(N, K, 10 + e) for e in range(E)])
    wq, ws64 = torch.cat(ws), torch.cat(ss)
    got = cu.grouped_linear_fp8(xp, wq.to(dev), ws64.to(dev), plan, E).cpu()
    torch.cuda.synchronize()
    cu.check_status(dev)
    offsets = plan.offsets.cpu().tolist()
    xp_c = xp.cpu()
    for e in range(E):
        lo, hi = offsets[e], offsets[e + 1]
        if hi > lo:
            want = ref.linear_fp8(xp_c[lo:hi], ws[e], ss[e])
            assert _rel(got[lo:hi], want) < 2e-2, e
