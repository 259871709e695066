"""sm_100a block-sparse indexer kernels against the PyTorch restatement, and the MSA engine."""

import pytest
import torch

from parallax_b200.models.config import named_config
from parallax_b200.ops import reference as ref

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return float((a.float().cpu() - b.float().cpu()).norm() / (b.float().cpu().norm() + 1e-12))


def test_block_scores_and_selection():
    from parallax_b200.ops import cuda as cu

    dev = torch.device("cuda", 0)
    torch.manual_seed(1)
    T, Hi, Di, page, sb = 6, 4, 128, 16, 128
    cache = (torch.randn(128, 1, page, Di) * 0.5).to(torch.bfloat16)
    bt = torch.randperm(128)[:120].int().view(3, 40)                 # 3 sequences, up to 640 tokens
    cu_q = torch.tensor([0, 2, 3, 6], dtype=torch.int32)
    pos = torch.tensor([600, 601, 5, 300, 301, 302], dtype=torch.int32)
    iq = (torch.randn(T, Hi, Di) * 0.5).to(torch.bfloat16)
    want = ref.msa_block_scores(iq, cache, bt, cu_q, pos, 640, sb, 0.088)
    got = cu.msa_block_scores(iq.to(dev), cache.to(dev), bt.to(dev), cu_q.to(dev), pos.to(dev), 640, sb, 0.088).cpu()
    fin = torch.isfinite(want)
    assert torch.equal(torch.isfinite(got), fin) and _rel(got[fin], want[fin]) < 1e-2
    vt_w, vc_w = ref.msa_select(got, pos, bt, cu_q, page, sb, 3, 1, 1)
    vt_g, vc_g = cu.msa_select(got.to(dev), pos.to(dev), bt.to(dev), cu_q.to(dev), page, sb, 3, 1, 1)
    assert torch.equal(vc_g.cpu(), vc_w) and torch.equal(vt_g.cpu(), vt_w)


def test_msa_engine_gpu_matches_cpu():
    from parallax_b200.engine.engine import Engine
    from parallax_b200.engine.request import Request, SamplingParams
    from parallax_b200.ops import cuda as cu

    cfg = named_config("small-msa")           # 128-token blocks, top-3
    kw = dict(num_blocks=128, page_size=16, max_batch_size=4, max_num_tokens_per_batch=1024, chunked_prefill_size=256,
              max_total_length=1024, seed=0)
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (700, 20, 450)]

    def conv(t):
        return t.detach().cpu().float() if t.dtype == torch.bfloat16 else t.detach().cpu()

    def run(device, dtype, src=None):
        eng = Engine(cfg, device=device, dtype=dtype, **kw)
        m = eng.stages[0].model
        if src is not None:
            for name in ("embed", "norm_w", "lm_head"):
                setattr(m, name, conv(getattr(src, name)))
            for ls, ld in zip(src.layers, m.layers):
                for slot in type(ls).__slots__:
                    v = getattr(ls, slot, None)
                    if isinstance(v, torch.Tensor):
                        setattr(ld, slot, conv(v))
            m.idx = {k: {n: conv(t) for n, t in d.items()} for k, d in src.idx.items()}
        eng.keep_logits = True
        for p in prompts:
            eng.add_request(Request(input_ids=p, sampling_params=SamplingParams(max_new_tokens=3, temperature=0.0,
                                                                               ignore_eos=True), max_total_length=1024))
        outs = []
        while eng.has_work():
            eng.step()
            if eng.last_logits is not None and eng.last_logits.shape[0] > 0:
                outs.append(eng.last_logits.float().cpu().clone())
            eng.last_logits = None
        return m, outs

    gm, got = run("cuda:0", torch.bfloat16)
    _, want = run("cpu", torch.float32, src=gm)
    cu.check_status(torch.device("cuda", 0))
    assert len(want) == len(got) and all(a.shape == b.shape for a, b in zip(got, want))
    assert _rel(got[0], want[0]) < 6e-2, _rel(got[0], want[0])
