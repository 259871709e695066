"""sm_100a gated-delta-net kernels against the fp32 PyTorch restatement, and the hybrid engine."""

import pytest
import torch

from parallax_b200.models.config import named_config
from parallax_b200.ops import reference as ref

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return float((a.float().cpu() - b.float().cpu()).norm() / (b.float().cpu().norm() + 1e-12))


def test_conv_delta_rule_and_gate_kernels():
    from parallax_b200.ops import cuda as cu

    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    Hk, Hv, Dk, Dv, K = 2, 4, 128, 128, 4
    C = 2 * Hk * Dk + Hv * Dv
    lens = [37, 1, 1, 64]                       # two prefill chunks (one continuing), two decode rows
    starts = [0, 12, 99, 32]
    T = sum(lens)
    seq_cu = torch.tensor([0, 37, 38, 39, 103], dtype=torch.int32)
    seq_slots = torch.tensor([5, 2, 7, 0], dtype=torch.int32)
    positions = torch.cat([torch.arange(s, s + n) for s, n in zip(starts, lens)]).int()
    proj = (torch.randn(T, C + Hv * Dv + 2 * Hv) * 0.5).to(torch.bfloat16)
    conv_w = (torch.randn(C, K) * 0.3).to(torch.bfloat16)
    conv_state = (torch.randn(8, C, K - 1) * 0.5).to(torch.bfloat16)
    rec_state = torch.randn(8, Hv, Dv, Dk) * 0.1
    A_log = torch.log(torch.linspace(1, 8, Hv))
    dt_bias = torch.linspace(-1, 1, Hv)
    norm_w = (torch.rand(Dv) + 0.5).to(torch.bfloat16)

    def run(mod, to):
        p, cs, rs = to(proj), to(conv_state.clone()), to(rec_state.clone())
        conv = mod.causal_conv1d_silu(p[:, :C], to(conv_w), None, cs, to(seq_cu), to(seq_slots), to(positions))
        z = p[:, C:C + Hv * Dv]
        b = p[:, C + Hv * Dv:C + Hv * Dv + Hv]
        a = p[:, C + Hv * Dv + Hv:]
        out = mod.gated_delta_rule(conv, a, b, to(A_log), to(dt_bias), z, to(norm_w), rs, to(seq_cu), to(seq_slots),
                                   to(positions), Hk, Hv, Dk, Dv, 1e-6)
        gated = mod.sigmoid_gate_mul(out, z)
        return conv, cs, out, rs, gated

    want = run(ref, lambda x: x)
    got = run(cu, lambda x: x.to(dev))
    torch.cuda.synchronize()
    for name, g, w in zip(["conv", "conv_state", "delta_out", "rec_state", "gate_mul"], got, want):
        assert _rel(g, w) < 2e-2, (name, _rel(g, w))


def test_hybrid_engine_gpu_matches_cpu():
    from parallax_b200.engine.engine import Engine
    from parallax_b200.engine.request import Request, SamplingParams
    from parallax_b200.ops import cuda as cu

    cfg = named_config("small-hybrid")
    kw = dict(num_blocks=128, page_size=16, max_batch_size=4, max_num_tokens_per_batch=512, chunked_prefill_size=96,
              max_total_length=512, seed=0)
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (150, 20, 97)]

    def conv(t):
        return t.detach().cpu().float() if t.dtype == torch.bfloat16 else t.detach().cpu()

    def run(device, dtype, src=None):
        eng = Engine(cfg, device=device, dtype=dtype, **kw)
        m = eng.stages[0].model
        if src is not None:
            for name in ("embed", "norm_w", "lm_head"):
                setattr(m, name, conv(getattr(src, name)))
            for ls, ld in zip(src.layers, m.layers):
                for cls in type(ls).__mro__:
                    for slot in getattr(cls, "__slots__", ()):
                        v = getattr(ls, slot, None)
                        if isinstance(v, torch.Tensor):
                            setattr(ld, slot, conv(v))
        eng.keep_logits = True
        for p in prompts:
            eng.add_request(Request(input_ids=p, sampling_params=SamplingParams(max_new_tokens=3, temperature=0.0,
                                                                               ignore_eos=True), max_total_length=512))
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
