"""MoE kernels on B200 against the fp32 restatement: routing modes, grouped GEMM pipeline, engine."""

import pytest
import torch

from parallax_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def cu():
    from parallax_b200.ops import cuda

    return cuda


def _rel(a, b):
    return float((a.float() - b.float()).norm() / (b.float().norm() + 1e-12))


@pytest.mark.parametrize("E,k,mode,n_group,topk_group,bias,bf16", [
    (128, 8, 0, 1, 1, False, False),
    (8, 2, 0, 1, 1, False, True),
    (256, 8, 1, 8, 4, True, False),
    (64, 6, 1, 1, 1, True, False),
    (160, 4, 0, 1, 1, False, False),
])
def test_moe_route(cu, E, k, mode, n_group, topk_group, bias, bf16):
    torch.manual_seed(0)
    T = 77
    logits = torch.randn(T, E, device=DEV) * 2
    if bf16:
        logits = logits.bfloat16()
    e_bias = torch.randn(E, device=DEV) * 0.1 if bias else None
    ids, w = cu.moe_route(logits, e_bias, k, mode, True, n_group, topk_group, 2.5)
    rids, rw = ref.moe_route(logits, e_bias, k, mode, True, n_group, topk_group, 2.5)
    # same expert SETS and matching weights per expert
    assert torch.equal(ids.sort(-1).values, rids.sort(-1).values)
    dense = torch.zeros(T, E, device=DEV).scatter_(1, ids.long(), w)
    rdense = torch.zeros(T, E, device=DEV).scatter_(1, rids.long(), rw)
    assert torch.allclose(dense, rdense, atol=2e-3, rtol=2e-3)


@pytest.mark.parametrize("T,E,k,H,I", [(300, 8, 2, 256, 128), (1000, 128, 8, 2048, 768), (5, 16, 4, 512, 256)])
def test_moe_ffn(cu, T, E, k, H, I):
    torch.manual_seed(1)
    x = torch.randn(T, H, device=DEV, dtype=torch.bfloat16)
    base = torch.randn(T, H, device=DEV, dtype=torch.bfloat16)
    g = torch.randn(E, I, H, device=DEV, dtype=torch.bfloat16) * 0.05
    u = torch.randn(E, I, H, device=DEV, dtype=torch.bfloat16) * 0.05
    w1 = torch.stack([ref.interleave_gate_up(g[e], u[e]) for e in range(E)]).view(E * 2 * I, H).contiguous()
    w2 = (torch.randn(E * H, I, device=DEV, dtype=torch.bfloat16) * 0.05)
    logits = torch.randn(T, E, device=DEV)
    ids, w = cu.moe_route(logits, None, k)
    got = cu.moe_ffn(x, ids, w, w1, w2, E, base=base)
    want = ref.moe_ffn(x, ids, w, w1, w2, E, base=base)
    torch.cuda.synchronize()
    cu.check_status(torch.device(DEV))
    assert _rel(got, want) < 1e-2
    # skewed routing: every token to the same two experts (one expert gets many m-tiles)
    ids2 = torch.zeros_like(ids)
    ids2[:, 1:] = torch.arange(1, k, device=DEV, dtype=torch.int32)
    got2 = cu.moe_ffn(x, ids2, w, w1, w2, E, base=None)
    want2 = ref.moe_ffn(x, ids2, w, w1, w2, E, base=None)
    assert _rel(got2, want2) < 1e-2
    cu.check_status(torch.device(DEV))


def test_moe_engine_gpu_matches_cpu():
    from parallax_b200.engine.engine import Engine
    from parallax_b200.engine.request import Request, SamplingParams
    from parallax_b200.models.config import config_from_hf

    cfg = config_from_hf(dict(architectures=["Qwen3MoeForCausalLM"], model_type="qwen3_moe", hidden_size=512,
                              num_hidden_layers=2, num_attention_heads=8, num_key_value_heads=2, head_dim=64,
                              intermediate_size=1024, moe_intermediate_size=256, num_experts=16,
                              num_experts_per_tok=4, norm_topk_prob=True, vocab_size=2048, rope_theta=1e4))
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, 2048, (40,), generator=g).tolist() for _ in range(4)]

    def first_logits(device, dtype, seed_engine=None):
        eng = Engine(cfg, device=device, dtype=dtype, num_blocks=64, max_batch_size=8)
        if seed_engine is not None:   # copy the GPU engine's (bf16-rounded) weights
            src, dst = seed_engine.stages[0].model, eng.stages[0].model
            for name in ("embed", "norm_w", "lm_head"):
                setattr(dst, name, getattr(src, name).float().cpu())
            for ls, ld in zip(src.layers, dst.layers):
                for slot in ("ln1", "ln2", "w_qkv", "q_norm", "k_norm", "w_o"):
                    setattr(ld, slot, getattr(ls, slot).float().cpu())
                for slot in ("router", "w1", "w2"):
                    setattr(ld.moe, slot, getattr(ls.moe, slot).float().cpu())
        eng.keep_logits = True
        for p in prompts:
            eng.add_request(Request(input_ids=p, sampling_params=SamplingParams(max_new_tokens=2, temperature=0.0,
                                                                                ignore_eos=True)))
        eng.step()
        return eng, eng.last_logits.float().cpu()

    gpu, lg = first_logits(DEV, torch.bfloat16)
    _, lc = first_logits("cpu", torch.float32, gpu)
    assert _rel(lg, lc) < 5e-2


def test_moe_ffn_swigluoai_with_expert_biases(cu):
    """Clipped swigluoai experts (GPT-OSS / MiniMax-M3): plain [gate | up] rows, biases per expert."""
    torch.manual_seed(4)
    T, E, k, H, I = 333, 8, 2, 512, 256
    x = torch.randn(T, H, device=DEV, dtype=torch.bfloat16)
    base = torch.randn(T, H, device=DEV, dtype=torch.bfloat16)
    w1 = (torch.randn(E * 2 * I, H, device=DEV) * 0.05).to(torch.bfloat16)
    w2 = (torch.randn(E * H, I, device=DEV) * 0.05).to(torch.bfloat16)
    b1 = (torch.randn(E * 2 * I, device=DEV) * 0.5).to(torch.bfloat16)
    b2 = (torch.randn(E * H, device=DEV) * 0.5).to(torch.bfloat16)
    ids = torch.stack([torch.randperm(E, device=DEV)[:k] for _ in range(T)]).int()
    w = torch.rand(T, k, device=DEV)
    got = cu.moe_ffn(x, ids, w, w1, w2, E, base=base, act_mode=1, limit=7.0, b1=b1, b2=b2)
    want = ref.moe_ffn(x.cpu(), ids.cpu(), w.cpu(), w1.cpu().float(), w2.cpu().float(), E, base=base.cpu(), act_mode=1,
                       limit=7.0, b1=b1.cpu().float(), b2=b2.cpu().float())
    cu.check_status(torch.device(DEV))
    assert _rel(got.cpu(), want) < 1e-2


def test_routed_experts_record_on_gpu():
    """The per-slot routing record with the lookahead engine on the GPU: complete for every token that has K/V,
    equal to the step-by-step engine's, and unchanged by prompt slicing."""
    from parallax_b200.engine.engine import Engine
    from parallax_b200.engine.request import Request, SamplingParams
    from parallax_b200.models.config import config_from_hf

    cfg = config_from_hf(dict(architectures=["Qwen3MoeForCausalLM"], model_type="qwen3_moe", hidden_size=512,
                              num_hidden_layers=2, num_attention_heads=8, num_key_value_heads=2, head_dim=64,
                              intermediate_size=1024, moe_intermediate_size=256, num_experts=16,
                              num_experts_per_tok=4, norm_topk_prob=True, vocab_size=2048, rope_theta=1e4))
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, 2048, (n,), generator=g).tolist() for n in (70, 9, 33)]

    def run(**kw):
        eng = Engine(cfg, device=DEV, dtype=torch.bfloat16, num_blocks=64, max_batch_size=8, seed=0,
                     enable_prefix_cache=False, return_routed_experts=True, **kw)
        reqs = [Request(input_ids=p, sampling_params=SamplingParams(max_new_tokens=5, temperature=0.0, ignore_eos=True))
                for p in prompts]
        for r in reqs:
            eng.add_request(r)
        while eng.has_work():
            eng.step()
        return reqs

    a = run()
    for r in a:
        rec = torch.tensor(r.routed_experts)
        assert rec.shape == (r.prompt_len + len(r.output_ids) - 1, 2, 4)
        assert int(rec.min()) >= 0 and int(rec.max()) < 16
    b = run(async_scheduling=False)
    c = run(chunked_prefill_size=32)
    same_b = sum(x.routed_experts == y.routed_experts for x, y in zip(a, b))
    assert same_b == len(a)                      # same kernels on the same rows
    for x, y in zip(a, c):
        # other row counts per step change the GEMM tiles: a router logit near a tie may flip, most do not
        rx, ry = torch.tensor(x.routed_experts)[:x.prompt_len], torch.tensor(y.routed_experts)[:y.prompt_len]
        assert (rx.sort(-1).values == ry.sort(-1).values).float().mean() > 0.97
    from parallax_b200.ops import cuda as cu

    cu.check_status(torch.device(DEV))
