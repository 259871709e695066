"""Hybrid gated-delta-net / gated-attention stages on CPU: parity with the Hugging Face
Qwen3-Next implementation (its plain-PyTorch path) and chunked-prefill consistency."""

import pytest
import torch

from parallax_b200.engine.engine import Engine
from parallax_b200.engine.request import Request, SamplingParams
from parallax_b200.models.config import config_from_hf, named_config


def test_hybrid_engine_matches_huggingface_qwen3_next():
    transformers = pytest.importorskip("transformers")
    if not hasattr(transformers, "Qwen3NextForCausalLM"):
        pytest.skip("this transformers release has no Qwen3-Next")
    E, I, H = 4, 64, 128
    hf_cfg = transformers.Qwen3NextConfig(
        hidden_size=H, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2, head_dim=32,
        intermediate_size=256, vocab_size=1024, rope_theta=1e4, partial_rotary_factor=0.25, full_attention_interval=2,
        linear_num_key_heads=2, linear_num_value_heads=4, linear_key_head_dim=32, linear_value_head_dim=32,
        linear_conv_kernel_dim=4, num_experts=E, num_experts_per_tok=2, moe_intermediate_size=I,
        shared_expert_intermediate_size=I, decoder_sparse_step=1, mlp_only_layers=[], norm_topk_prob=True,
        max_position_embeddings=512, tie_word_embeddings=False)
    torch.manual_seed(0)
    hf = transformers.Qwen3NextForCausalLM(hf_cfg).eval().float()
    with torch.no_grad():          # make the zero-centred norm weights and the gates non-trivial
        for n, p in hf.named_parameters():
            if n.endswith("layernorm.weight") or n.endswith("_norm.weight") or n.endswith("model.norm.weight"):
                p.add_(torch.randn_like(p) * 0.1)
    cfg = config_from_hf(hf_cfg.to_dict() | {"architectures": ["Qwen3NextForCausalLM"]})
    assert cfg.has_linear_layers and cfg.layer_kind(0) == "linear" and cfg.layer_kind(1) == "attention"
    sd = {k: v.detach().clone() for k, v in hf.state_dict().items()}
    for li in range(4):
        p = f"model.layers.{li}.mlp.experts."
        if p + "gate_up_proj" in sd:
            gu, dn = sd.pop(p + "gate_up_proj"), sd.pop(p + "down_proj")
            for e in range(E):
                g_u = gu[e] if gu[e].shape[0] == 2 * I else gu[e].t()
                sd[f"{p}{e}.gate_proj.weight"], sd[f"{p}{e}.up_proj.weight"] = g_u[:I], g_u[I:]
                sd[f"{p}{e}.down_proj.weight"] = dn[e] if dn[e].shape == (H, I) else dn[e].t()
    eng = Engine(cfg, device="cpu", num_blocks=64, page_size=16, max_batch_size=4, chunked_prefill_size=16, weights=sd)
    eng.keep_logits = True
    g = torch.Generator().manual_seed(4)
    prompt = torch.randint(0, 1024, (37,), generator=g).tolist()
    req = Request(input_ids=prompt, sampling_params=SamplingParams(max_new_tokens=3, temperature=0.0, ignore_eos=True))
    eng.add_request(req)
    logits = []
    while eng.has_work():
        eng.step()
        if eng.last_logits is not None and eng.last_logits.shape[0] > 0:
            logits.append(eng.last_logits[0].clone())
            eng.last_logits = None
    seq = list(prompt)
    for got, tok in zip(logits, req.output_ids):
        with torch.no_grad():
            want = hf(torch.tensor([seq])).logits[0, -1]
        assert torch.allclose(got, want, atol=5e-4, rtol=2e-3), float((got - want).abs().max())
        assert int(want.argmax()) == tok
        seq.append(tok)


def test_hybrid_chunked_prefill_and_slots_are_consistent():
    cfg = named_config("tiny-hybrid")
    prompts = [[1, 2, 3, 4, 5, 6, 7] * 6, [9] * 30, list(range(50, 70)), [3, 1, 4, 1, 5, 9, 2, 6] * 4]
    sp = SamplingParams(max_new_tokens=6, temperature=0.0, ignore_eos=True)
    a = Engine(cfg, device="cpu", num_blocks=64, page_size=16, max_batch_size=4, max_num_tokens_per_batch=256,
               chunked_prefill_size=24, max_total_length=256).generate(prompts, sp)
    b = Engine(cfg, device="cpu", num_blocks=64, page_size=16, max_batch_size=2, max_num_tokens_per_batch=256,
               chunked_prefill_size=None, max_total_length=256).generate(prompts, sp)
    assert a == b
    eng = Engine(cfg, device="cpu", num_blocks=64, page_size=16, max_batch_size=4, linear_prefix_slots=0)
    assert eng.cache.prefix_cache is None      # without snapshot slots a recurrent state cannot be resumed


def test_hybrid_prefix_cache_resumes_from_state_snapshots():
    """Requests that share a prefix reuse its KV pages AND the recurrent state as of the end of the prefix:
    the state is snapshotted when a prompt slice ends on a block boundary, and a later request starts from a
    copy of the snapshot. Outputs must equal a run without any prefix caching."""
    cfg = named_config("tiny-hybrid")
    g = torch.Generator().manual_seed(9)
    shared = torch.randint(0, cfg.vocab_size, (64,), generator=g).tolist()
    tails = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (7, 21, 3, 40)]
    prompts = [shared + t for t in tails]
    sp = SamplingParams(max_new_tokens=5, temperature=0.0, ignore_eos=True)
    kw = dict(device="cpu", num_blocks=128, page_size=16, max_batch_size=4, max_num_tokens_per_batch=256,
              chunked_prefill_size=32, max_total_length=256)
    want = Engine(cfg, linear_prefix_slots=0, **kw).generate(prompts, sp)
    eng = Engine(cfg, linear_prefix_slots=8, **kw)
    assert eng.cache.prefix_cache is not None and eng.cache.needs_slots
    first = eng.generate(prompts[:1], sp)             # computes the prefix, snapshots at 32 and 64 tokens
    rest = eng.generate(prompts[1:], sp)              # resume from the snapshot at 64 tokens
    assert first + rest == want
    assert eng.cache.prefix_cache.hits >= 3
    snap = [n for n in eng.cache.prefix_cache.get_path(shared) if n.linear_slot is not None]
    assert len(snap) >= 1 and snap[-1] is eng.cache.prefix_cache.get_path(shared)[-1]
    again = eng.generate(prompts, sp)                 # everything cached now, still the same tokens
    assert again == want
