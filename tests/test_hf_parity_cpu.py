"""Hugging Face parity on CPU for decoder families that differ only by configuration flags:
MiniMax-M2 (qk-norm over the whole projection, partial rotary, sigmoid routing with a selection
bias) and GLM-4-MoE (partial rotary, grouped sigmoid routing, shared experts, leading dense layers)."""

import pytest
import torch

from parallax_b200.engine.engine import Engine
from parallax_b200.engine.request import Request, SamplingParams
from parallax_b200.models.config import config_from_hf


def _unfuse_experts(sd, n_layers, E, I, H):
    """Newer transformers releases store experts fused as [E, 2I, H] / [E, H, I]."""
    for li in range(n_layers):
        p = f"model.layers.{li}.mlp.experts."
        if p + "gate_up_proj" not in sd:
            continue
        gu, dn = sd.pop(p + "gate_up_proj"), sd.pop(p + "down_proj")
        for e in range(E):
            g_u = gu[e] if gu[e].shape == (2 * I, H) else gu[e].t()
            sd[f"{p}{e}.gate_proj.weight"], sd[f"{p}{e}.up_proj.weight"] = g_u[:I], g_u[I:]
            sd[f"{p}{e}.down_proj.weight"] = dn[e] if dn[e].shape == (H, I) else dn[e].t()
    return sd


def _check(hf, cfg, sd, vocab, n_prompt=41, chunk=16, atol=1e-3):
    eng = Engine(cfg, device="cpu", num_blocks=64, page_size=16, max_batch_size=4, chunked_prefill_size=chunk, weights=sd)
    eng.keep_logits = True
    g = torch.Generator().manual_seed(4)
    prompt = torch.randint(0, vocab, (n_prompt,), generator=g).tolist()
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
        assert torch.allclose(got, want, atol=atol, rtol=2e-3), float((got - want).abs().max())
        seq.append(tok)


def test_minimax_m2():
    transformers = pytest.importorskip("transformers")
    if not hasattr(transformers, "MiniMaxM2ForCausalLM"):
        pytest.skip("this transformers release has no MiniMax-M2")
    E, I, H = 4, 64, 128
    hc = transformers.MiniMaxM2Config(hidden_size=H, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                                      head_dim=32, intermediate_size=I, num_local_experts=E, num_experts_per_tok=2,
                                      vocab_size=512, max_position_embeddings=512,
                                      tie_word_embeddings=False, rotary_dim=16, use_qk_norm=True,
                                      rope_parameters={"rope_type": "default", "rope_theta": 10000.0,
                                                       "partial_rotary_factor": 0.5})
    torch.manual_seed(0)
    hf = transformers.MiniMaxM2ForCausalLM(hc).eval().float()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if n.endswith("norm.weight"):
                p.add_(torch.randn_like(p) * 0.1)
        for n, b in hf.named_buffers():
            if n.endswith("e_score_correction_bias"):
                b.copy_(torch.randn_like(b) * 0.5)
    cfg = config_from_hf(hc.to_dict() | {"architectures": ["MiniMaxM2ForCausalLM"]})
    assert cfg.qk_norm_full and cfg.rot_dim == 16 and cfg.scoring_func == "sigmoid"
    sd = _unfuse_experts({k: v.detach().clone() for k, v in hf.state_dict().items()}, 2, E, I, H)
    _check(hf, cfg, sd, 512)


def test_glm4_moe():
    transformers = pytest.importorskip("transformers")
    if not hasattr(transformers, "Glm4MoeForCausalLM"):
        pytest.skip("this transformers release has no GLM-4-MoE")
    E, I, H = 8, 64, 128
    hc = transformers.Glm4MoeConfig(hidden_size=H, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2,
                                    head_dim=32, intermediate_size=256, moe_intermediate_size=I, n_routed_experts=E,
                                    num_experts_per_tok=2, n_shared_experts=1, first_k_dense_replace=1, n_group=2,
                                    topk_group=1, norm_topk_prob=True, routed_scaling_factor=1.5, vocab_size=512,
                                    max_position_embeddings=512, rope_theta=10000.0, partial_rotary_factor=0.5,
                                    use_qk_norm=True, attention_bias=True, tie_word_embeddings=False)
    torch.manual_seed(0)
    hf = transformers.Glm4MoeForCausalLM(hc).eval().float()
    with torch.no_grad():
        for n, b in list(hf.named_buffers()) + list(hf.named_parameters()):
            if n.endswith("e_score_correction_bias"):
                b.copy_(torch.randn_like(b) * 0.5)
    cfg = config_from_hf(hc.to_dict() | {"architectures": ["Glm4MoeForCausalLM"]})
    assert cfg.first_k_dense_replace == 1 and cfg.n_group == 2 and cfg.rot_dim == 16
    sd = _unfuse_experts({k: v.detach().clone() for k, v in hf.state_dict().items()}, 3, E, I, H)
    _check(hf, cfg, sd, 512)
