"""GPT-OSS family on CPU against Hugging Face: attention sinks, alternating sliding-window layers,
QKV / output biases, router bias, clipped swigluoai experts with biases, YaRN without truncation."""

import pytest
import torch

from parallax_b200.engine.engine import Engine
from parallax_b200.engine.request import Request, SamplingParams
from parallax_b200.models.config import config_from_hf


def test_engine_matches_huggingface_gpt_oss():
    transformers = pytest.importorskip("transformers")
    if not hasattr(transformers, "GptOssForCausalLM"):
        pytest.skip("this transformers release has no GPT-OSS")
    hf_cfg = transformers.GptOssConfig(
        hidden_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=32,
        intermediate_size=64, num_local_experts=4, num_experts_per_tok=2, sliding_window=16,
        layer_types=["sliding_attention", "full_attention"], vocab_size=512, max_position_embeddings=512,
        rope_theta=10000.0, tie_word_embeddings=False, attention_bias=True)
    torch.manual_seed(0)
    hf = transformers.GptOssForCausalLM(hf_cfg).eval().float()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if n.endswith("sinks") or n.endswith("bias"):
                p.copy_(torch.randn_like(p) * 0.5)
    cfg = config_from_hf(hf_cfg.to_dict() | {"architectures": ["GptOssForCausalLM"]})
    assert cfg.attention_sinks and cfg.swiglu_limit == 7.0 and cfg.layer_window(0) == 16 and cfg.layer_window(1) == 0
    sd = {k: v.detach().clone() for k, v in hf.state_dict().items()}
    eng = Engine(cfg, device="cpu", num_blocks=64, page_size=16, max_batch_size=4, chunked_prefill_size=24, weights=sd)
    eng.keep_logits = True
    g = torch.Generator().manual_seed(4)
    prompt = torch.randint(0, 512, (45,), generator=g).tolist()
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
        assert torch.allclose(got, want, atol=1e-3, rtol=2e-3), float((got - want).abs().max())
        seq.append(tok)


def test_mxfp4_expert_checkpoint_layout():
    """Experts stored as MXFP4 blocks + scales (the published GPT-OSS format) load to the same model as
    the bf16 layout holding the expanded values, and the expansion agrees with Hugging Face's converter."""
    transformers = pytest.importorskip("transformers")
    if not hasattr(transformers, "GptOssForCausalLM"):
        pytest.skip("this transformers release has no GPT-OSS")
    from parallax_b200.loader.quant import dequant_mxfp4, quantize_mxfp4

    hf_cfg = transformers.GptOssConfig(
        hidden_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=32,
        intermediate_size=64, num_local_experts=4, num_experts_per_tok=2, sliding_window=16,
        layer_types=["sliding_attention", "full_attention"], vocab_size=512, max_position_embeddings=512,
        rope_theta=10000.0, tie_word_embeddings=False, attention_bias=True)
    torch.manual_seed(1)
    hf = transformers.GptOssForCausalLM(hf_cfg).eval().float()
    cfg = config_from_hf(hf_cfg.to_dict() | {"architectures": ["GptOssForCausalLM"]})
    sd = {k: v.detach().clone() for k, v in hf.state_dict().items()}
    packed, expanded = dict(sd), dict(sd)
    for name in list(sd):
        if name.endswith("experts.gate_up_proj") or name.endswith("experts.down_proj"):
            blocks, scales = quantize_mxfp4(sd[name].transpose(1, 2).contiguous() * 20.0)   # [E, out, in]
            del packed[name]
            packed[name + "_blocks"], packed[name + "_scales"] = blocks, scales
            expanded[name] = dequant_mxfp4(blocks, scales, torch.float32).transpose(1, 2).contiguous()
    try:
        from transformers.integrations.mxfp4 import convert_moe_packed_tensors
    except ImportError:
        convert_moe_packed_tensors = None
    if convert_moe_packed_tensors is not None:
        name = "model.layers.0.mlp.experts.down_proj"
        want = convert_moe_packed_tensors(packed[name + "_blocks"], packed[name + "_scales"]).float()
        assert torch.equal(want, expanded[name])

    def run(weights):
        eng = Engine(cfg, device="cpu", num_blocks=64, page_size=16, max_batch_size=4, weights=weights)
        eng.keep_logits = True
        req = Request(input_ids=list(range(3, 40)),
                      sampling_params=SamplingParams(max_new_tokens=2, temperature=0.0, ignore_eos=True))
        eng.add_request(req)
        out = []
        while eng.has_work():
            eng.step()
            if eng.last_logits is not None and eng.last_logits.shape[0] > 0:
                out.append(eng.last_logits[0].clone())
            eng.last_logits = None
        return out, req.output_ids

    a, ta = run(packed)
    b, tb = run(expanded)
    assert ta == tb and len(a) == len(b) > 0
    for x, y in zip(a, b):
        assert torch.allclose(x, y, atol=1e-5, rtol=1e-5)
