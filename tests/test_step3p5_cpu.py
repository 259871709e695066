"""Step-3.5-style decoder: head-wise sigmoid gate on the attention output."""

import torch

from parallax_b200.engine.engine import Engine
from parallax_b200.engine.request import Request, SamplingParams
from parallax_b200.models.config import config_from_hf


def _logits(cfg, mutate):
    torch.manual_seed(0)
    eng = Engine(cfg, device="cpu", num_blocks=64, page_size=16, max_batch_size=4, seed=0)
    mutate(eng.stages[0].model)
    eng.keep_logits = True
    g = torch.Generator().manual_seed(1)
    for n in (19, 5):
        eng.add_request(Request(input_ids=torch.randint(0, 512, (n,), generator=g).tolist(),
                                sampling_params=SamplingParams(max_new_tokens=3, temperature=0.0, ignore_eos=True)))
    eng.step()
    first = eng.last_logits.float().clone()
    eng.step()
    return first, eng.last_logits.float().clone()


def test_head_gate_scales_each_head_of_the_attention_output():
    base = dict(architectures=["Step3p5ForCausalLM"], model_type="step3p5", hidden_size=128, num_hidden_layers=2,
                num_attention_heads=4, num_key_value_heads=2, head_dim=32, intermediate_size=256, vocab_size=512,
                tie_word_embeddings=True, rope_theta=1e4)
    gated = config_from_hf(dict(base, use_head_wise_attn_gate=True))
    plain = config_from_hf(dict(base))

    # a gate projection of zeros gives sigmoid(0) = 1/2 on every head: the same as halving o_proj's input columns
    def zero_gate(m):
        assert all(lw.w_g is not None and lw.w_g.shape == (4, 128) for lw in m.layers)
        for lw in m.layers:
            lw.w_g.zero_()

    def half_o(m):
        assert all(lw.w_g is None for lw in m.layers)
        for lw in m.layers:
            lw.w_o.mul_(0.5)

    a, b = _logits(gated, zero_gate), _logits(plain, half_o)
    for x, y in zip(a, b):
        assert torch.allclose(x, y, atol=1e-4, rtol=1e-4)

    # and the gate is live: with its random projection the logits differ from the half-open gate's
    c = _logits(gated, lambda m: None)
    assert not torch.allclose(c[0], a[0], atol=1e-3)
