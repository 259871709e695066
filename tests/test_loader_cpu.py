"""Shard loader: per-layer-range loading from sharded safetensors, and expansion of affine group-quantised
checkpoints (the format of MLX-converted models) with per-module overrides."""

import json

import pytest
import torch

from helpers.hf_weights import hf_state_dict
from parallax_b200.loader.quant import dequant_affine, expand_affine_quantized, quantize_affine
from parallax_b200.loader.shard_loader import ShardLoader
from parallax_b200.models.config import named_config

safetensors = pytest.importorskip("safetensors.torch")

HF = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=256, num_hidden_layers=4,
          num_attention_heads=4, num_key_value_heads=2, head_dim=64, intermediate_size=512, vocab_size=1024,
          tie_word_embeddings=True, rope_theta=1e4)


def _write(tmp_path, sd, hf, n_files=2):
    keys = sorted(sd)
    per = (len(keys) + n_files - 1) // n_files
    index = {}
    for i in range(n_files):
        part = {k: sd[k].contiguous() for k in keys[i * per:(i + 1) * per]}
        name = f"model-{i + 1:05d}-of-{n_files:05d}.safetensors"
        safetensors.save_file(part, str(tmp_path / name))
        index.update({k: name for k in part})
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": index}))
    (tmp_path / "config.json").write_text(json.dumps(hf))


def test_layer_range_loading_from_sharded_safetensors(tmp_path):
    cfg = named_config("tiny")
    sd = hf_state_dict(cfg, "decoder", seed=4)
    _write(tmp_path, sd, HF, n_files=3)
    mid = ShardLoader(str(tmp_path), 1, 3).load_weights("cpu", torch.float32)
    layers = {int(k.split(".")[2]) for k in mid if k.startswith("model.layers.")}
    assert layers == {1, 2} and "model.embed_tokens.weight" not in mid and "model.norm.weight" not in mid
    assert all(torch.equal(mid[k], sd[k]) for k in mid)
    first = ShardLoader(str(tmp_path), 0, 2).load_weights("cpu", torch.float32)
    assert "model.embed_tokens.weight" in first and "model.norm.weight" not in first
    last = ShardLoader(str(tmp_path), 2, 4).load_weights("cpu", torch.float32)
    # tied embeddings: the last stage needs the table for its head
    assert "model.norm.weight" in last and "model.embed_tokens.weight" in last


@pytest.mark.parametrize("bits,group", [(4, 32), (8, 64), (2, 32)])
def test_affine_quantisation_round_trip(bits, group):
    torch.manual_seed(0)
    w = torch.randn(48, 256)
    words, s, b = quantize_affine(w, bits, group)
    assert words.shape == (48, 256 * bits // 32) and s.shape == b.shape == (48, 256 // group)
    back = dequant_affine(words, s, b, bits, group, torch.float32)
    step = (w.view(48, -1, group).amax(-1) - w.view(48, -1, group).amin(-1)) / ((1 << bits) - 1)
    assert float(((back - w).abs().view(48, -1, group).amax(-1) - 0.51 * step - 2e-2).max()) <= 0
    # the same words seen as unsigned, as safetensors hands them out
    if hasattr(torch, "uint32"):
        assert torch.equal(dequant_affine(words.view(torch.uint32), s, b, bits, group, torch.float32), back)
    with pytest.raises(ValueError):
        dequant_affine(words, s, b, 3, group)


def test_quantised_checkpoint_with_per_module_overrides_loads_as_floating_point(tmp_path):
    from parallax_b200.engine.engine import Engine
    from parallax_b200.engine.request import SamplingParams

    cfg = named_config("tiny")
    sd = hf_state_dict(cfg, "decoder", seed=5)
    quant = {"group_size": 32, "bits": 4,
             "model.layers.0.mlp.down_proj": {"group_size": 64, "bits": 8},       # override
             "model.layers.1.self_attn.o_proj": False}                             # left in floating point
    packed, want = {}, {}
    for k, v in sd.items():
        mod = k[: -len(".weight")]
        linear = k.endswith("_proj.weight") or k == "model.embed_tokens.weight"
        spec = quant.get(mod)
        if not linear or spec is False:
            packed[k] = want[k] = v
            continue
        bits, group = (spec["bits"], spec["group_size"]) if isinstance(spec, dict) else (4, 32)
        words, s, b = quantize_affine(v, bits, group)
        packed[k], packed[mod + ".scales"], packed[mod + ".biases"] = words, s, b
        want[k] = dequant_affine(words, s, b, bits, group, torch.float32)
    _write(tmp_path, packed, dict(HF, quantization=quant))
    got = ShardLoader(str(tmp_path), 0, 4).load_weights("cpu", torch.float32)
    assert set(got) == set(want)                                   # scales / biases are gone
    for k in want:
        assert got[k].dtype == torch.float32 and torch.allclose(got[k], want[k], atol=1e-6), k
    # a wrong global setting would not reproduce the 8-bit layer: the override was used
    w8 = want["model.layers.0.mlp.down_proj.weight"]
    assert float((w8 - sd["model.layers.0.mlp.down_proj.weight"]).abs().max()) < 2e-3
    # and the engine serves the expanded weights
    prompts = [[5, 9, 77, 3, 250, 12, 8], list(range(20, 60))]
    sp = SamplingParams(max_new_tokens=5, temperature=0.0, ignore_eos=True)
    kw = dict(device="cpu", num_blocks=64, max_batch_size=4, chunked_prefill_size=16)
    assert Engine(cfg, weights=got, **kw).generate(prompts, sp) == Engine(cfg, weights=want, **kw).generate(prompts, sp)
    assert expand_affine_quantized(dict(sd), None) == 0
