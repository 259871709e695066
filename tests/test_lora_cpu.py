"""Per-request LoRA adapters: a batch in which every request uses its own adapter (or none) must produce what
separate engines with the adapter merged into their weights produce."""

import json

import torch
from safetensors.torch import save_file

from parallax_b200.engine.engine import Engine
from parallax_b200.engine.request import Request, SamplingParams
from parallax_b200.loader.lora import LoRAAdapter, parse_lora_paths
from parallax_b200.loader.shard_loader import apply_lora_adapter
from parallax_b200.models.config import named_config


def _make_adapter(cfg, path, seed, rank=4, alpha=8):
    g = torch.Generator().manual_seed(seed)
    D, Hq, Hkv, H, I = cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.hidden_size, cfg.intermediate_size
    dims = {"self_attn.q_proj": (H, Hq * D), "self_attn.k_proj": (H, Hkv * D), "self_attn.v_proj": (H, Hkv * D),
            "self_attn.o_proj": (Hq * D, H), "mlp.down_proj": (I, H)}
    t = {}
    for li in range(cfg.num_hidden_layers):
        for mod, (n_in, n_out) in dims.items():
            if li == 1 and mod == "self_attn.k_proj":
                continue          # an adapter need not cover every module
            base = f"base_model.model.model.layers.{li}.{mod}"
            t[base + ".lora_A.weight"] = torch.randn(rank, n_in, generator=g) * 0.2
            t[base + ".lora_B.weight"] = torch.randn(n_out, rank, generator=g) * 0.2
    path.mkdir()
    save_file(t, str(path / "adapter_model.safetensors"))
    (path / "adapter_config.json").write_text(json.dumps({"r": rank, "lora_alpha": alpha}))
    return str(path)


def _export(eng):
    from tests.test_engine_gpu import _export_weights

    return _export_weights(eng)


def test_batched_adapters_match_merged_weights(tmp_path):
    cfg = named_config("tiny")
    a1 = _make_adapter(cfg, tmp_path / "a1", 1)
    a2 = _make_adapter(cfg, tmp_path / "a2", 2, rank=8, alpha=4)
    assert LoRAAdapter.load(a1).rank == 4 and parse_lora_paths(["x=" + a1, a2]) == {"x": a1, "a2": a2}
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (21, 9, 33)]
    sp = dict(max_new_tokens=6, temperature=0.0, ignore_eos=True)
    kw = dict(device="cpu", num_blocks=64, max_batch_size=4, chunked_prefill_size=16)
    base = Engine(cfg, **kw)
    weights = _export(base)

    def merged(adapter):
        w = {k: v.clone() for k, v in weights.items()}
        if adapter:
            assert apply_lora_adapter(w, adapter) > 0
        return Engine(cfg, weights=w, **kw)

    want = [merged(a1).generate([prompts[0]], SamplingParams(**sp))[0],
            merged(a2).generate([prompts[1]], SamplingParams(**sp))[0],
            merged(None).generate([prompts[2]], SamplingParams(**sp))[0]]
    eng = Engine(cfg, weights={k: v.clone() for k, v in weights.items()},
                 lora={"max_loaded": 2, "max_rank": 8, "paths": {"one": a1, "two": a2}}, **kw)
    reqs = [Request(input_ids=prompts[0], sampling_params=SamplingParams(**sp), lora_path="one"),
            Request(input_ids=prompts[1], sampling_params=SamplingParams(**sp), lora_path="two"),
            Request(input_ids=prompts[2], sampling_params=SamplingParams(**sp))]
    for r in reqs:
        eng.add_request(r)
    while eng.has_work():
        eng.step()
    eng.flush()
    assert [r.output_ids for r in reqs] == want
    assert want[0] != want[2] or want[1] != want[2]        # the adapters do change the model
    assert all(v == 0 for v in eng.lora.pins.values())     # finished requests unpinned their adapters
    # a third adapter takes the slot of the least recently used one
    a3 = _make_adapter(cfg, tmp_path / "a3", 3)
    r = Request(input_ids=prompts[0], sampling_params=SamplingParams(**sp), lora_path=a3)
    eng.add_request(r)
    while eng.has_work():
        eng.step()
    assert len(eng.lora.slot_of) == 2 and a3 in eng.lora.slot_of and "one" not in eng.lora.slot_of
    assert r.output_ids == merged(a3).generate([prompts[0]], SamplingParams(**sp))[0]


import pytest


@pytest.mark.gpu
def test_lora_update_on_grouped_tcgen05_gemms(tmp_path):
    """The adapter update on the GPU path (rows gathered per adapter, two grouped GEMMs, scaled add) against
    plain fp32 math, on the qkv / o / down projections of a small model, with rows that use no adapter."""
    from parallax_b200.loader.lora import LoRAStack
    from parallax_b200.models.config import config_from_hf
    from parallax_b200.models.decoder import DecoderStage
    from parallax_b200.ops import cuda as cu

    cfg = config_from_hf(dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=512,
                              num_hidden_layers=2, num_attention_heads=8, num_key_value_heads=2, head_dim=128,
                              intermediate_size=1024, vocab_size=2048, tie_word_embeddings=False, rope_theta=1e4))
    dev = torch.device("cuda", 0)
    stage = DecoderStage(cfg, 0, 2, dev, torch.bfloat16)
    stage.init_random(0)
    stack = LoRAStack(stage, max_slots=3, max_rank=16)
    ads = [LoRAAdapter.load(_make_adapter(cfg, tmp_path / f"g{i}", 10 + i, rank=r, alpha=2 * r)) for i, r in enumerate((4, 16))]
    stack.load(0, ads[0])
    stack.load(2, ads[1])
    T = 300
    g = torch.Generator().manual_seed(1)
    slot = torch.tensor([[-1, 0, 2][int(i)] for i in torch.randint(0, 3, (T,), generator=g)], dtype=torch.int32)
    for tgt, n_in in (("qkv", 512), ("o", 1024), ("down", 1024)):
        x = (torch.randn(T, n_in, generator=g) * 0.5).to(torch.bfloat16)
        n_out = stack.dims[tgt][1]
        y = (torch.randn(T, n_out, generator=g)).to(torch.bfloat16)
        got = stack.apply(tgt, 1, x.to(dev), y.to(dev), slot.to(dev)).float().cpu()
        want = y.float().clone()
        for s, ad in ((0, ads[0]), (2, ads[1])):
            rows = (slot == s).nonzero().flatten()
            mods = {"qkv": ("q_proj", "k_proj", "v_proj"), "o": ("o_proj",), "down": ("down_proj",)}[tgt]
            col = 0
            for mod in mods:
                A, B = ad.tensors[(1, mod)] if (1, mod) in ad.tensors else (None, None)
                width = B.shape[0] if B is not None else (cfg.num_key_value_heads * cfg.head_dim)
                if A is not None:
                    want[rows, col:col + width] += ad.scaling * (x[rows].float() @ A.t()) @ B.t()
                col += width
        rel = float((got - want).norm() / want.norm())
        assert rel < 2e-2, (tgt, rel)
        untouched = (slot == -1).nonzero().flatten()
        assert torch.equal(got[untouched], y[untouched].float())
    cu.check_status(dev)


import pytest


@pytest.mark.parametrize("model,pp,tp,ep", [("tiny", 2, 1, 1), ("tiny", 1, 2, 1), ("tiny", 2, 2, 1), ("tiny-moe", 1, 1, 2)])
def test_per_request_adapters_across_ranks(model, pp, tp, ep, tmp_path):
    """Several ranks as processes: rank 0 decides which adapter lives in which slot, the load travels with the
    step plan and every rank loads its own part of the adapter - its layers (pipeline stages), its heads and
    intermediate slice (tensor-parallel ranks), or the whole adapter (expert-parallel lanes, which run whole
    attention layers on their own requests). Same tokens as the single-process engine with the same adapters."""
    import os
    import subprocess
    import sys

    from parallax_b200.parallel.launcher import free_port

    cfg = named_config(model)
    a1 = _make_adapter(cfg, tmp_path / "a1", 1)
    a2 = _make_adapter(cfg, tmp_path / "a2", 2, rank=8, alpha=4)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (21, 9, 33, 17)]
    lora_of = ["x", "y", None, "x"]
    world = pp * tp * ep
    lora = {"max_loaded": 2, "max_rank": 8, "paths": {"x": a1, "y": a2}}
    kw = dict(num_blocks=128, page_size=16, max_batch_size=4, max_num_tokens_per_batch=64, chunked_prefill_size=16,
              max_total_length=256, seed=0)
    torch.manual_seed(0)
    eng = Engine(cfg, device="cpu", lora=lora, **kw)
    reqs = [Request(input_ids=p, sampling_params=SamplingParams(max_new_tokens=6, temperature=0.0, ignore_eos=True),
                    lora_path=a) for p, a in zip(prompts, lora_of)]
    for r in reqs:
        eng.add_request(r)
    while eng.has_work():
        eng.step()
    want = [r.output_ids for r in reqs]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    helper = os.path.join(root, "tests", "helpers", "dist_engine_rank.py")
    spec = dict(model_name=model, pp=pp, tp=tp, ep=ep, device_type="cpu", prompts=prompts, max_new=6, lora=lora,
                lora_of=lora_of, **kw)
    out, port = tmp_path / "out.json", free_port()
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                   OMP_NUM_THREADS="2", PYTHONPATH=root + os.pathsep + os.environ.get("PYTHONPATH", ""))
        procs.append(subprocess.Popen([sys.executable, helper, json.dumps(spec), str(out)], env=env))
    assert [p.wait(timeout=240) for p in procs] == [0] * world
    got = json.loads(out.read_text())["outputs"]
    assert got == want
    # the adapters really change the output of their requests
    base = Engine(cfg, device="cpu", **kw).generate(prompts, SamplingParams(max_new_tokens=6, temperature=0.0, ignore_eos=True))
    assert got[2] == base[2] and (got[0] != base[0] or got[1] != base[1])


def test_adapter_preparation_and_both_layouts(tmp_path):
    """An adapter prepared for either layout loads to the same matrices and scale, and the completed config
    carries the fields of both."""
    from parallax_b200.utils.prepare_adapter import main as prepare_main, prepare_adapter

    cfg = named_config("tiny")
    src = _make_adapter(cfg, tmp_path / "peft", 5, rank=4, alpha=8)
    (tmp_path / "base").mkdir()
    (tmp_path / "base" / "config.json").write_text(json.dumps({"num_hidden_layers": cfg.num_hidden_layers}))
    mlx = prepare_adapter(src, str(tmp_path / "mlx"), base=str(tmp_path / "base"), layout="mlx", dtype="float32")
    c = json.loads((mlx / "adapter_config.json").read_text())
    assert c["fine_tune_type"] == "lora" and c["num_layers"] == cfg.num_hidden_layers
    assert c["lora_parameters"] == {"rank": 4, "scale": 2.0, "dropout": 0.0} and c["r"] == 4 and c["lora_alpha"] == 8
    assert (mlx / "adapters.safetensors").exists() and not (mlx / "adapter_model.safetensors").exists()
    a, b = LoRAAdapter.load(src), LoRAAdapter.load(str(mlx))
    assert a.rank == b.rank == 4 and a.scaling == b.scaling == 2.0 and set(a.tensors) == set(b.tensors)
    for k in a.tensors:
        assert torch.equal(a.tensors[k][0], b.tensors[k][0]) and torch.equal(a.tensors[k][1], b.tensors[k][1])
    # and back, through the command
    prepare_main([str(mlx), "--out", str(tmp_path / "back"), "--layout", "peft", "--dtype", "float32"])
    c2 = LoRAAdapter.load(str(tmp_path / "back"))
    assert c2.scaling == 2.0 and all(torch.equal(a.tensors[k][1], c2.tensors[k][1]) for k in a.tensors)
