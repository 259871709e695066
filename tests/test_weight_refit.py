"""Weight refit data path: content ids, partitioned tensors, layer filter, in-memory safetensors, and a whole refit
request applied to a live stage."""

import os

import pytest
import torch
from safetensors.torch import save, save_file

from parallax_b200.engine.engine import Engine
from parallax_b200.engine.request import Request, SamplingParams
from parallax_b200.models.config import named_config
from parallax_b200.utils.weight_refit import (RefitVersionStore, apply_refit_to_stage, calculate_cid,
                                              concat_weight_partition, filter_weight_cid_list,
                                              parse_safetensors_from_memory, verify_block)


def test_content_ids_and_block_check():
    data = b"some weight block"
    cid = calculate_cid(data)
    assert cid.startswith("bafkrei") and cid == cid.lower() and len(cid) == 59        # CIDv1, raw, sha2-256, base32
    assert verify_block(data, cid) and not verify_block(data + b"x", cid)
    assert calculate_cid(b"") != cid


def test_partitions_are_joined_in_order_and_gaps_are_refused(tmp_path):
    a, b, c = torch.arange(6.).view(2, 3), torch.arange(6., 12.).view(2, 3), torch.ones(4)
    out = concat_weight_partition({"m.q_proj.weight_part1": b, "m.q_proj.weight_part0": a, "m.norm.weight": c})
    assert set(out) == {"m.q_proj.weight", "m.norm.weight"} and torch.equal(out["m.q_proj.weight"], torch.cat([a, b]))
    with pytest.raises(ValueError):
        concat_weight_partition({"m.q_proj.weight_part0": a, "m.q_proj.weight_part2": b})
    assert concat_weight_partition({"m.x.weight_part0": a}, save_directory=str(tmp_path / "v")) == {}
    assert os.path.exists(tmp_path / "v" / "adapter_model.safetensors")


def test_layer_filter_and_in_memory_parse():
    index = {"model.embed_tokens.weight": "c0", "model.layers.0.mlp.down_proj.weight": "c1",
             "model.layers.3.mlp.down_proj.weight": "c2", "model.norm.weight": "c3", "lm_head.weight": "c3"}
    assert filter_weight_cid_list(0, 2, 4, index) == ["c0", "c1"]
    assert filter_weight_cid_list(2, 4, 4, index) == ["c0", "c2", "c3"]       # tied head: the last stage takes the embedding too
    t = {"a": torch.randn(3, 5), "b": torch.arange(7, dtype=torch.int32), "c": torch.randn(2, 2).to(torch.bfloat16),
         "e": torch.empty(0, 4)}
    got = parse_safetensors_from_memory(save(t))
    assert set(got) == set(t) and all(torch.equal(got[k], t[k]) and got[k].dtype == t[k].dtype for k in t)


def test_version_store_keeps_the_newest(tmp_path):
    store = RefitVersionStore(root=str(tmp_path), keep=2)
    for ts in (1, 2, 3):
        os.makedirs(store.path_for(ts))
        dropped = store.add(ts)
    assert dropped == [store.path_for(1)] and not os.path.exists(store.path_for(1)) and os.path.exists(store.path_for(3))


def _first_logits(eng, prompt):
    eng.keep_logits = True
    eng.add_request(Request(input_ids=prompt, sampling_params=SamplingParams(max_new_tokens=1, temperature=0.0, ignore_eos=True)))
    while eng.has_work():
        eng.step()
    return eng.last_logits.float().clone()


def test_refit_request_applied_to_a_live_stage(tmp_path):
    """Blocks of a second model's weights, named by content id and split over files (one tensor in two partitions):
    after the refit the live engine computes what the second model computes; a damaged block is refused."""
    from tests.test_engine_gpu import _export_weights

    cfg = named_config("tiny")
    kw = dict(device="cpu", num_blocks=64, page_size=16, max_batch_size=2, max_total_length=128, enable_prefix_cache=False)
    live, other = Engine(cfg, seed=0, **kw), Engine(cfg, seed=7, **kw)
    prompt = list(range(5, 30))
    want = _first_logits(other, prompt)
    assert not torch.allclose(_first_logits(live, prompt), want, atol=1e-3)
    w = _export_weights(other)
    w.pop("lm_head.weight", None)                                  # tied
    big = "model.layers.1.mlp.down_proj.weight"
    full = w.pop(big)
    half = full.shape[0] // 2
    w[big.replace(".weight", ".weight_part0")], w[big.replace(".weight", ".weight_part1")] = full[:half], full[half:]
    names = sorted(w)
    groups = [names[0::3], names[1::3], names[2::3]]
    index_map, paths = {}, {}
    for i, g in enumerate(groups):
        f = tmp_path / f"block{i}.safetensors"
        save_file({k: w[k].contiguous() for k in g}, str(f))
        cid = calculate_cid(f.read_bytes())
        paths[cid] = str(f)
        index_map.update({k: cid for k in g})
    refit = {"time_stamp": 1, "index_map": index_map, "paths": paths}
    used = apply_refit_to_stage(live.stages[0], cfg, refit)
    assert used >= len(names) - 2
    assert torch.allclose(_first_logits(live, prompt), want, atol=1e-4, rtol=1e-4)
    bad = tmp_path / "block0.safetensors"
    raw = bad.read_bytes()
    bad.write_bytes(raw[:-1] + bytes([raw[-1] ^ 0xFF]))
    with pytest.raises(ValueError):
        apply_refit_to_stage(live.stages[0], cfg, refit)


def test_refit_drops_cached_prefixes():
    """K/V pages cached for prefix reuse belong to the weights that computed them: after a refit the same prompt
    must be computed anew, also while a request that started before the refit still runs and publishes blocks."""
    from tests.test_engine_gpu import _export_weights

    cfg = named_config("tiny")
    kw = dict(device="cpu", num_blocks=64, page_size=16, max_batch_size=4, max_total_length=128)
    live, other = Engine(cfg, seed=0, **kw), Engine(cfg, seed=7, **kw)
    prompt = list(range(5, 60))
    want = _first_logits(other, prompt)
    _first_logits(live, prompt)                       # fills the prefix cache of the live engine
    assert live.cache.prefix_cache.num_nodes >= 3
    running = Request(input_ids=prompt[:40] + [7, 7, 7], sampling_params=SamplingParams(max_new_tokens=30, temperature=0.0,
                                                                                      ignore_eos=True))
    live.add_request(running)
    live.step()                                       # a request of the old weights is in flight during the refit
    w = _export_weights(other)
    w.pop("lm_head.weight", None)
    live.update_weights(w)
    while live.has_work():                            # it ends under the new weights and leaves its blocks behind
        live.step()
    hits = live.cache.prefix_cache.hits
    got = _first_logits(live, prompt)
    assert live.cache.prefix_cache.hits == hits       # nothing of the old epoch was matched
    assert torch.allclose(got, want, atol=1e-4, rtol=1e-4)
    assert running.is_finished and not live.cache.reqs


def test_refit_endpoint_of_a_stand_alone_server(tmp_path):
    """`POST /weight/refit` on a server without a scheduler: applied on the engine thread between steps, the next
    reply comes from the new weights; a damaged block is refused with an error and changes nothing."""
    from fastapi.testclient import TestClient
    from safetensors.torch import save_file

    from parallax_b200.engine.service import EngineLoop
    from parallax_b200.frontend.openai_api import create_app
    from parallax_b200.frontend.tokenizer import TokenizerWrapper
    from tests.test_engine_gpu import _export_weights

    cfg = named_config("tiny")
    kw = dict(device="cpu", num_blocks=64, page_size=16, max_batch_size=2, max_total_length=128)
    live, other = Engine(cfg, seed=0, **kw), Engine(cfg, seed=7, **kw)
    w = _export_weights(other)
    w.pop("lm_head.weight", None)
    f = tmp_path / "all.safetensors"
    save_file({k: v.contiguous() for k, v in w.items()}, str(f))
    cid = calculate_cid(f.read_bytes())
    refit = {"time_stamp": 1, "index_map": {k: cid for k in w}, "paths": {cid: str(f)}}
    body = {"prompt": list(range(5, 40)), "max_tokens": 4, "temperature": 0, "ignore_eos": True, "return_probs": True}

    def reply(engine):
        loop = EngineLoop(engine)
        loop.start()
        try:
            with TestClient(create_app(loop, TokenizerWrapper.from_pretrained(None, vocab_size=cfg.vocab_size), "tiny", 128)) as c:
                return c.post("/v1/completions", json=body).json()["choices"][0]["token_probs"]
        finally:
            loop.stop()

    want = reply(other)
    loop = EngineLoop(live)
    loop.start()
    try:
        with TestClient(create_app(loop, TokenizerWrapper.from_pretrained(None, vocab_size=cfg.vocab_size), "tiny", 128)) as c:
            before = c.post("/v1/completions", json=body).json()["choices"][0]["token_probs"]
            assert any(abs(a - b) > 1e-4 for a, b in zip(before, want))
            bad = dict(refit, paths={cid: str(tmp_path / "missing.safetensors")})
            assert c.post("/weight/refit", json=bad).status_code == 400
            r = c.post("/weight/refit", json=refit)
            assert r.status_code == 200 and r.json()["data"]["tensors"] >= len(w) - 1
            after = c.post("/v1/completions", json=body).json()["choices"][0]["token_probs"]
    finally:
        loop.stop()
    assert all(abs(a - b) <= 1e-5 for a, b in zip(after, want)), (after, want)
