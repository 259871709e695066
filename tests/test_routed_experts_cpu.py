"""Routed-experts record (``--enable-return-routed-experts``): every finished request carries, for each of its
tokens that has K/V, the experts each MoE layer routed it to."""

import torch

from parallax_b200.engine.engine import Engine
from parallax_b200.engine.request import Request, SamplingParams
from parallax_b200.models.config import named_config


def _run(prompts, **kw):
    cfg = named_config("tiny-moe")
    torch.manual_seed(0)
    eng = Engine(cfg, device="cpu", num_blocks=128, page_size=16, max_batch_size=4, max_num_tokens_per_batch=256,
                 max_total_length=256, seed=0, return_routed_experts=True, **kw)
    assert eng.return_routed_experts
    reqs = [Request(input_ids=list(p), sampling_params=SamplingParams(max_new_tokens=5, temperature=0.0, ignore_eos=True))
            for p in prompts]
    for r in reqs:
        eng.add_request(r)
    while eng.has_work():
        eng.step()
    return cfg, reqs


def test_record_covers_every_token_and_does_not_depend_on_batching():
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (40, 7, 23)]
    cfg, reqs = _run(prompts, chunked_prefill_size=None, enable_prefix_cache=False)
    for r in reqs:
        rec = torch.tensor(r.routed_experts)
        # the last sampled token was never fed back, so it has no K/V and no routing
        assert rec.shape == (r.prompt_len + len(r.output_ids) - 1, cfg.num_hidden_layers, cfg.num_experts_per_tok)
        assert int(rec.min()) >= 0 and int(rec.max()) < cfg.num_experts
        assert all(len(set(row)) == cfg.num_experts_per_tok for row in rec[:, 0].tolist())      # distinct experts
    # prompt slices of 16 tokens and one request at a time: the same record
    _cfg, chunked = _run(prompts, chunked_prefill_size=16, enable_prefix_cache=False)
    for a, b in zip(reqs, chunked):
        assert a.output_ids == b.output_ids and a.routed_experts == b.routed_experts
    for p, a in zip(prompts, reqs):
        _c, (solo,) = _run([p], chunked_prefill_size=None, enable_prefix_cache=False)
        assert solo.routed_experts == a.routed_experts


def test_tokens_taken_from_the_prefix_cache_keep_their_record():
    g = torch.Generator().manual_seed(4)
    shared = torch.randint(0, 1024, (48,), generator=g).tolist()
    cfg = named_config("tiny-moe")
    torch.manual_seed(0)
    eng = Engine(cfg, device="cpu", num_blocks=128, page_size=16, max_batch_size=4, max_num_tokens_per_batch=256,
                 max_total_length=256, seed=0, return_routed_experts=True)
    sp = SamplingParams(max_new_tokens=3, temperature=0.0, ignore_eos=True)
    first = Request(input_ids=shared + [5, 6, 7], sampling_params=sp)
    eng.add_request(first)
    while eng.has_work():
        eng.step()
    second = Request(input_ids=shared + [9, 9], sampling_params=SamplingParams.from_dict(sp.to_dict()))
    eng.add_request(second)
    while eng.has_work():
        eng.step()
    assert eng.cache.prefix_cache.hits > 0
    assert second.routed_experts[:48] == first.routed_experts[:48]
    assert len(second.routed_experts) == 50 + 3 - 1


def test_dense_model_leaves_the_record_off():
    eng = Engine(named_config("tiny"), device="cpu", num_blocks=32, page_size=16, max_batch_size=2, max_total_length=128,
                 return_routed_experts=True)
    assert not eng.return_routed_experts


def test_record_in_the_http_reply():
    from fastapi.testclient import TestClient

    from parallax_b200.engine.service import EngineLoop
    from parallax_b200.frontend.openai_api import create_app
    from parallax_b200.frontend.tokenizer import ByteTokenizer, TokenizerWrapper

    cfg = named_config("tiny-moe")
    eng = Engine(cfg, device="cpu", num_blocks=128, page_size=16, max_batch_size=4, return_routed_experts=True)
    loop = EngineLoop(eng)
    loop.start()
    app = create_app(loop, TokenizerWrapper(ByteTokenizer(), vocab_size=cfg.vocab_size), "tiny-moe", max_model_len=512)
    try:
        with TestClient(app) as c:
            r = c.post("/v1/completions", json={"model": "tiny-moe", "prompt": [3, 4, 5, 6, 7], "max_tokens": 4,
                                                "temperature": 0, "ignore_eos": True}).json()
        rec = r["choices"][0]["routed_experts"]
        assert len(rec) == 5 + 4 - 1 and len(rec[0]) == cfg.num_hidden_layers and len(rec[0][0]) == cfg.num_experts_per_tok
    finally:
        loop.stop()
