"""Three pipeline peers chained in one process with the wire emulated: every hop goes through
request_to_proto / proto_to_request, as the reference's executor test does
(tests/test_executor.py:67-285). The result must equal the single-engine run."""

import torch

from parallax_b200.engine.engine import Engine
from parallax_b200.engine.peer import PeerExecutor
from parallax_b200.engine.request import Request, SamplingParams
from parallax_b200.models.config import named_config
from parallax_b200.p2p.message_util import proto_to_request, request_to_proto


def _wire(packets):
    return proto_to_request(request_to_proto(packets)) if packets else []


def _prompts(n, length, vocab, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (length,), generator=g).tolist() for _ in range(n)]


def _run_pipeline(cfg, spans, prompts, max_new, **kw):
    peers = [PeerExecutor(cfg, s, e, device="cpu", node_id=f"n{i}", num_blocks=128, max_batch_size=8, **kw)
             for i, (s, e) in enumerate(spans)]
    table = [p.node_id for p in peers]
    reqs = [Request(input_ids=p, routing_table=table,
                    sampling_params=SamplingParams(max_new_tokens=max_new, temperature=0.0, ignore_eos=True))
            for p in prompts]
    for r in reqs:
        peers[0].add_request(r)
    steps = 0
    while peers[0].has_work() and steps < 500:
        steps += 1
        packets, _events, releases = peers[0].step_first()
        for peer in peers[1:]:
            peer.release(releases)
        back = []
        for peer in peers[1:]:
            packets = peer.process_packets(_wire(packets))
            back = packets
        if len(peers) > 1:
            _events, releases = peers[0].receive_tokens(_wire([p for p in back if p.hidden_states is None]))
            for peer in peers[1:]:
                peer.release(releases)
    return [r.output_ids for r in reqs], peers


def test_three_peers_match_single_engine():
    cfg = named_config("tiny")
    prompts = _prompts(3, 41, cfg.vocab_size, seed=4)
    want = Engine(cfg, device="cpu", num_blocks=128, max_batch_size=8).generate(
        prompts, SamplingParams(max_new_tokens=9, temperature=0.0, ignore_eos=True))
    got, peers = _run_pipeline(cfg, [(0, 1), (1, 3), (3, 4)], prompts, 9)
    assert got == want
    # every peer released every request
    for p in peers:
        assert not p.cache.reqs and not p.mirror


def test_chunked_prefill_streams_through_peers_and_prefix_cache_is_per_peer():
    cfg = named_config("tiny")
    prompts = _prompts(2, 100, cfg.vocab_size, seed=5)
    want = Engine(cfg, device="cpu", num_blocks=128, max_batch_size=8, chunked_prefill_size=None,
                  enable_prefix_cache=False).generate(prompts, SamplingParams(max_new_tokens=5, temperature=0.0,
                                                                              ignore_eos=True))
    got, peers = _run_pipeline(cfg, [(0, 2), (2, 4)], prompts, 5, chunked_prefill_size=32)
    assert got == want
    assert all(p.cache.prefix_cache.num_nodes >= 2 * (100 // 16) for p in peers)


def test_single_peer_pipeline_samples_locally():
    cfg = named_config("tiny")
    prompts = _prompts(2, 20, cfg.vocab_size, seed=6)
    want = Engine(cfg, device="cpu", num_blocks=64, max_batch_size=8).generate(
        prompts, SamplingParams(max_new_tokens=4, temperature=0.0, ignore_eos=True))
    got, _ = _run_pipeline(cfg, [(0, 4)], prompts, 4)
    assert got == want


def test_peer_without_the_prefix_aborts_the_request():
    cfg = named_config("tiny")
    first = PeerExecutor(cfg, 0, 2, device="cpu", node_id="a", num_blocks=64)
    last = PeerExecutor(cfg, 2, 4, device="cpu", node_id="b", num_blocks=64)
    prompt = _prompts(1, 48, cfg.vocab_size, seed=7)[0]
    # warm only the first peer's prefix cache
    warm = Request(input_ids=prompt, routing_table=["a", "b"],
                   sampling_params=SamplingParams(max_new_tokens=1, temperature=0.0, ignore_eos=True))
    first.add_request(warm)
    pk, _, _ = first.step_first()
    first.receive_tokens(_wire(last.process_packets(_wire(pk))))
    last.release([warm.request_id])
    last.cache.prefix_cache.reset()
    again = Request(input_ids=prompt, routing_table=["a", "b"],
                    sampling_params=SamplingParams(max_new_tokens=2, temperature=0.0, ignore_eos=True))
    first.add_request(again)
    pk, _, _ = first.step_first()
    assert pk[0].chunk_start > 0                                   # first peer skipped cached tokens
    back = last.process_packets(_wire(pk))
    assert back and back[0].abort
    events, releases = first.receive_tokens(_wire(back))
    assert again.is_finished and releases == [again.request_id]


def test_later_peer_out_of_kv_drops_only_that_request():
    """The second peer runs out of KV blocks while decoding: the request that cannot get a block is
    aborted, and the requests behind it in the batch keep their own activations (same tokens as an
    engine with enough memory)."""
    cfg = named_config("tiny")
    prompts = _prompts(3, 15, cfg.vocab_size, seed=11)      # one 16-token page each
    sp = dict(max_new_tokens=6, temperature=0.0, ignore_eos=True)
    want = Engine(cfg, device="cpu", num_blocks=128, max_batch_size=8).generate(prompts, SamplingParams(**sp))
    peers = [PeerExecutor(cfg, 0, 2, device="cpu", node_id="n0", num_blocks=128, max_batch_size=8),
             PeerExecutor(cfg, 2, 4, device="cpu", node_id="n1", num_blocks=5, max_batch_size=8, enable_prefix_cache=False)]
    table = [p.node_id for p in peers]
    reqs = [Request(input_ids=p, routing_table=table, sampling_params=SamplingParams(**sp)) for p in prompts]
    for r in reqs:
        peers[0].add_request(r)
    steps = 0
    while peers[0].has_work() and steps < 100:
        steps += 1
        packets, _events, releases = peers[0].step_first()
        peers[1].release(releases)
        back = peers[1].process_packets(_wire(packets))
        _events, releases = peers[0].receive_tokens(_wire([p for p in back if p.hidden_states is None]))
        peers[1].release(releases)
    aborted = [r for r in reqs if r.status.value == "FINISHED_ABORT"]
    done = [r for r in reqs if r.status.value == "FINISHED_MAX_LENGTH"]
    assert len(aborted) == 1 and len(done) == 2, [r.status for r in reqs]
    for r in done:
        assert r.output_ids == want[reqs.index(r)]
    # the aborted request produced correct tokens up to the point where it was dropped
    a = aborted[0]
    assert a.output_ids == want[reqs.index(a)][:len(a.output_ids)]


def test_per_request_adapters_travel_with_the_packets(tmp_path):
    """Every peer keeps the adapter slots of its own layers and loads an adapter when the first packet that names it
    arrives; the chained peers produce what the single engine with the same adapters produces, and every pin is
    released at the end."""
    from tests.test_lora_cpu import _make_adapter

    cfg = named_config("tiny")
    lora = {"max_loaded": 2, "max_rank": 8,
            "paths": {"x": _make_adapter(cfg, tmp_path / "x", 1), "y": _make_adapter(cfg, tmp_path / "y", 2, rank=8, alpha=4)}}
    prompts = _prompts(4, 27, cfg.vocab_size, seed=8)
    lora_of = ["x", None, "y", "x"]
    sp = dict(max_new_tokens=5, temperature=0.0, ignore_eos=True)
    eng = Engine(cfg, device="cpu", num_blocks=128, max_batch_size=8, lora=lora)
    ref = [Request(input_ids=p, sampling_params=SamplingParams(**sp), lora_path=a) for p, a in zip(prompts, lora_of)]
    for r in ref:
        eng.add_request(r)
    while eng.has_work():
        eng.step()
    peers = [PeerExecutor(cfg, s, e, device="cpu", node_id=f"n{i}", num_blocks=128, max_batch_size=8, lora=lora)
             for i, (s, e) in enumerate([(0, 1), (1, 3), (3, 4)])]
    table = [p.node_id for p in peers]
    reqs = [Request(input_ids=p, routing_table=table, sampling_params=SamplingParams(**sp), lora_path=a)
            for p, a in zip(prompts, lora_of)]
    for r in reqs:
        peers[0].add_request(r)
    steps = 0
    while peers[0].has_work() and steps < 300:
        steps += 1
        packets, _events, releases = peers[0].step_first()
        for peer in peers[1:]:
            peer.release(releases)
        back = []
        for peer in peers[1:]:
            packets = peer.process_packets(_wire(packets))
            back = packets
        _events, releases = peers[0].receive_tokens(_wire([p for p in back if p.hidden_states is None]))
        for peer in peers[1:]:
            peer.release(releases)
    assert [r.output_ids for r in reqs] == [r.output_ids for r in ref]
    base = Engine(cfg, device="cpu", num_blocks=128, max_batch_size=8).generate(prompts, SamplingParams(**sp))
    assert reqs[1].output_ids == base[1] and (reqs[0].output_ids != base[0] or reqs[2].output_ids != base[2])
    for p in peers:
        assert not any(p.lora.pins.values()) and not p.mirror and not p.cache.reqs


def test_constrained_requests_through_chained_peers():
    """The last peer samples under the request's JSON schema, the first peer notices the end of the document: the reply
    is a valid document and equals the single engine's; the unconstrained request next to it is untouched."""
    import json

    from parallax_b200.engine.structured import JsonSchemaMatcher
    from parallax_b200.frontend.tokenizer import TokenizerWrapper

    cfg = named_config("tiny")
    tok = TokenizerWrapper.from_pretrained(None, vocab_size=cfg.vocab_size)
    schema = {"type": "object", "properties": {"ok": {"type": "boolean"}, "n": {"type": "integer"}}, "required": ["ok", "n"]}
    prompts = [[t % 250 for t in p] for p in _prompts(2, 19, cfg.vocab_size, seed=9)]
    sps = [dict(max_new_tokens=120, temperature=0.0, json_schema=json.dumps(schema)),
           dict(max_new_tokens=5, temperature=0.0, ignore_eos=True)]
    eng = Engine(cfg, device="cpu", num_blocks=128, max_batch_size=8, tokenizer=tok)
    ref = [Request(input_ids=p, sampling_params=SamplingParams(**sp)) for p, sp in zip(prompts, sps)]
    for r in ref:
        eng.add_request(r)
    while eng.has_work():
        eng.step()
    for spans in ([(0, 4)], [(0, 2), (2, 4)]):
        peers = [PeerExecutor(cfg, s, e, device="cpu", node_id=f"n{i}", num_blocks=128, max_batch_size=8)
                 for i, (s, e) in enumerate(spans)]
        for p in peers:
            p.tokenizer = tok
        table = [p.node_id for p in peers]
        reqs = [Request(input_ids=p, routing_table=table, sampling_params=SamplingParams(**sp)) for p, sp in zip(prompts, sps)]
        for r in reqs:
            peers[0].add_request(r)
        steps = 0
        while peers[0].has_work() and steps < 400:
            steps += 1
            packets, _events, releases = peers[0].step_first()
            for peer in peers[1:]:
                peer.release(releases)
            back = []
            for peer in peers[1:]:
                packets = peer.process_packets(_wire(packets))
                back = packets
            if len(peers) > 1:
                _events, releases = peers[0].receive_tokens(_wire([p for p in back if p.hidden_states is None]))
                for peer in peers[1:]:
                    peer.release(releases)
        text = tok.decode(reqs[0].output_ids)
        m = JsonSchemaMatcher(schema)
        assert m.advance(text) and m.done and set(json.loads(text)) >= {"ok", "n"}, text
        assert reqs[0].status.name == "FINISHED_EOS" and len(reqs[0].output_ids) < 120
        assert [r.output_ids for r in reqs] == [r.output_ids for r in ref]
        assert not peers[-1]._grammars and not any(p.cache.reqs for p in peers)


def test_every_model_family_through_chained_peers():
    """MLA, sparse-indexer, block-sparse, hybrid (recurrent state slots) and MoE models split over two peers, with
    prompts that share a prefix and prompt slices, against the single engine."""
    for name in ("tiny-hybrid", "tiny-mla", "tiny-dsa", "tiny-msa", "tiny-moe"):
        cfg = named_config(name)
        L = cfg.num_hidden_layers
        g = torch.Generator().manual_seed(1)
        shared = torch.randint(0, cfg.vocab_size, (40,), generator=g).tolist()
        prompts = [shared + torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (5, 9)] \
            + _prompts(1, 23, cfg.vocab_size, seed=3)
        want = Engine(cfg, device="cpu", num_blocks=128, max_batch_size=8).generate(
            prompts, SamplingParams(max_new_tokens=5, temperature=0.0, ignore_eos=True))
        got, peers = _run_pipeline(cfg, [(0, L // 2), (L // 2, L)], prompts, 5, chunked_prefill_size=16)
        assert got == want, name
        for p in peers:
            assert not p.cache.reqs and not p.mirror, name


def test_request_time_out_releases_every_peer():
    """The time-out counts the time without progress (as in the reference, ``src/parallax/server/scheduler.py:314-333``):
    when the next peer stops answering, the first peer aborts the request after `request_timeout_s`, every peer releases
    it, and the pipeline serves the next request as if nothing had happened."""
    import time

    cfg = named_config("tiny")
    peers = [PeerExecutor(cfg, s, e, device="cpu", node_id=f"n{i}", num_blocks=64, max_batch_size=4, request_timeout_s=0.3)
             for i, (s, e) in enumerate([(0, 2), (2, 4)])]
    table = [p.node_id for p in peers]
    slow = Request(input_ids=list(range(3, 30)), routing_table=table,
                   sampling_params=SamplingParams(max_new_tokens=500, temperature=0.0, ignore_eos=True))
    peers[0].add_request(slow)
    events, pending_releases = [], []
    deadline = time.time() + 20
    steps = 0
    while peers[0].has_work() and time.time() < deadline:
        steps += 1
        packets, ev, releases = peers[0].step_first()
        events += ev
        pending_releases += releases
        if steps <= 5:                                   # the second peer answers for five steps, then goes silent
            back = peers[1].process_packets(_wire(packets))
            ev, releases = peers[0].receive_tokens(_wire([p for p in back if p.hidden_states is None]))
            events += ev
            pending_releases += releases
        time.sleep(0.02)
    assert slow.status.name == "FINISHED_ABORT" and 0 < len(slow.output_ids) <= 5
    assert any(r is slow and r.is_finished for r, _t in events) and slow.request_id in pending_releases
    peers[1].release(pending_releases)                   # the abort notice reaches the silent peer when it is back
    for p in peers:
        assert not p.cache.reqs and not p.mirror
    got, _ = _run_pipeline(cfg, [(0, 2), (2, 4)], _prompts(1, 12, cfg.vocab_size, seed=1), 3)
    assert len(got[0]) == 3


def test_e4m3_kv_pages_through_chained_peers():
    cfg = named_config("tiny")
    prompts = _prompts(3, 37, cfg.vocab_size, seed=2)
    want = Engine(cfg, device="cpu", num_blocks=128, max_batch_size=8, kv_cache_dtype="fp8_e4m3").generate(
        prompts, SamplingParams(max_new_tokens=6, temperature=0.0, ignore_eos=True))
    got, peers = _run_pipeline(cfg, [(0, 2), (2, 4)], prompts, 6, kv_cache_dtype="fp8_e4m3")
    assert got == want
    assert all(p.worker.pool.layers[0].kv_scale is not None for p in peers)
