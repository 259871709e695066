"""End-to-end engine checks on CPU (fp32, reference ops): sharding, chunked prefill, prefix
cache and agreement with HuggingFace's implementation of the same architecture."""

import pytest
import torch

from parallax_b200.engine.engine import Engine
from parallax_b200.engine.request import Request, SamplingParams
from parallax_b200.models.config import config_from_hf, named_config


def _prompts(n, length, vocab, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (length,), generator=g).tolist() for _ in range(n)]


def _run(cfg, prompts, max_new=8, **kw):
    eng = Engine(cfg, device="cpu", num_blocks=256, page_size=16, max_batch_size=8, **kw)
    return eng.generate(prompts, SamplingParams(max_new_tokens=max_new, temperature=0.0, ignore_eos=True))


def test_sharded_equals_unsharded_tiny():
    cfg = named_config("tiny")
    prompts = _prompts(4, 37, cfg.vocab_size)
    full = _run(cfg, prompts)
    two = _run(cfg, prompts, stage_layers=[(0, 2), (2, 4)])
    three = _run(cfg, prompts, stage_layers=[(0, 1), (1, 3), (3, 4)])
    assert full == two == three
    assert all(len(o) == 8 for o in full)


def test_chunked_prefill_and_prefix_cache_do_not_change_outputs():
    cfg = named_config("tiny")
    prompts = _prompts(3, 100, cfg.vocab_size, seed=1)
    base = _run(cfg, prompts, chunked_prefill_size=None, enable_prefix_cache=False)
    chunked = _run(cfg, prompts, chunked_prefill_size=32, enable_prefix_cache=False)
    assert base == chunked
    # same prompts twice through one engine: second pass must hit the prefix cache
    eng = Engine(cfg, device="cpu", num_blocks=256, page_size=16, max_batch_size=8)
    sp = SamplingParams(max_new_tokens=8, temperature=0.0, ignore_eos=True)
    first = eng.generate(prompts, sp)
    second = eng.generate(prompts, sp)
    assert first == base and second == base
    assert eng.cache.prefix_cache.hits >= 3


def test_matches_huggingface_qwen3():
    transformers = pytest.importorskip("transformers")
    hf_cfg = transformers.Qwen3Config(
        hidden_size=128, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2, head_dim=32,
        intermediate_size=256, vocab_size=512, rope_theta=10000.0, tie_word_embeddings=False,
        max_position_embeddings=512, rms_norm_eps=1e-6)
    torch.manual_seed(0)
    hf = transformers.Qwen3ForCausalLM(hf_cfg).eval().float()
    cfg = config_from_hf(hf_cfg.to_dict() | {"architectures": ["Qwen3ForCausalLM"]})
    weights = {k: v.detach().clone() for k, v in hf.state_dict().items()}
    eng = Engine(cfg, device="cpu", num_blocks=64, page_size=16, max_batch_size=4, weights=weights,
                 stage_layers=[(0, 2), (2, 3)])
    eng.keep_logits = True
    prompt = _prompts(1, 29, 512, seed=3)[0]
    req = Request(input_ids=prompt, sampling_params=SamplingParams(max_new_tokens=6, temperature=0.0, ignore_eos=True))
    eng.add_request(req)
    eng.step()
    with torch.no_grad():
        want = hf(torch.tensor([prompt])).logits[0, -1]
    assert torch.allclose(eng.last_logits[0], want, atol=2e-4, rtol=1e-3)
    while eng.has_work():
        eng.step()
    with torch.no_grad():
        gen = hf.generate(torch.tensor([prompt]), max_new_tokens=6, do_sample=False)[0, len(prompt):].tolist()
    assert req.output_ids == gen


@pytest.mark.slow
def test_cpu_plumbing_qwen3_0p6b_two_shards():
    """Qwen3-0.6B shape, fp32, 2 shards x 14 layers, page 16, 4 x 128-token prompts, greedy 32
    tokens; the sharded pipeline must reproduce the unsharded model's logits."""
    cfg = named_config("qwen3-0.6b")
    prompts = _prompts(4, 128, cfg.vocab_size, seed=7)
    sp = SamplingParams(max_new_tokens=32, temperature=0.0, ignore_eos=True)
    outs, logits = [], []
    for layers in ([(0, 28)], [(0, 14), (14, 28)]):
        eng = Engine(cfg, device="cpu", num_blocks=64, page_size=16, max_batch_size=4, stage_layers=layers)
        eng.keep_logits = True
        reqs = [Request(input_ids=p, sampling_params=SamplingParams.from_dict(sp.to_dict())) for p in prompts]
        for r in reqs:
            eng.add_request(r)
        trace = []
        while eng.has_work():
            eng.step()
            trace.append(eng.last_logits.clone())
        outs.append([r.output_ids for r in reqs])
        logits.append(trace)
    assert outs[0] == outs[1]
    assert len(logits[0]) == len(logits[1])
    for a, b in zip(logits[0], logits[1]):
        assert torch.allclose(a, b, atol=1e-4, rtol=1e-4)


def test_moe_engine_matches_huggingface_qwen3_moe():
    transformers = pytest.importorskip("transformers")
    hf_cfg = transformers.Qwen3MoeConfig(
        hidden_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=32,
        intermediate_size=256, moe_intermediate_size=64, num_experts=8, num_experts_per_tok=2, norm_topk_prob=True,
        vocab_size=512, rope_theta=10000.0, tie_word_embeddings=False, max_position_embeddings=512,
        decoder_sparse_step=1, mlp_only_layers=[])
    torch.manual_seed(0)
    hf = transformers.Qwen3MoeForCausalLM(hf_cfg).eval().float()
    cfg = config_from_hf(hf_cfg.to_dict() | {"architectures": ["Qwen3MoeForCausalLM"]})
    assert cfg.is_moe and cfg.layer_is_moe(0)
    sd = {k: v.detach().clone() for k, v in hf.state_dict().items()}
    # newer HF releases store experts fused: split them back into per-expert tensors
    for li in range(2):
        p = f"model.layers.{li}.mlp.experts."
        if p + "gate_up_proj" in sd:
            gu, dn = sd.pop(p + "gate_up_proj"), sd.pop(p + "down_proj")
            for e in range(8):
                g_u = gu[e] if gu[e].shape[0] == 128 else gu[e].t()
                sd[f"{p}{e}.gate_proj.weight"], sd[f"{p}{e}.up_proj.weight"] = g_u[:64], g_u[64:]
                sd[f"{p}{e}.down_proj.weight"] = dn[e] if dn[e].shape == (128, 64) else dn[e].t()
    eng = Engine(cfg, device="cpu", num_blocks=64, page_size=16, max_batch_size=4, weights=sd)
    eng.keep_logits = True
    prompt = _prompts(1, 23, 512, seed=9)[0]
    req = Request(input_ids=prompt, sampling_params=SamplingParams(max_new_tokens=4, temperature=0.0, ignore_eos=True))
    eng.add_request(req)
    eng.step()
    with torch.no_grad():
        want = hf(torch.tensor([prompt])).logits[0, -1]
    assert torch.allclose(eng.last_logits[0], want, atol=3e-4, rtol=1e-3)


def test_tiny_moe_sharded_equals_unsharded():
    cfg = named_config("tiny-moe")
    prompts = _prompts(3, 30, cfg.vocab_size, seed=11)
    assert _run(cfg, prompts, max_new=5) == _run(cfg, prompts, max_new=5, stage_layers=[(0, 2), (2, 4)])


def test_step_tracer_writes_chrome_trace(tmp_path):
    import json

    path = tmp_path / "trace.json"
    eng = Engine(named_config("tiny"), device="cpu", num_blocks=64, page_size=16, max_batch_size=4, trace=str(path))
    eng.generate(_prompts(2, 20, 1024, seed=3), SamplingParams(max_new_tokens=3, temperature=0.0, ignore_eos=True))
    eng.tracer.save()
    ev = json.loads(path.read_text())["traceEvents"]
    names = {e["name"] for e in ev}
    assert {"schedule+plan", "build+launch", "wait for tokens", "commit"} <= names
    assert all(e["dur"] > 0 for e in ev)


def test_scheduler_prefill_cap_spreads_a_prompt_over_batches():
    """With a per-batch cap on prompt tokens a long prompt is prefilled in consecutive slices while the
    decode rows of the other requests ride along in every batch."""
    from parallax_b200.engine.request import Request, SamplingParams
    from parallax_b200.engine.scheduler import BatchScheduler

    sched = BatchScheduler(max_batch_size=8, max_num_tokens_per_batch=4096, chunked_prefill_size=None,
                           max_prefill_tokens_per_batch=100)
    sp = SamplingParams(max_new_tokens=4, temperature=0.0, ignore_eos=True)
    long_req = Request(input_ids=list(range(250)), sampling_params=sp)
    short = Request(input_ids=list(range(40)), sampling_params=sp)
    sched.enque_request(long_req)
    sched.enque_request(short)
    seen = []
    for _ in range(5):
        batch = sched.form_batch()
        seen.append([(s.req is long_req, s.num_tokens, s.is_prefill) for s in batch])
        for s in batch:
            if s.is_prefill:
                s.req.num_computed_tokens = s.start + s.num_tokens
                if s.produces_token:
                    s.req.commit_new_token(1)
            else:
                s.req.commit_new_token(1)
            sched.enque_request(s.req)
    for batch in seen:
        assert sum(n for _, n, p in batch if p) <= 100
    slices = [n for batch in seen for is_long, n, p in batch if is_long and p]
    assert sum(slices) == 250 and len(slices) >= 3
    assert sum(n for batch in seen for is_long, n, p in batch if not is_long and p) == 40
    # once the short prompt is done its decode rows share batches with the long prompt's slices
    assert any(any(p for _, _, p in batch) and any(not p for _, _, p in batch) for batch in seen)


def test_nonzero_device_status_fails_the_batch():
    """A kernel that gave up (here: a faked status word) must not let the step commit tokens: the
    step raises and the serving loop releases the running requests with an error event."""
    import time

    from parallax_b200.engine.service import EngineLoop
    from parallax_b200.ops import KernelError

    cfg = named_config("tiny")
    eng = Engine(cfg, device="cpu", num_blocks=64, max_batch_size=4)
    calls = {"n": 0}

    def fake_status():
        calls["n"] += 1
        return 105 if calls["n"] == 3 else 0      # the third step reports "wait on a peer flag ran out"

    eng._step_status = fake_status
    r = Request(input_ids=[1, 2, 3, 4, 5], sampling_params=SamplingParams(max_new_tokens=8, temperature=0.0, ignore_eos=True))
    eng.add_request(r)
    eng.step()
    eng.step()
    n_before = len(r.output_ids)
    with pytest.raises(KernelError, match="peer flag"):
        eng.step()
    assert len(r.output_ids) == n_before          # nothing of the failed step was committed

    # through the serving loop: the request ends with an ERROR event, the loop keeps running
    eng2 = Engine(cfg, device="cpu", num_blocks=64, max_batch_size=4)
    calls2 = {"n": 0}

    def fake_status2():
        calls2["n"] += 1
        return 106 if calls2["n"] == 2 else 0

    eng2._step_status = fake_status2
    loop = EngineLoop(eng2)
    loop.start()
    q = loop.submit(Request(input_ids=[7, 8, 9], sampling_params=SamplingParams(max_new_tokens=20, temperature=0.0, ignore_eos=True)))
    evs = []
    t0 = time.time()
    while time.time() - t0 < 30:
        ev = q.get(timeout=30)
        evs.append(ev)
        if ev.finished:
            break
    assert evs[-1].finished and evs[-1].error and "index out of range" in evs[-1].error
    # a new request after the failure is served normally
    q2 = loop.submit(Request(input_ids=[3, 4], sampling_params=SamplingParams(max_new_tokens=3, temperature=0.0, ignore_eos=True)))
    toks = []
    while True:
        ev = q2.get(timeout=30)
        if ev.token_id is not None:
            toks.append(ev.token_id)
        if ev.finished:
            break
    loop.stop()
    assert len(toks) == 3 and ev.error is None


def test_async_scheduling_matches_synchronous_steps():
    """Launching step s before reading the tokens of step s-1 (decode input ids patched on the device,
    placeholders on the host) must not change any result: same tokens, same finish reasons, also when a
    request ends on an EOS / stop token that is only seen one step late, with chunked prompts, shared
    prefixes and more requests than batch slots."""
    cfg = named_config("tiny")
    g = torch.Generator().manual_seed(5)
    shared = torch.randint(0, cfg.vocab_size, (40,), generator=g).tolist()
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (5, 33, 70, 18, 9, 50, 3)]
    prompts[2][:40] = shared
    prompts[5][:40] = shared

    def run(async_mode, eos=None, stop=None, min_new=0):
        eng = Engine(cfg, device="cpu", num_blocks=128, max_batch_size=4, max_num_tokens_per_batch=96,
                     chunked_prefill_size=32, eos_token_id=eos, async_scheduling=async_mode)
        reqs = [Request(input_ids=p, sampling_params=SamplingParams(max_new_tokens=12, temperature=0.0,
                                                                    stop_token_ids=stop, min_new_tokens=min_new))
                for p in prompts]
        for r in reqs:
            eng.add_request(r)
        events, steps = [], 0
        while eng.has_work() and steps < 400:
            events += eng.step()
            steps += 1
        events += eng.flush()
        assert not eng.cache.reqs, "every request released its KV blocks"
        streamed = {}
        for req, tok in events:
            if tok is not None:
                streamed.setdefault(req.request_id, []).append(tok)
        for r in reqs:
            assert streamed.get(r.request_id, []) == r.output_ids      # every token was reported exactly once
            assert -1 not in r.output_ids
        return [r.output_ids for r in reqs], [r.status.value for r in reqs]

    base, status = run(False)
    assert run(True) == (base, status)
    # an EOS that really occurs: the token request 1 produced third
    eos = base[1][2]
    want = run(False, eos=eos)
    assert any(s == "FINISHED_EOS" for s in want[1])
    assert run(True, eos=eos) == want
    # stop ids and min_new_tokens
    stop = [base[0][1], base[3][4]]
    want = run(False, stop=stop, min_new=2)
    assert run(True, stop=stop, min_new=2) == want


def test_sampling_penalties_change_greedy_output_as_specified():
    """Repetition / presence / frequency penalties reach the logits: a greedy run with a strong frequency
    penalty never repeats a token, the penalty math equals a hand computation, and a run with neutral
    penalties equals the plain run (asynchronous scheduling falls back to step-by-step for such rows)."""
    from parallax_b200.engine.sampling import apply_penalties, build_penalties
    from parallax_b200.ops import reference as ref

    cfg = named_config("tiny")
    prompt = [3, 7, 7, 11, 250, 9]

    def gen(async_mode=False, **pen):
        eng = Engine(cfg, device="cpu", num_blocks=64, max_batch_size=4, async_scheduling=async_mode)
        return eng.generate([prompt], SamplingParams(max_new_tokens=24, temperature=0.0, ignore_eos=True, **pen))[0]

    plain = gen()
    assert gen(repetition_penalty=1.0, presence_penalty=0.0, frequency_penalty=0.0) == plain
    strong = gen(frequency_penalty=2.0, presence_penalty=2.0)
    assert len(set(strong)) > len(set(plain)) or len(set(plain)) == len(plain)
    assert gen(async_mode=True, frequency_penalty=2.0, presence_penalty=2.0) == strong
    # the arithmetic
    r = Request(input_ids=[1, 2, 2, 5], sampling_params=SamplingParams(repetition_penalty=2.0, presence_penalty=0.5,
                                                                       frequency_penalty=0.25))
    r.output_ids = [5, 9, 9, -1]
    logits = torch.tensor([[4.0, -4.0, 2.0, 1.0, 0.0, 8.0, 0.0, 0.0, 0.0, -2.0]])
    got = apply_penalties(logits.clone(), build_penalties([r]))
    want = logits.clone()
    want[0, 1] = -8.0                      # prompt token, negative logit: multiplied
    want[0, 2] = 1.0                       # prompt token, positive logit: divided
    want[0, 5] = 8.0 / 2 - (0.25 * 1 + 0.5)    # prompt + generated once
    want[0, 9] = -2.0 * 2 - (0.25 * 2 + 0.5)   # generated twice
    assert torch.allclose(got, want)


def test_positions_beyond_the_advertised_context_length():
    """A checkpoint whose config advertises a shorter context than the engine is asked to serve: the rotary table
    follows the engine's ``max_total_length`` (not the advertised length), and a request cannot outgrow the engine's
    own limit even if it asks for more."""
    import copy

    cfg = copy.copy(named_config("tiny"))
    cfg.max_position_embeddings = 64
    eng = Engine(cfg, device="cpu", num_blocks=64, page_size=16, max_batch_size=2, chunked_prefill_size=32,
                 max_total_length=160, seed=0)
    assert eng.stages[0].model.cos_sin.shape[0] >= 160
    ref = Engine(named_config("tiny"), device="cpu", num_blocks=64, page_size=16, max_batch_size=2,
                 chunked_prefill_size=32, max_total_length=160, seed=0)
    prompt = [(7 * i + 1) % 1000 for i in range(100)]          # positions 0..120 cross the advertised 64
    sp = SamplingParams(max_new_tokens=20, temperature=0.0, ignore_eos=True)
    assert eng.generate([prompt], sp) == ref.generate([prompt], sp)
    # asks for 10000 tokens in total: stops at the engine's 160
    r = Request(input_ids=prompt, sampling_params=SamplingParams(max_new_tokens=500, temperature=0.0, ignore_eos=True),
                max_total_length=10000)
    eng.add_request(r)
    while eng.has_work():
        eng.step()
    assert len(r.input_ids) + len(r.output_ids) <= 160 and len(r.output_ids) >= 50


def test_a_backlog_of_prompt_tokens_does_not_starve_decoding_requests():
    """Token budget = one prompt slice + one row per request. While a long prompt is being prefilled slice by
    slice, a request that is already decoding gets a token in every step (its row is reserved before prompt
    slices are cut to fill the budget)."""
    cfg = named_config("tiny")
    eng = Engine(cfg, device="cpu", num_blocks=128, page_size=16, max_batch_size=4, chunked_prefill_size=32,
                 max_num_tokens_per_batch=32 + 4, enable_prefix_cache=False, max_total_length=512, seed=0,
                 async_scheduling=False)
    short = Request(input_ids=[3, 4, 5, 6, 7], sampling_params=SamplingParams(max_new_tokens=30, temperature=0.0,
                                                                               ignore_eos=True))
    eng.add_request(short)
    eng.step()
    assert len(short.output_ids) == 1
    longs = [Request(input_ids=[(11 * i + j) % 1000 for i in range(200)],
                     sampling_params=SamplingParams(max_new_tokens=2, temperature=0.0, ignore_eos=True)) for j in range(2)]
    for r in longs:
        eng.add_request(r)
    produced = []
    for _ in range(10):                       # 400 prompt tokens at <= 35 per step: the backlog outlasts these steps
        before = len(short.output_ids)
        eng.step()
        st = eng.last_step_stats
        assert st["tokens"] <= 36
        produced.append(len(short.output_ids) - before)
        assert st["prefill_tokens"] >= 30      # the prompt slices still take (almost) the whole budget
    assert produced == [1] * 10, produced


def test_abort_of_a_waiting_request_closes_its_stream():
    """A request aborted before it was ever admitted (the running set is full) ends with one finished event, so that
    whoever waits on its stream is released and the loop's stream table does not grow."""
    from parallax_b200.engine.service import EngineLoop

    cfg = named_config("tiny")
    eng = Engine(cfg, device="cpu", num_blocks=64, page_size=16, max_batch_size=1, max_total_length=256)
    loop = EngineLoop(eng)
    long_sp = SamplingParams(max_new_tokens=60, temperature=0.0, ignore_eos=True)
    first = Request(input_ids=list(range(3, 20)), sampling_params=long_sp)
    waiting = Request(input_ids=list(range(5, 12)), sampling_params=SamplingParams.from_dict(long_sp.to_dict()))
    q1 = loop.submit(first)
    q2 = loop.submit(waiting)
    loop.abort(waiting.request_id)          # queued behind the add: the request is still waiting when it is cancelled
    loop.start()
    try:
        ev = q2.get(timeout=30)
        assert ev.finished and ev.token_id is None and waiting.status.name == "CANCELLED"
        loop.abort(first.request_id)
        while True:
            ev = q1.get(timeout=30)
            if ev.finished:
                break
        assert loop.num_inflight == 0
    finally:
        loop.stop()
