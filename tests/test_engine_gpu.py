"""The engine on B200 (bf16, sm_100a kernels) against the same engine on CPU (fp32, reference ops)."""

import pytest
import torch

from parallax_b200.engine.engine import Engine
from parallax_b200.engine.request import Request, SamplingParams
from parallax_b200.models.config import config_from_hf

pytestmark = pytest.mark.gpu


def _cfg():
    return config_from_hf(dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=512,
                               num_hidden_layers=4, num_attention_heads=8, num_key_value_heads=2, head_dim=128,
                               intermediate_size=1024, vocab_size=2048, tie_word_embeddings=False, rope_theta=1e4))


def _prompts(n, length, vocab, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (length,), generator=g).tolist() for _ in range(n)]


def _first_step_logits(device, dtype, prompts, weights=None, **kw):
    eng = Engine(_cfg(), device=device, dtype=dtype, num_blocks=128, page_size=16, max_batch_size=8,
                 weights=weights, **kw)
    eng.keep_logits = True
    for p in prompts:
        eng.add_request(Request(input_ids=p, sampling_params=SamplingParams(max_new_tokens=4, temperature=0.0,
                                                                            ignore_eos=True)))
    eng.step()
    first = eng.last_logits.float().cpu()
    eng.step()  # one decode step
    second = eng.last_logits.float().cpu()
    return eng, first, second


def _export_weights(eng):
    """HF-named fp32 weights of a random-init stage (undo the fused layouts)."""
    m = eng.stages[0].model
    cfg = m.cfg
    Hq, Hkv, D, I = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.intermediate_size
    w = {"model.embed_tokens.weight": m.embed, "model.norm.weight": m.norm_w, "lm_head.weight": m.lm_head}
    for lw in m.layers:
        p = f"model.layers.{lw.layer_idx}."
        q, k, v = lw.w_qkv.split([Hq * D, Hkv * D, Hkv * D], dim=0)
        gu = lw.w_gu.view(I // 64, 2, 64, -1)
        w.update({p + "input_layernorm.weight": lw.ln1, p + "post_attention_layernorm.weight": lw.ln2,
                  p + "self_attn.q_proj.weight": q, p + "self_attn.k_proj.weight": k,
                  p + "self_attn.v_proj.weight": v, p + "self_attn.o_proj.weight": lw.w_o,
                  p + "self_attn.q_norm.weight": lw.q_norm, p + "self_attn.k_norm.weight": lw.k_norm,
                  p + "mlp.gate_proj.weight": gu[:, 0].reshape(I, -1), p + "mlp.up_proj.weight": gu[:, 1].reshape(I, -1),
                  p + "mlp.down_proj.weight": lw.w_down})
    return {k: v.detach().float().cpu() for k, v in w.items()}


def test_gpu_engine_matches_cpu_engine():
    prompts = _prompts(5, 70, 2048) + _prompts(2, 5, 2048, seed=1)
    gpu, g1, g2 = _first_step_logits("cuda:0", torch.bfloat16, prompts)
    weights = _export_weights(gpu)
    # the CPU engine runs the bf16-rounded weights in fp32
    _cpu, c1, c2 = _first_step_logits("cpu", torch.float32, prompts, weights=weights)
    from parallax_b200.ops import cuda as cu
    cu.check_status(torch.device("cuda:0"))
    for g, c in ((g1, c1), (g2, c2)):
        assert g.shape == c.shape
        rel = (g - c).norm() / c.norm()
        assert rel < 3e-2, rel
        # margin-aware arg-max check: with N(0, 0.02) weights many rows are near-ties, so a row counts when
        # the fp32 gap between its two best tokens exceeds four times the largest logit error of that row;
        # every such row must agree
        top2 = c.topk(2, dim=-1).values
        clear = (top2[:, 0] - top2[:, 1]) > 4 * (g - c).abs().amax(dim=-1)
        assert clear.float().mean() >= 0.4, clear
        assert bool((g.argmax(-1) == c.argmax(-1))[clear].all())


def _generate_with_margins(eng, prompts, sp):
    """Tokens per prompt and, per generated token, the gap between the two best logits it was chosen from."""
    reqs = [Request(input_ids=list(p), sampling_params=SamplingParams.from_dict(sp.to_dict())) for p in prompts]
    for r in reqs:
        eng.add_request(r)
    eng.keep_logits = True
    gaps = {r.request_id: [] for r in reqs}
    noise = 0.0
    while eng.has_work():
        results = eng.step()
        lg = eng.last_logits.float()
        produced = [rq for rq, tok in results if tok is not None]
        assert len(produced) == lg.shape[0]
        top2 = lg.topk(2, dim=-1).values
        noise = max(noise, 0.04 * float(lg.std()))
        for rq, gap in zip(produced, (top2[:, 0] - top2[:, 1]).tolist()):
            gaps[rq.request_id].append(gap)
    return [r.output_ids for r in reqs], [gaps[r.request_id] for r in reqs], noise


def _agree_where_clear(a, b, gaps_b, noise):
    """(tokens compared, tokens equal): each sequence is compared up to its first step whose margin in run b
    is below the noise of a different summation order (after such a step the runs may legitimately part)."""
    compared = equal = 0
    for x, y, gp in zip(a, b, gaps_b):
        for i, (u, v) in enumerate(zip(x, y)):
            if gp[i] < noise:
                break
            compared += 1
            equal += int(u == v)
    return compared, equal


def test_gpu_sharded_chunked_prefix_consistency():
    prompts = _prompts(6, 150, 2048, seed=2)
    sp = SamplingParams(max_new_tokens=12, temperature=0.0, ignore_eos=True)
    kw = dict(device="cuda:0", num_blocks=256, max_batch_size=8, async_scheduling=False)
    base, base_gaps, noise = _generate_with_margins(
        Engine(_cfg(), chunked_prefill_size=None, enable_prefix_cache=False, **kw), prompts, sp)
    shard = Engine(_cfg(), chunked_prefill_size=None, enable_prefix_cache=False, stage_layers=[(0, 2), (2, 4)],
                   **kw).generate(prompts, sp)
    assert base == shard
    eng = Engine(_cfg(), chunked_prefill_size=64, **kw)
    a = eng.generate(prompts, sp)
    b = eng.generate(prompts, sp)  # served from the prefix cache
    assert eng.cache.prefix_cache.hits >= 6
    # chunking and cached prefixes change the reduction order: tokens chosen with a clear margin must not move
    for other in (a, b):
        compared, equal = _agree_where_clear(other, base, base_gaps, noise)
        assert compared >= 12 and equal == compared, (compared, equal)
    # and the asynchronous schedule produces exactly what the step-by-step schedule does
    assert Engine(_cfg(), device="cuda:0", num_blocks=256, max_batch_size=8, chunked_prefill_size=None,
                  enable_prefix_cache=False, async_scheduling=True).generate(prompts, sp) == base


def test_gpu_sampling_requests_finish():
    eng = Engine(_cfg(), device="cuda:0", num_blocks=128, max_batch_size=8)
    reqs = [Request(input_ids=p, sampling_params=SamplingParams(max_new_tokens=10, temperature=0.8, top_k=40,
                                                                top_p=0.9, ignore_eos=True), return_probs=True)
            for p in _prompts(4, 20, 2048, seed=5)]
    for r in reqs:
        eng.add_request(r)
    n = 0
    while eng.has_work() and n < 100:
        eng.step()
        n += 1
    assert all(len(r.output_ids) == 10 for r in reqs)
    assert all(0 <= t < 2048 for r in reqs for t in r.output_ids)
    assert all(0.0 < p <= 1.0 for r in reqs for p in r.output_probs)
    assert eng.cache.num_free_blocks() + eng.cache.prefix_cache.num_nodes == eng.cache.num_blocks


def test_native_stage_executor_equals_python_layer_loop():
    """One call into the library per stage must launch exactly the kernels of the Python loop."""
    prompts = _prompts(4, 90, 2048, seed=7) + _prompts(2, 7, 2048, seed=8)
    native, n1, n2 = _first_step_logits("cuda:0", torch.bfloat16, prompts)
    assert native.stages[0].model._native, "the dense GQA stage should use the native executor"
    weights = _export_weights(native)
    eng = Engine(_cfg(), device="cuda:0", dtype=torch.bfloat16, num_blocks=128, page_size=16, max_batch_size=8,
                 weights=weights)
    eng.stages[0].model._native = False          # force the per-layer Python loop
    eng.keep_logits = True
    for p in prompts:
        eng.add_request(Request(input_ids=p, sampling_params=SamplingParams(max_new_tokens=4, temperature=0.0,
                                                                            ignore_eos=True)))
    eng.step()
    p1 = eng.last_logits.float().cpu()
    eng.step()
    p2 = eng.last_logits.float().cpu()
    assert torch.equal(n1, p1) and torch.equal(n2, p2)


def test_long_context_chunked_prefill_32k():
    """A 32768-token prompt on a two-layer Qwen3-32B-shaped model: prefilled in 8192-token chunks (each chunk
    attends to the chunks before it through the block table) it must give the logits and tokens of the same
    prompt prefilled in one pass, and decode attention over the 32k context must continue from there."""
    from parallax_b200.models.config import named_config
    from parallax_b200.ops import cuda as cu

    cfg = named_config("qwen3-32b")
    cfg.num_hidden_layers = 2
    n_ctx = 32768
    g = torch.Generator().manual_seed(3)
    prompt = torch.randint(0, cfg.vocab_size, (n_ctx,), generator=g).tolist()
    sp = SamplingParams(max_new_tokens=6, temperature=0.0, ignore_eos=True)

    def run(chunk):
        eng = Engine(cfg, device="cuda:0", page_size=16, num_blocks=2200, max_batch_size=2,
                     max_num_tokens_per_batch=n_ctx + 64, chunked_prefill_size=chunk, enable_prefix_cache=False,
                     max_total_length=n_ctx + 64, async_scheduling=False, seed=1)
        eng.keep_logits = True
        r = Request(input_ids=prompt, sampling_params=SamplingParams.from_dict(sp.to_dict()), max_total_length=n_ctx + 64)
        eng.add_request(r)
        steps, first = 0, None
        while eng.has_work():
            res = eng.step()
            steps += 1
            if first is None and any(tok is not None for _rq, tok in res):
                first = eng.last_logits.float().cpu()
        cu.check_status(torch.device("cuda:0"))
        return r.output_ids, first, steps

    one, lg_one, steps_one = run(n_ctx)
    four, lg_four, steps_four = run(8192)
    assert steps_four == steps_one + 3                       # four prompt slices instead of one
    rel = float((lg_four - lg_one).norm() / lg_one.norm())
    assert rel < 3e-2, rel
    top2 = lg_one.topk(2, dim=-1).values
    if float(top2[0, 0] - top2[0, 1]) > 4 * float((lg_four - lg_one).abs().max()):
        assert four[0] == one[0]
    assert len(four) == len(one) == 6


def test_constrained_decoding_on_gpu():
    """JSON-schema requests on the GPU engine (lookahead on): valid documents that end by themselves, next to an
    unconstrained request whose tokens are what they are without the neighbours."""
    import json

    from parallax_b200.engine.structured import JsonSchemaMatcher
    from parallax_b200.frontend.tokenizer import TokenizerWrapper

    cfg = _cfg()
    tok = TokenizerWrapper(None, vocab_size=cfg.vocab_size)
    schema = {"type": "object", "properties": {"ok": {"type": "boolean"}, "n": {"type": "integer"}}, "required": ["ok", "n"]}
    kw = dict(device="cuda:0", dtype=torch.bfloat16, num_blocks=128, page_size=16, max_batch_size=8, seed=0)
    eng = Engine(cfg, tokenizer=tok, **kw)
    free_sp = SamplingParams(max_new_tokens=10, temperature=0.0, ignore_eos=True)
    p = _prompts(3, 24, 250, seed=2)
    reqs = [Request(input_ids=p[0], sampling_params=SamplingParams(max_new_tokens=150, temperature=0.0,
                                                                   json_schema=json.dumps(schema))),
            Request(input_ids=p[1], sampling_params=SamplingParams(max_new_tokens=150, temperature=0.8,
                                                                   json_schema=json.dumps(schema))),
            Request(input_ids=p[2], sampling_params=free_sp)]
    for r in reqs:
        eng.add_request(r)
    while eng.has_work():
        eng.step()
    for r in reqs[:2]:
        text = tok.decode(r.output_ids)
        m = JsonSchemaMatcher(schema)
        assert m.advance(text) and m.done, text
        assert set(json.loads(text)) >= {"ok", "n"} and r.status.name == "FINISHED_EOS" and len(r.output_ids) < 150
    assert len(reqs[2].output_ids) == 10
    from parallax_b200.ops import cuda as cu

    cu.check_status(torch.device("cuda:0"))
