"""Property test of the engine loop on CPU: whatever the mix of prompt lengths, budgets, slice sizes and shared
prefixes, every step respects its limits, every request ends with the tokens it asked for, and all KV memory comes back."""

import torch
from hypothesis import HealthCheck, given, settings
from hypothesis import strategies as st

from parallax_b200.engine.engine import Engine
from parallax_b200.engine.request import Request, SamplingParams
from parallax_b200.models.config import config_from_hf, named_config

CFG = config_from_hf(dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=64, num_hidden_layers=1,
                          num_attention_heads=2, num_key_value_heads=1, head_dim=32, intermediate_size=128, vocab_size=128,
                          tie_word_embeddings=True, rope_theta=1e4))

MODELS = {"dense": CFG, "hybrid": named_config("tiny-hybrid"), "mla": named_config("tiny-mla"),
          "dsa": named_config("tiny-dsa"), "msa": named_config("tiny-msa"), "moe": named_config("tiny-moe")}

workload = st.fixed_dictionaries({
    "model": st.sampled_from(sorted(MODELS)),
    "batch": st.integers(1, 6), "ratio": st.integers(1, 2), "budget": st.integers(24, 96),
    "chunk": st.sampled_from([None, 16, 32]), "lookahead": st.booleans(), "prefix_cache": st.booleans(),
    "blocks": st.sampled_from([6, 10, 24, 96]),
    "reqs": st.lists(st.tuples(st.integers(1, 70), st.integers(1, 6), st.booleans()), min_size=1, max_size=9),
    "sampled": st.lists(st.sampled_from(["greedy", "sample", "penalty"]), min_size=9, max_size=9),
    "abort_at": st.one_of(st.none(), st.integers(1, 12)),
})


@settings(max_examples=150, deadline=None, suppress_health_check=[HealthCheck.too_slow])
@given(workload)
def test_limits_hold_and_everything_finishes(w):
    cfg = MODELS[w["model"]]
    V = cfg.vocab_size
    eng = Engine(cfg, device="cpu", num_blocks=w["blocks"], page_size=16, max_batch_size=w["batch"], micro_batch_ratio=w["ratio"],
                 max_num_tokens_per_batch=w["budget"], chunked_prefill_size=w["chunk"], enable_prefix_cache=w["prefix_cache"],
                 max_total_length=128, seed=0, async_scheduling=w["lookahead"])
    g = torch.Generator().manual_seed(1)
    shared = torch.randint(0, V, (48,), generator=g).tolist()
    reqs = []
    for n, max_new, share in w["reqs"]:
        ids = (shared[:min(n, 48)] if share else []) + torch.randint(0, V, (max(n - 48, 1) if share else n,), generator=g).tolist()
        kind = w["sampled"][len(reqs)]
        sp = SamplingParams(max_new_tokens=max_new, temperature=0.8 if kind == "sample" else 0.0, ignore_eos=True,
                            top_k=5 if kind == "sample" else -1, repetition_penalty=1.3 if kind == "penalty" else 1.0)
        reqs.append(Request(input_ids=ids, sampling_params=sp))
    pending = list(reqs)
    micro = max(w["batch"] // w["ratio"], 1)
    steps = 0
    aborted = set()
    while pending or eng.has_work():
        if pending:
            eng.add_request(pending.pop(0))         # arrivals interleave with steps
        eng.step()
        steps += 1
        if w["abort_at"] == steps:               # a client goes away
            live = [r for r in reqs if not r.is_finished and r not in pending]
            if live:
                eng.abort_request(live[0].request_id)
                aborted.add(live[0].request_id)
        s = eng.last_step_stats
        if s:
            assert s["tokens"] <= w["budget"] + micro, s           # prompt tokens within the budget, plus the decode rows
            assert s["decode"] <= micro and s["new_tokens"] <= micro, s
            if w["chunk"]:
                assert s["prefill_tokens"] <= max(w["budget"], w["chunk"]), s
        assert steps < 2000, "the loop does not terminate"
    for r in reqs:
        # a request ends with all its tokens, or aborted when the KV memory ran out (small pools)
        assert r.is_finished, (r.status, len(r.input_ids))
        assert len(r.output_ids) == r.sampling_params.max_new_tokens or \
            (r.status.name == "FINISHED_ABORT" and (w["blocks"] < 96 or r.request_id in aborted)) or \
            (r.status.name == "CANCELLED" and r.request_id in aborted and not r.output_ids), (r.status, r.output_ids)
        assert all(0 <= t < V for t in r.output_ids)
    assert not eng.cache.reqs
    held = 0
    if eng.cache.prefix_cache is not None:
        stack = list(eng.cache.prefix_cache.root.children.values())
        while stack:
            n = stack.pop()
            held += 1
            stack.extend(n.children.values())
    assert eng.cache.num_free_blocks() == w["blocks"] - held
    if eng.cache.needs_slots:
        # recurrent-state slots: the requests' own are all back, snapshots are held by tree nodes only
        assert eng.cache.slot_allocator.get_num_free_slots() == eng.cache.slot_allocator.num_slots
        snaps = 0
        stack = list(eng.cache.prefix_cache.root.children.values()) if eng.cache.prefix_cache is not None else []
        while stack:
            n = stack.pop()
            snaps += int(n.linear_slot is not None)
            stack.extend(n.children.values())
        if eng.cache.prefix_slot_allocator is not None:
            assert eng.cache.prefix_slot_allocator.get_num_free_slots() == eng.cache.prefix_slot_allocator.num_slots - snaps
