"""Property test: adapters, JSON schemas, penalties, sampling and plain requests mixed in one engine, with staggered
arrivals, a client that goes away and the one-step lookahead on or off."""

import json
import tempfile
from pathlib import Path

import torch
from hypothesis import HealthCheck, given, settings
from hypothesis import strategies as st

from parallax_b200.engine.engine import Engine
from parallax_b200.engine.request import Request, SamplingParams
from parallax_b200.engine.structured import JsonSchemaMatcher
from parallax_b200.frontend.tokenizer import TokenizerWrapper
from parallax_b200.models.config import named_config
from tests.test_lora_cpu import _make_adapter

CFG = named_config("tiny")
TOK = TokenizerWrapper.from_pretrained(None, vocab_size=CFG.vocab_size)
SCHEMA = {"type": "object", "properties": {"ok": {"type": "boolean"}, "n": {"type": "integer"}}, "required": ["ok"]}
_DIR = Path(tempfile.mkdtemp(prefix="pxl_mix_"))
ADAPTERS = {"x": _make_adapter(CFG, _DIR / "x", 1), "y": _make_adapter(CFG, _DIR / "y", 2, rank=8, alpha=4)}

kinds = st.sampled_from(["plain", "lora_x", "lora_y", "schema", "schema_sampled", "penalty", "sampled"])
workload = st.fixed_dictionaries({
    "lookahead": st.booleans(), "batch": st.integers(1, 4), "chunk": st.sampled_from([None, 16]),
    "reqs": st.lists(st.tuples(kinds, st.integers(1, 40), st.integers(0, 6)), min_size=1, max_size=7),
    "abort_at": st.one_of(st.none(), st.integers(1, 15)),
})


@settings(max_examples=40, deadline=None, suppress_health_check=[HealthCheck.too_slow])
@given(workload)
def test_features_do_not_get_in_each_others_way(w):
    eng = Engine(CFG, device="cpu", num_blocks=96, page_size=16, max_batch_size=w["batch"], chunked_prefill_size=w["chunk"],
                 max_total_length=256, seed=0, async_scheduling=w["lookahead"], tokenizer=TOK,
                 lora={"max_loaded": 2, "max_rank": 8, "paths": ADAPTERS})
    g = torch.Generator().manual_seed(3)
    plan = []
    for kind, n, at in w["reqs"]:
        d = dict(max_new_tokens=60 if kind.startswith("schema") else 4, temperature=0.0, ignore_eos=not kind.startswith("schema"))
        if kind in ("schema_sampled", "sampled"):
            d.update(temperature=0.9, top_k=8)
        if kind == "penalty":
            d.update(repetition_penalty=1.2, frequency_penalty=0.3)
        if kind.startswith("schema"):
            d["json_schema"] = json.dumps(SCHEMA)
        ids = torch.randint(0, 250, (n,), generator=g).tolist()
        plan.append((at, kind, Request(input_ids=ids, sampling_params=SamplingParams.from_dict(d),
                                       lora_path={"lora_x": "x", "lora_y": "y"}.get(kind))))
    reqs = [(k, r) for _a, k, r in plan]
    step, aborted = 0, set()
    while plan or eng.has_work():
        for _a, _k, r in [p for p in plan if p[0] <= step]:
            eng.add_request(r)
        plan = [p for p in plan if p[0] > step]
        eng.step()
        step += 1
        if w["abort_at"] == step:
            live = [r for _k, r in reqs if not r.is_finished and r.output_ids]
            if live:
                aborted.add(live[0].request_id)
                eng.abort_request(live[0].request_id)
        assert step < 3000
    for kind, r in reqs:
        assert r.is_finished and all(t >= 0 for t in r.output_ids), (kind, r.status, r.output_ids)
        if r.request_id in aborted:
            continue
        if kind.startswith("schema"):
            if r.status.name == "FINISHED_EOS":
                text = TOK.decode(r.output_ids)
                m = JsonSchemaMatcher(SCHEMA)
                assert m.advance(text) and m.done and isinstance(json.loads(text)["ok"], bool), text
            else:
                assert r.status.name == "FINISHED_MAX_LENGTH" and len(r.output_ids) == 60
        else:
            assert len(r.output_ids) == 4, (kind, r.status, r.output_ids)
    assert not eng.cache.reqs and not any(eng.lora.pins.values()), eng.lora.pins
