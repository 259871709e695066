"""DistEngine (pipeline x tensor parallel) on CPU ranks over gloo: the sharded, pipelined
engine must generate exactly what the single-process engine generates."""

import json
import os
import subprocess
import sys

import pytest
import torch

from parallax_b200.engine.engine import Engine
from parallax_b200.engine.request import SamplingParams
from parallax_b200.models.config import named_config
from parallax_b200.parallel.dist_engine import split_layers
from parallax_b200.parallel.launcher import free_port
from parallax_b200.parallel.tp_comm import padded_rows_per_rank

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HELPER = os.path.join(os.path.dirname(__file__), "helpers", "dist_engine_rank.py")
PROMPTS = [[5, 9, 77, 3, 250, 12, 8], [100, 101, 102], list(range(20, 75)), [7] * 19, [1, 2, 3, 4, 5, 6, 7, 8, 9]]


def _run_group(pp, tp, tmp_path, max_new=6, chunk=16, model="tiny", prompts=None, **extra):
    spec = dict(model_name=model, pp=pp, tp=tp, device_type="cpu", num_blocks=256, page_size=16, max_batch_size=4,
                max_num_tokens_per_batch=64, chunked_prefill_size=chunk, max_total_length=256,
                prompts=prompts or PROMPTS,
                max_new=max_new, seed=0)
    spec.update(extra)
    world, port = pp * tp * extra.get("ep", 1), free_port()
    out = tmp_path / f"out_{pp}_{tp}.json"
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                   OMP_NUM_THREADS="2", PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
        procs.append(subprocess.Popen([sys.executable, HELPER, json.dumps(spec), str(out)], env=env))
    codes = []
    for p in procs:
        try:
            codes.append(p.wait(timeout=240))
        except subprocess.TimeoutExpired:
            p.kill()
            codes.append(-9)
    assert codes == [0] * world, codes
    return json.loads(out.read_text())


def _single(max_new=6, chunk=16, model="tiny", prompts=None):
    torch.manual_seed(0)
    eng = Engine(named_config(model), device="cpu", num_blocks=256, page_size=16, max_batch_size=4,
                 max_num_tokens_per_batch=64, chunked_prefill_size=chunk, max_total_length=256, seed=0)
    return eng.generate(prompts or PROMPTS, SamplingParams(max_new_tokens=max_new, temperature=0.0, ignore_eos=True))


def test_split_layers_and_padding():
    assert split_layers(28, 4) == [(0, 7), (7, 14), (14, 21), (21, 28)]
    assert split_layers(10, 3) == [(0, 3), (3, 7), (7, 10)]      # the remainder goes to a middle stage
    assert [b - a for a, b in split_layers(36, 8)] == [4, 5, 5, 5, 5, 4, 4, 4]
    assert padded_rows_per_rank(1, 2, 128) == 128
    assert padded_rows_per_rank(300, 2, 128) == 256
    assert padded_rows_per_rank(7, 2, 1) == 4


@pytest.mark.parametrize("pp,tp", [(1, 2), (2, 1), (2, 2)])
def test_dist_engine_matches_single_process(pp, tp, tmp_path):
    want = _single()
    got = _run_group(pp, tp, tmp_path)
    assert got["outputs"] == want
    assert got["probe"]["device_ms"] > 0 and got["probe"]["h2d_bytes"] > 0


def test_rank0_executor_thread_and_aligned_rows(tmp_path):
    """Rank 0 launching its stage from a thread of its own, three micro-batches in flight and prompt
    slices trimmed to a row multiple: same tokens as the single-process engine."""
    want = _single()
    got = _run_group(2, 1, tmp_path, executor_thread=True, micro_batch_ratio=2, max_in_flight=3,
                     max_prefill_tokens_per_batch=24, align_rows=8)
    assert got["outputs"] == want


def test_dist_engine_moe_expert_parallel(tmp_path):
    """Attention tensor-parallel, experts expert-parallel over the same two ranks."""
    want = _single(model="tiny-moe")
    got = _run_group(1, 2, tmp_path, model="tiny-moe")
    assert got["outputs"] == want


@pytest.mark.parametrize("pp,ep", [(1, 2), (2, 2)])
def test_expert_parallel_with_data_parallel_attention(pp, ep, tmp_path):
    """Every lane keeps the whole attention stack and half of the experts and serves its own requests
    (five prompts over two lanes: the lanes run different row counts, and a lane goes idle while the
    other still decodes). Same tokens as the single-process engine."""
    want = _single(model="tiny-moe", max_new=7)
    got = _run_group(pp, 1, tmp_path, model="tiny-moe", ep=ep, max_new=7)
    assert got["outputs"] == want


def test_deepseek_stage_under_expert_parallelism(tmp_path):
    """MLA attention data-parallel, routed experts sharded over two lanes (sigmoid routing with groups, shared
    expert replicated): same tokens as the single-process engine."""
    want = _single(model="tiny-mla", max_new=5)
    got = _run_group(1, 1, tmp_path, model="tiny-mla", ep=2, max_new=5)
    assert got["outputs"] == want


@pytest.mark.parametrize("model,pp", [("tiny-mla", 1), ("tiny-dsa", 1), ("tiny-hybrid", 1), ("tiny-msa", 1),
                                      ("tiny-hybrid", 2)])
def test_tensor_parallel_stages_of_the_other_families(model, pp, tmp_path):
    """Heads split over two ranks for latent attention (dense and indexer-sparse), gated delta-net / gated
    attention and block-sparse attention; sequence-sharded residual stream; experts (where the model has
    them) split over the same two ranks. Same tokens as the single-process engine."""
    # one prompt long enough that block selection (more than 2 blocks of 32 tokens) and top-k key selection
    # (more than 16 keys) really select
    prompts = PROMPTS + [[(7 * i + 3) % 1000 for i in range(100)]]
    want = _single(model=model, max_new=5, prompts=prompts)
    got = _run_group(pp, 2, tmp_path, model=model, max_new=5, prompts=prompts)
    assert got["outputs"] == want


@pytest.mark.parametrize("pp,tp", [(2, 1), (1, 2)])
def test_hybrid_prefix_cache_across_ranks(pp, tp, tmp_path):
    """Gated delta-net layers under pipeline / tensor parallelism with the prefix cache on: rank 0 decides
    which recurrent-state snapshots are taken and restored, every rank carries the copies out around its
    forward in plan order. Six prompts share a 64-token prefix, four run at a time: the later ones resume
    from the snapshots the earlier ones left. Same tokens as the single-process engine."""
    base = [(13 * i + 5) % 1000 for i in range(64)]
    prompts = [base + [100 + j, 200 + j, 300 + j][: 1 + j % 3] for j in range(6)]
    want = _single(model="tiny-hybrid", max_new=5, prompts=prompts)
    got = _run_group(pp, tp, tmp_path, model="tiny-hybrid", max_new=5, prompts=prompts)
    assert got["outputs"] == want
    assert got["prefix_hits"] >= 2 and got["state_snapshots"] >= 1, got


@pytest.mark.parametrize("pp,tp", [(2, 1), (1, 2)])
def test_constrained_decoding_on_the_sampling_rank(pp, tp, tmp_path):
    """JSON-schema requests in a multi-rank engine: the rank that samples keeps the matcher, rank 0 ends the
    request when the document is complete; the result equals the single-process engine's, and the
    unconstrained request of the same batch is untouched."""
    from parallax_b200.engine.request import Request
    from parallax_b200.engine.structured import JsonSchemaMatcher
    from parallax_b200.frontend.tokenizer import TokenizerWrapper

    schema = {"type": "object", "properties": {"ok": {"type": "boolean"}, "n": {"type": "integer"}},
              "required": ["ok", "n"]}
    schema_of = [schema, None, schema]
    prompts = PROMPTS[:3]
    got = _run_group(pp, tp, tmp_path, prompts=prompts, schema_of=schema_of)["outputs"]
    cfg = named_config("tiny")
    tok = TokenizerWrapper.from_pretrained(None, vocab_size=cfg.vocab_size)
    torch.manual_seed(0)
    eng = Engine(cfg, device="cpu", num_blocks=256, page_size=16, max_batch_size=4, max_num_tokens_per_batch=64,
                 chunked_prefill_size=16, max_total_length=256, seed=0, tokenizer=tok)
    reqs = []
    for p, sch in zip(prompts, schema_of):
        d = dict(max_new_tokens=6 if sch is None else 120, temperature=0.0, ignore_eos=sch is None)
        if sch is not None:
            d["json_schema"] = json.dumps(sch)
        reqs.append(Request(input_ids=list(p), sampling_params=SamplingParams.from_dict(d)))
        eng.add_request(reqs[-1])
    while eng.has_work():
        eng.step()
    for r, ids, sch in zip(reqs, got, schema_of):
        if sch is not None:
            text = tok.decode(ids)
            m = JsonSchemaMatcher(sch)
            assert m.advance(text) and m.done, text
            assert set(json.loads(text)) >= {"ok", "n"}
        if tp == 1:
            assert ids == r.output_ids      # same summation order as the single process
    assert len(got[1]) == 6


@pytest.mark.parametrize("model,pp,tp,ep,seed", [("tiny", 2, 1, 1, 1), ("tiny", 1, 2, 1, 2), ("tiny-moe", 1, 1, 2, 3),
                                                 ("tiny", 3, 1, 1, 4)])
def test_random_mix_drains_and_returns_all_memory(model, pp, tp, ep, seed, tmp_path):
    """A random mix of requests (staggered arrivals, shared prefixes, sampling, penalties, client aborts) on a
    small KV pool: every request ends - with all its tokens, or aborted - and rank 0's bookkeeping is empty
    afterwards, with every block either free or held by the prefix tree."""
    extra = dict(ep=ep) if ep > 1 else {}
    r = _run_group(pp, tp, tmp_path, model=model, stress_seed=seed, num_blocks=40, **extra)["stress"]
    for status, want, got, aborted in zip(r["status"], r["want"], _lens(r, tmp_path, pp, tp), r["aborted"]):
        assert status.startswith("FINISHED"), r
        assert got == want or status == "FINISHED_ABORT", (status, want, got, aborted)
    assert r["live_requests"] == 0 and all(r["probs_ok"]), r
    for free, tree in zip(r["free_blocks"], r["tree_blocks"]):
        assert free + tree == r["num_blocks"], r


@pytest.mark.parametrize("pp,tp", [(2, 1), (1, 2)])
def test_random_mix_with_adapters_and_schemas(pp, tp, tmp_path):
    """The same random mix with per-request LoRA adapters and JSON-schema requests among the others: adapter pins and
    the matchers' bookkeeping are back to zero at the end, and finished schema requests hold valid documents."""
    from parallax_b200.engine.structured import JsonSchemaMatcher
    from parallax_b200.frontend.tokenizer import TokenizerWrapper
    from tests.test_lora_cpu import _make_adapter

    cfg = named_config("tiny")
    lora = {"max_loaded": 2, "max_rank": 8,
            "paths": {"x": _make_adapter(cfg, tmp_path / "x", 1), "y": _make_adapter(cfg, tmp_path / "y", 2, rank=8, alpha=4)}}
    schema = {"type": "object", "properties": {"ok": {"type": "boolean"}}, "required": ["ok"]}
    out = _run_group(pp, tp, tmp_path, stress_seed=11, num_blocks=64, lora=lora, stress_features=["lora", "schema"],
                     stress_schema=schema, stress_requests=16)
    r = out["stress"]
    tok = TokenizerWrapper.from_pretrained(None, vocab_size=cfg.vocab_size)
    assert any(r["schema"])
    for status, want, ids, is_schema in zip(r["status"], r["want"], out["outputs"], r["schema"]):
        assert status.startswith("FINISHED"), r
        if is_schema and status == "FINISHED_EOS":
            text = tok.decode(ids)
            m = JsonSchemaMatcher(schema)
            assert m.advance(text) and m.done, text
        elif not is_schema:
            assert len(ids) == want or status == "FINISHED_ABORT", (status, want, ids)
    assert r["live_requests"] == 0 and r["lora_pins"] == 0 and r["grammars_known"] == 0 and all(r["probs_ok"]), r


def test_random_mix_on_a_hybrid_model_with_state_snapshots(tmp_path):
    out = _run_group(2, 1, tmp_path, model="tiny-hybrid", stress_seed=5, num_blocks=48)
    r = out["stress"]
    for status, want, ids in zip(r["status"], r["want"], out["outputs"]):
        assert status.startswith("FINISHED") and (len(ids) == want or status == "FINISHED_ABORT"), (status, want, ids)
    assert r["live_requests"] == 0


def _lens(r, tmp_path, pp, tp):
    return [len(o) for o in json.loads((tmp_path / f"out_{pp}_{tp}.json").read_text())["outputs"]]


def test_rank_loss_is_detected_on_the_host(tmp_path):
    """Failure detection without touching a device: the second pipeline rank exits between steps;
    the scheduling rank sees its heartbeat stop and raises within seconds."""
    spec = dict(model_name="tiny", pp=2, tp=1, device_type="cpu", num_blocks=256, page_size=16, max_batch_size=4,
                max_num_tokens_per_batch=64, chunked_prefill_size=16, max_total_length=256, seed=0,
                prompts=[[5, 9, 77, 3], [100, 101, 102]], plans_before_exit=6)
    helper = os.path.join(os.path.dirname(__file__), "helpers", "dist_engine_fail_rank.py")
    port = free_port()
    out = tmp_path / "fail.json"
    procs = []
    for r in range(2):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                   OMP_NUM_THREADS="2", PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
        procs.append(subprocess.Popen([sys.executable, helper, json.dumps(spec), str(out)], env=env))
    for p in procs:
        try:
            p.wait(timeout=120)
        except subprocess.TimeoutExpired:
            p.kill()
            raise AssertionError("the scheduling rank kept waiting for a rank that had left")
    res = json.loads(out.read_text())
    assert res["error"] is not None and "stopped responding" in res["error"], res
    assert res["steps"] >= 3 and res["seconds"] < 60, res
