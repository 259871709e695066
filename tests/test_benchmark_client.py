"""The serving benchmark client against a live node frontend (tiny CPU model, real HTTP + SSE)."""

import importlib.util
import os
import time

import pytest

from parallax_b200.engine.engine import Engine
from parallax_b200.engine.service import EngineLoop
from parallax_b200.frontend.openai_api import create_app
from parallax_b200.frontend.tokenizer import TokenizerWrapper
from parallax_b200.launch import serve_http
from parallax_b200.models.config import named_config
from parallax_b200.parallel.launcher import free_port

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _load_client():
    spec = importlib.util.spec_from_file_location("benchmark_serving", os.path.join(ROOT, "benchmarks", "benchmark_serving.py"))
    mod = importlib.util.module_from_spec(spec)
    import sys

    sys.modules["benchmark_serving"] = mod      # dataclasses look the module up by name
    spec.loader.exec_module(mod)
    return mod


@pytest.mark.parametrize("chat", [False, True])
def test_benchmark_client_end_to_end(chat):
    pytest.importorskip("aiohttp")
    cfg = named_config("tiny")
    eng = Engine(cfg, device="cpu", num_blocks=256, page_size=16, max_batch_size=8, max_total_length=512)
    loop = EngineLoop(eng)
    loop.start()
    tok = TokenizerWrapper.from_pretrained(None, vocab_size=cfg.vocab_size)
    app = create_app(loop, tok, "tiny", max_model_len=512)
    port = free_port()
    server, thread = serve_http(app, "127.0.0.1", port, "warning")
    try:
        for _ in range(100):
            if server.started:
                break
            time.sleep(0.05)
        client = _load_client()
        argv = ["--base-url", f"http://127.0.0.1:{port}", "--model", "tiny", "--num-prompts", "6",
                "--random-input-len", "24", "--random-output-len", "5", "--request-rate", "200", "--ignore-eos",
                "--goodput", "ttft:60000", "e2el:120000"] + (["--chat"] if chat else [])
        rep = client.main(argv)
        assert rep["completed"] == 6 and rep["failed"] == 0, rep
        assert rep["total_output_tokens"] >= 6 and rep["mean_ttft_ms"] > 0 and rep["output_throughput"] > 0
        assert rep["request_goodput"] > 0
    finally:
        server.should_exit = True
        thread.join(5)
        loop.stop()


def test_sharegpt_dataset_loader(tmp_path):
    import json

    client = _load_client()
    data = [
        {"conversations": [{"from": "human", "value": "tell me about paged attention in detail please"},
                           {"from": "gpt", "value": "it keeps the cache in fixed size blocks " * 3}]},
        {"conversations": [{"from": "human", "value": "hi"}, {"from": "gpt", "value": "hello"}]},          # too short
        {"conversations": [{"from": "human", "value": "only one turn here, no reply at all"}]},             # no reply
        {"conversations": [{"from": "human", "value": "how do pipeline stages hand activations over"},
                           {"from": "gpt", "value": "with point to point sends between neighbouring ranks"}]},
    ]
    path = tmp_path / "sharegpt.json"
    path.write_text(json.dumps(data))
    samples = client.load_sharegpt_dataset(str(path), 10, 64, seed=0)
    assert len(samples) == 2
    by_prompt = {s.prompt: s for s in samples}
    s = by_prompt["how do pipeline stages hand activations over"]
    assert s.prompt_len == 7 and s.max_tokens == 8
    assert len(client.load_sharegpt_dataset(str(path), 1, 64, seed=0)) == 1


def test_hf_and_wildchat_loaders(tmp_path):
    import json

    import pyarrow as pa
    import pyarrow.parquet as pq

    from benchmarks.benchmark_serving import load_hf_dataset, load_wildchat_dataset, make_random_dataset

    rows = [{"question": f"what is {i} plus {i}", "answer": "it is " + " ".join(["x"] * (i + 1))} for i in range(6)]
    pq.write_table(pa.Table.from_pylist(rows), tmp_path / "d.parquet")
    got = load_hf_dataset(str(tmp_path / "d.parquet"), 4, 32, seed=0)
    assert len(got) == 4 and all(s.prompt.startswith("what is") and s.max_tokens >= 3 for s in got)
    with open(tmp_path / "d.jsonl", "w") as f:
        for r in rows:
            f.write(json.dumps({"text": r["question"]}) + "\n")
    got = load_hf_dataset(str(tmp_path / "d.jsonl"), 10, 17, seed=1)
    assert len(got) == 6 and all(s.max_tokens == 17 for s in got)
    chats = [{"conversation": [{"role": "user", "content": f"hello {i}"}, {"role": "assistant", "content": "a b c d"}]}
             for i in range(3)] + [{"conversation": []}]
    with open(tmp_path / "w.json", "w") as f:
        json.dump(chats, f)
    got = load_wildchat_dataset(str(tmp_path / "w.json"), 5, 9, seed=0)
    assert len(got) == 3 and all(s.max_tokens == 4 for s in got)
    b = make_random_dataset(3, 50, 5, 0.0, seed=0, byte_level=True)
    assert all(len(s.prompt) == 50 == s.prompt_len for s in b)
