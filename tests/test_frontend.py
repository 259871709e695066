"""OpenAI-compatible frontend against a tiny CPU engine (FastAPI TestClient)."""

import json

import pytest

from parallax_b200.engine.engine import Engine
from parallax_b200.engine.service import EngineLoop
from parallax_b200.frontend.openai_api import create_app, sampling_params_from_body
from parallax_b200.frontend.tokenizer import ByteTokenizer, IncrementalDetokenizer, TokenizerWrapper
from parallax_b200.models.config import named_config


@pytest.fixture(scope="module")
def client():
    from fastapi.testclient import TestClient

    cfg = named_config("tiny")
    eng = Engine(cfg, device="cpu", num_blocks=128, page_size=16, max_batch_size=4)
    loop = EngineLoop(eng)
    loop.start()
    tok = TokenizerWrapper(ByteTokenizer(), vocab_size=cfg.vocab_size)
    app = create_app(loop, tok, "tiny-test", max_model_len=512)
    with TestClient(app) as c:
        yield c
    loop.stop()


def test_models_and_health(client):
    assert client.get("/v1/models").json()["data"][0]["id"] == "tiny-test"
    assert client.get("/health").json()["status"] == "ok"


def test_chat_completion_non_stream(client):
    r = client.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi there"}],
                                                   "max_tokens": 6, "temperature": 0, "ignore_eos": True})
    assert r.status_code == 200
    body = r.json()
    assert body["object"] == "chat.completion" and body["choices"][0]["finish_reason"] == "length"
    assert body["usage"]["completion_tokens"] == 6 and body["usage"]["prompt_tokens"] > 8
    assert isinstance(body["choices"][0]["message"]["content"], str)


def test_completion_stream_sse(client):
    with client.stream("POST", "/v1/completions", json={"prompt": "abc", "max_tokens": 5, "temperature": 0,
                                                         "stream": True, "ignore_eos": True}) as r:
        assert r.status_code == 200
        lines = [l for l in r.iter_lines() if l.startswith("data: ")]
    assert lines[-1] == "data: [DONE]"
    chunks = [json.loads(l[6:]) for l in lines[:-1]]
    assert chunks[-1]["choices"][0]["finish_reason"] == "length"
    assert chunks[-1]["usage"]["completion_tokens"] == 5


def test_bad_requests(client):
    assert client.post("/v1/chat/completions", json={"messages": []}).status_code == 400
    r = client.post("/v1/completions", json={"prompt": "x", "top_p": 0})
    assert r.status_code == 400 and r.json()["error"]["type"] == "invalid_request_error"
    r = client.post("/v1/completions", json={"prompt": "x" * 600})
    assert r.status_code == 400


def test_token_id_prompt_and_probs(client):
    r = client.post("/v1/completions", json={"prompt": [1, 2, 3, 4], "max_tokens": 3, "temperature": 0.8,
                                             "top_k": 5, "return_probs": True, "ignore_eos": True})
    body = r.json()
    assert len(body["choices"][0]["token_probs"]) == 3


def test_sampling_params_mapping():
    sp = sampling_params_from_body({"max_completion_tokens": 9, "temperature": 0, "stop": "END", "top_k": 0})
    assert sp.max_new_tokens == 9 and sp.top_k == 1 and sp.stop_strs == ["END"]


def test_incremental_detokenizer_utf8_and_stop():
    t = TokenizerWrapper(ByteTokenizer())
    d = IncrementalDetokenizer(t, stop=["STOP"])
    text = "héllo wörld STOP never shown"
    out = "".join(d.add(b) for b in text.encode("utf-8")) + d.flush()
    assert out == "héllo wörld " and d.stopped
    d2 = IncrementalDetokenizer(t)
    out2 = "".join(d2.add(b) for b in "日本語".encode("utf-8")) + d2.flush()
    assert out2 == "日本語"


def test_response_format_json_schema_over_http(client):
    schema = {"type": "object", "properties": {"answer": {"type": "boolean"}, "n": {"type": "integer"}},
              "required": ["answer", "n"]}
    r = client.post("/v1/chat/completions", json={
        "messages": [{"role": "user", "content": "reply in json"}], "max_tokens": 120, "temperature": 0,
        "response_format": {"type": "json_schema", "json_schema": {"name": "reply", "schema": schema}}})
    assert r.status_code == 200, r.text
    body = r.json()
    doc = json.loads(body["choices"][0]["message"]["content"])
    assert isinstance(doc["answer"], bool) and isinstance(doc["n"], int) and set(doc) == {"answer", "n"}
    assert body["choices"][0]["finish_reason"] == "stop"
