"""Cluster backend: node join/heartbeat/leave over HTTP, status, routing + forwarding, refit."""

import json

import httpx
import pytest
from fastapi.testclient import TestClient

from parallax_b200.backend.app import create_app
from parallax_b200.backend.request_handler import RequestHandler
from parallax_b200.backend.scheduler_manage import SchedulerManage
from parallax_b200.scheduling.model_info import ModelInfo

MODEL = ModelInfo(model_name="test/model", head_size=64, hidden_dim=512, intermediate_dim=1024,
                  num_attention_heads=8, num_kv_heads=2, vocab_size=1000, num_layers=8,
                  param_bytes_per_element=2, cache_bytes_per_element=2, embedding_bytes_per_element=2)


def _node_msg(nid, port):
    return {"node_id": nid, "http_addr": f"http://node-{nid}:{port}", "wait_seconds": 5,
            "hardware": {"node_id": nid, "num_gpus": 1, "tflops_fp16": 2250.0, "gpu_name": "NVIDIA B200",
                         "memory_gb": 180.0, "memory_bandwidth_gbps": 7700.0, "device": "cuda"},
            "kvcache_mem_ratio": 0.25, "param_mem_ratio": 0.65, "max_concurrent_requests": 4,
            "max_sequence_length": 2048, "rtt_to_nodes": {"a": 0.1, "b": 0.1}}


class _Nodes:
    def __init__(self):
        self.seen = []

    def handler(self, request: httpx.Request) -> httpx.Response:
        body = json.loads(request.content)
        self.seen.append((request.url.host, body))
        if body.get("stream"):
            sse = (b'data: {"choices":[{"delta":{"content":"hi"}}]}\n\n'
                   b'data: {"choices":[],"usage":{"prompt_tokens":3,"completion_tokens":2,"total_tokens":5}}\n\n'
                   b'data: [DONE]\n\n')
            return httpx.Response(200, content=sse, headers={"content-type": "text/event-stream"})
        return httpx.Response(200, json={"id": body["request_id"], "choices": [{"message": {"content": "ok"}}]})


@pytest.fixture()
def backend():
    nodes = _Nodes()
    sm = SchedulerManage(http_port=3001, scheduler_kwargs={"strategy": "greedy"})
    rh = RequestHandler(http_client_factory=lambda: httpx.AsyncClient(transport=httpx.MockTransport(nodes.handler)))
    rh.RETRY_DELAY_SEC = rh.FORWARD_DELAY_SEC = 0.01
    rh.MAX_ROUTING_RETRY = 2
    with TestClient(create_app(sm, rh)) as c:
        yield c, sm, nodes
    sm.stop()


def test_cluster_lifecycle_and_forwarding(backend):
    c, sm, nodes = backend
    assert c.post("/v1/chat/completions", json={"messages": []}).status_code == 503
    assert c.post("/node/join", json=_node_msg("a", 3000)).status_code == 503          # scheduler not started
    assert c.post("/scheduler/init", json={"model_name": "x"}).status_code == 400
    sm.run("test/model", 1, True, model_info=MODEL)
    st = c.get("/cluster/status_json").json()["data"]
    assert st["status"] == "waiting" and st["need_more_nodes"] and st["node_join_command"]["command"] == "parallax join"
    alloc = c.post("/node/join", json=_node_msg("a", 3000)).json()
    assert alloc["start_layer"] == 0 and alloc["end_layer"] == 8 and alloc["model_name"] == "test/model"
    st = c.get("/cluster/status_json").json()["data"]
    assert st["status"] == "available" and st["max_running_request"] >= 4 and len(st["node_list"]) == 1
    assert c.get("/v1/models").json()["data"][0]["id"] == "test/model"
    # heartbeat
    hb = dict(_node_msg("a", 3000), current_requests=1, layer_latency_ms=0.7)
    r = c.post("/node/update", json=hb).json()
    assert r["layer_allocation"]["end_layer"] == 8 and r["refit_request"] == {}
    # forwarding: routing table and scheduler request id are injected
    r = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "x"}]})
    assert r.status_code == 200 and r.json()["choices"][0]["message"]["content"] == "ok"
    host, sent = nodes.seen[-1]
    assert host == "node-a" and sent["vllm_xargs"]["parallax_routing_table"] == ["a"] and sent["model"] == "test/model"
    with c.stream("POST", "/v1/chat/completions", json={"messages": [], "stream": True}) as s:
        assert b"[DONE]" in b"".join(s.iter_bytes())
    assert sm.scheduler.get_node("a").current_requests <= 1                      # slots are handed back
    # refit is delivered exactly once per node through the heartbeat
    assert c.post("/weight/refit", json={"time_stamp": 42, "cid": ["c"], "index_map": {}}).status_code == 200
    assert c.post("/node/update", json=hb).json()["refit_request"]["time_stamp"] == 42
    assert c.post("/node/update", json=hb).json()["refit_request"] == {}
    assert "latest_timestamp" in c.get("/weight/refit/timestamp").json()
    # leave: the cluster goes back to waiting
    c.post("/node/leave", json={"node_id": "a"})
    import time
    for _ in range(100):
        if c.get("/cluster/status_json").json()["data"]["status"] == "waiting":
            break
        time.sleep(0.02)
    assert c.get("/cluster/status_json").json()["data"]["status"] == "waiting"
    assert c.get("/model/list").json()["type"] == "model_list"
    assert "cluster" in c.get("/").text.lower()


def test_all_pipelines_busy_is_429(backend):
    c, sm, _ = backend
    sm.run("test/model", 1, True, model_info=MODEL)
    c.post("/node/join", json=_node_msg("a", 3000))
    node = sm.scheduler.get_node("a")
    node.current_requests = node.max_requests
    r = c.post("/v1/chat/completions", json={"messages": []})
    assert r.status_code in (429, 503)
    assert r.json()["error"]["code"] in ("rate_limit_exceeded", "routing_not_ready")


def test_web_app_pages_and_the_calls_they_make(backend):
    """The cluster web app is one static file with three views; every endpoint it calls answers in the shape
    the page reads (set up -> /model/list + /scheduler/init, join -> /node/join/command + /cluster/status,
    chat -> /v1/models + /v1/chat/completions)."""
    import re

    c, sm, _ = backend
    page = c.get("/").text
    for view in ("#/setup", "#/join", "#/chat"):
        assert view in page
    called = set(re.findall(r"['\"`](/(?:model|scheduler|node|cluster|v1)/[a-z_/]+)['\"`]", page))
    assert {"/model/list", "/scheduler/init", "/node/join/command", "/cluster/status", "/cluster/status_json",
            "/v1/models", "/v1/chat/completions"} <= called
    models = c.get("/model/list").json()["data"]
    assert models and {"name", "vram_gb"} <= set(models[0])
    # before set-up: no model, the page starts on the set-up view
    d = c.get("/cluster/status_json").json()["data"]
    assert d["model_name"] is None and d["node_list"] == []
    assert c.post("/scheduler/init", json={"init_nodes_num": 2}).status_code == 400
    sm.run("test/model", 2, True, model_info=MODEL)
    cmd = c.get("/node/join/command").json()["data"]
    assert "command" in cmd and "parallax" in cmd["command"]
    c.post("/node/join", json=_node_msg("a", 3000))
    d = c.get("/cluster/status_json").json()["data"]       # the stream sends this same object once a second
    assert {"status", "model_name", "init_nodes_num", "node_list", "need_more_nodes", "max_running_request"} <= set(d)
    assert d["init_nodes_num"] == 2 and [n["node_id"] for n in d["node_list"]] == ["a"]
    assert {"node_id", "status", "gpu_num", "gpu_name", "gpu_memory", "start_layer", "end_layer"} <= set(d["node_list"][0])
    assert "chat" in c.get("/chat").text
