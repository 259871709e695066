"""Router: strategies, runtime config, health-aware selection, streaming proxy metrics."""

import json
import types

import httpx
import pytest
from fastapi.testclient import TestClient

from parallax_b200.router.app import SSEMeter, create_app, filter_forward_headers
from parallax_b200.router.lb_strategy import PerformanceConfig, PerformanceStrategy, RoundRobinStrategy, make_strategy
from parallax_b200.router.registry import EndpointMetrics, EndpointRegistry, RouterConfig


def _cand(url, **m):
    return types.SimpleNamespace(base_url=url, metrics=EndpointMetrics(**m))


def test_round_robin_prefers_least_normalised_load_then_rotates():
    rr = RoundRobinStrategy()
    a, b, c = _cand("http://a"), _cand("http://b"), _cand("http://c")
    assert [rr.select([c, a, b]).base_url for _ in range(4)] == ["http://a", "http://b", "http://c", "http://a"]
    a.metrics.inflight, a.metrics.max_running_request = 4, 8       # 0.5
    b.metrics.inflight, b.metrics.max_running_request = 1, 8       # 0.125
    c.metrics.inflight, c.metrics.max_running_request = 3, 4       # 0.75
    assert rr.select([a, b, c]).base_url == "http://b"


def test_performance_score_terms():
    s = PerformanceStrategy(PerformanceConfig())
    cold = _cand("http://a")
    assert s.score(cold) == pytest.approx(3000 + 50)
    busy = _cand("http://b", inflight=2, ema_ttft_ms=100.0, ema_tpot_ms=10.0, total_requests=10, total_errors=1)
    assert s.score(busy) == pytest.approx(2 * 1000 + 100 + 10 + 0.1 * 5000)
    assert s.select([cold, busy]) is busy
    with pytest.raises(ValueError):
        make_strategy("nope", performance_cfg=PerformanceConfig())


def test_sse_meter_and_header_filter():
    m = SSEMeter()
    m.feed(b'data: {"a":1}\n\nda')
    m.feed(b'ta: {"a":2}\r\n\ndata: [DONE]\n\n: comment\n')
    s = m.summary()
    assert s["output_units"] == 2 and s["ttft_ms"] is not None and sum(s["output_buckets"].values()) == 2
    h = filter_forward_headers({"Authorization": "x", "Cookie": "y", "content-type": "application/json"})
    assert "Cookie" not in h and h["Accept"] == "application/json"


class _Upstream:
    """Fake cluster answering status probes and chat completions."""

    def __init__(self):
        self.status = {"http://c1": "available", "http://c2": "available", "http://c3": "waiting"}
        self.calls = []

    def handler(self, request: httpx.Request) -> httpx.Response:
        base = f"{request.url.scheme}://{request.url.host}"
        if request.url.path == "/cluster/status_json":
            return httpx.Response(200, json={"data": {"status": self.status.get(base), "max_running_request": 8}})
        if request.url.path == "/v1/chat/completions":
            self.calls.append(base)
            body = json.loads(request.content)
            if body.get("stream"):
                sse = b'data: {"choices":[{"delta":{"content":"a"}}]}\n\ndata: {"choices":[{"delta":{"content":"b"}}]}\n\ndata: [DONE]\n\n'
                return httpx.Response(200, content=sse, headers={"content-type": "text/event-stream"})
            return httpx.Response(200, json={"id": "x", "served_by": base})
        if request.url.path == "/weight/refit":
            return httpx.Response(200, json={"ok": True})
        return httpx.Response(404)


@pytest.fixture()
def router():
    up = _Upstream()
    reg = EndpointRegistry(config=RouterConfig(status_check_ttl_sec=0.0),
                           http_client_factory=lambda: httpx.AsyncClient(transport=httpx.MockTransport(up.handler)))
    with TestClient(create_app(reg)) as c:
        yield c, up


def test_register_route_and_metrics(router):
    c, up = router
    assert c.post("/v1/chat/completions", json={"messages": []}).status_code == 503
    assert c.post("/register", json={"endpoint": "http://c1"}).status_code == 200
    assert c.post("/register", json={"endpoint": "http://c2/"}).status_code == 200
    assert c.post("/register", json={"endpoint": "ftp://bad"}).status_code == 400
    assert c.post("/register", json={"endpoint": "http://c3"}).status_code == 200   # registered but not available
    seen = {c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "x"}]}).json()["served_by"]
            for _ in range(4)}
    assert seen == {"http://c1", "http://c2"}                      # the waiting cluster is never chosen
    with c.stream("POST", "/v1/chat/completions", json={"stream": True, "messages": []}) as r:
        data = b"".join(r.iter_bytes())
    assert data.count(b"data:") == 3
    eps = {e["base_url"]: e for e in c.get("/endpoints").json()["endpoints"]}
    assert sum(e["metrics"]["total_requests"] for e in eps.values()) == 5
    assert all(e["metrics"]["inflight"] == 0 for e in eps.values())
    streamed = [e for e in eps.values() if e["metrics"]["ema_tpot_ms"] is not None]
    assert len(streamed) == 1 and streamed[0]["metrics"]["request_samples"][-1]["output_units"] == 2
    assert eps["http://c3"]["metrics"]["last_status_ok"] is False
    # disable c1: everything goes to c2
    assert c.post("/endpoint/enabled", json={"base_url": "http://c1", "enabled": False}).json()["enabled"] is False
    up.calls.clear()
    for _ in range(3):
        c.post("/v1/chat/completions", json={"messages": []})
    assert set(up.calls) == {"http://c2"}
    assert c.post("/endpoint/enabled", json={"base_url": "http://nope", "enabled": True}).status_code == 404
    r = c.post("/weight/refit", json={"time_stamp": 1, "cid": [], "index_map": {}})
    assert r.status_code == 200 and r.json()["broadcast_count"] == 3
    assert c.post("/unregister", json={"endpoint": "http://c1"}).json()["removed"] == 1
    assert "endpoints" in c.get("/").text.lower()


def test_runtime_balancer_config(router):
    c, _ = router
    assert c.get("/balancer/config").json()["config"]["strategy"] == "round_robin"
    assert c.post("/balancer/config", json={"config": {"top_k": 2}}).status_code == 400   # needs performance strategy
    r = c.post("/balancer/config", json={"strategy": "performance", "top_k": 2, "status_check_ttl_sec": 1})
    assert r.status_code == 200 and r.json()["config"]["top_k"] == 2 and r.json()["prob"]["status_check_ttl_sec"] == 1.0
    for bad in ({"strategy": "x"}, {"ema_alpha": 0}, {"top_k": 1.5}, {"explore_ratio": 1.0}, {"prob": {"zzz": 1}},
                {"status_check_timeout_sec": 0}, {"top_k": True}):
        assert c.post("/balancer/config", json=bad).status_code == 400, bad
    c.post("/register", json={"endpoint": "http://c1"})
    assert "score" in c.get("/endpoints").json()["endpoints"][0]
    assert c.get("/health").json()["status"] == "ok"
