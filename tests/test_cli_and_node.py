"""CLI argv construction, server args, node agent (join / heartbeat / allocation change), peer loops."""

import time

import pytest
from fastapi.testclient import TestClient

from parallax_b200 import cli
from parallax_b200.args import parse_args
from parallax_b200.engine.peer import PeerExecutor
from parallax_b200.frontend.tokenizer import ByteTokenizer, TokenizerWrapper
from parallax_b200.launch_chat import create_chat_app
from parallax_b200.models.config import named_config
from parallax_b200.p2p.message_util import proto_to_request, request_to_proto
from parallax_b200.p2p.node_runtime import PeerLoop, create_peer_app
from parallax_b200.p2p.server import NodeAgent
from parallax_b200.utils.hardware import HardwareInfo, match_gpu_specs
from parallax_b200.utils.shared_state import SharedState


def _capture(monkeypatch):
    seen = {}
    monkeypatch.setattr(cli, "_execute_with_graceful_shutdown", lambda cmd, env=None: seen.update(cmd=cmd, env=env))
    return seen


def test_cli_commands_build_expected_argv(monkeypatch):
    seen = _capture(monkeypatch)
    cli.main(["serve", "-m", "Qwen/Qwen3-0.6B", "--port", "4000", "--max-batch-size", "32"])
    assert seen["cmd"][1:4] == ["-m", "parallax_b200.launch", "--model-path"] and "--max-batch-size" in seen["cmd"]
    cli.main(["run", "-m", "Qwen/Qwen3-8B", "-n", "2"])
    assert "parallax_b200.backend.app" in seen["cmd"] and seen["cmd"][-4:] == ["--model-name", "Qwen/Qwen3-8B", "--init-nodes-num", "2"]
    assert seen["cmd"][seen["cmd"].index("--port") + 1] == "3001"
    cli.main(["run", "--port", "3005"])
    assert seen["cmd"].count("--port") == 1 and "3005" in seen["cmd"]
    cli.main(["join", "-s", "10.0.0.5:3001", "--tp-size", "4"])
    assert seen["cmd"][3:5] == ["--scheduler-addr", "10.0.0.5:3001"] and seen["cmd"][-2:] == ["--tp-size", "4"]
    cli.main(["join"])
    assert seen["cmd"][4] == "127.0.0.1:3001"
    cli.main(["chat", "-s", "h:1"])
    assert "parallax_b200.launch_chat" in seen["cmd"]
    with pytest.raises(SystemExit):
        cli.main([])


def test_server_args_defaults_and_validation():
    a = parse_args(["--model-path", "x"])
    assert (a.port, a.max_batch_size, a.max_num_tokens_per_batch, a.chunked_prefill_size) == (3000, 8, 16384, 1024)
    assert a.enable_prefix_cache and a.micro_batch_ratio == 1 and a.request_timeout_s == 600 and a.dtype == "bfloat16"
    assert parse_args(["--disable-prefix-cache"]).enable_prefix_cache is False
    assert parse_args(["--chunked-prefill-size", "0"]).chunked_prefill_size is None
    assert parse_args(["--chunked-prefill-size", "1000", "--kv-block-size", "16"]).chunked_prefill_size == 992
    for bad in (["--start-layer", "-1"], ["--start-layer", "4", "--end-layer", "4"], ["--kv-cache-memory-fraction", "1.5"],
                ["--max-batch-size", "0"], ["--kv-block-size", "0"], ["--micro-batch-ratio", "0"],
                ["--enable-weight-refit", "--weight-refit-mode", "tape"], ["--pp-size", "0"]):
        with pytest.raises(ValueError):
            parse_args(bad)


def test_hardware_table_has_blackwell():
    assert match_gpu_specs("NVIDIA B200", 180)[0] >= 2000
    assert match_gpu_specs("NVIDIA A100-SXM4-80GB", 80) == (312.0, 2039.0)
    assert match_gpu_specs("Mystery GPU", 8) == (50.0, 600.0)
    assert HardwareInfo.detect().memory_gb > 0


class _FakeScheduler:
    def __init__(self):
        self.alloc = {"node_id": "n", "model_name": "m", "start_layer": 0, "end_layer": 4, "tp_size": 1,
                      "enable_weight_refit": True, "weight_refit_mode": "disk"}
        self.refit = {}
        self.updates, self.left = [], []

    def node_join(self, info):
        self.joined = info
        return dict(self.alloc)

    def node_update(self, info):
        self.updates.append(info)
        refit, self.refit = self.refit, {}
        return dict(self.alloc), refit

    def node_leave(self, node_id):
        self.left.append(node_id)
        return {}


def test_node_agent_join_heartbeat_reallocation_and_refit():
    sched, state, refits = _FakeScheduler(), SharedState.create(in_process=True), []
    hw = HardwareInfo(1, "NVIDIA B200", 2250.0, 180.0, 7700.0)
    agent = NodeAgent(sched, state, "http://127.0.0.1:3000", node_id="n", hardware=hw, on_refit=refits.append,
                      heartbeat_interval_s=0.02)
    agent.join()
    info = state.get_model_info()
    assert (info["block_start_index"], info["block_end_index"], info["model_name"]) == (0, 4, "m")
    assert not state.get_layer_allocation_changed() and sched.joined["hardware"]["gpu_name"] == "NVIDIA B200"
    state.set_status("available")
    state.update_metrics(current_requests=3, layer_latency_ms_sample=1.5)
    state.update_metrics(layer_latency_ms_sample=2.5)
    alloc, _ = agent.heartbeat_once()
    sent = sched.updates[-1]
    assert sent["current_requests"] == 3 and sent["is_active"] and sent["layer_latency_ms"] == pytest.approx(1.7)
    sched.alloc.update(start_layer=2, end_layer=4)               # scheduler rebalanced the cluster
    sched.refit = {"time_stamp": 99.0, "cid": [], "index_map": {}}
    agent.start()
    for _ in range(100):
        if state.get_layer_allocation_changed():
            break
        time.sleep(0.01)
    agent.stop()
    assert state.get_layer_allocation_changed() and state.get_status() == "initializing"
    assert state["block_start_index"] == 2 and refits and agent.last_refit_time == 99.0 and sched.left == ["n"]


class _DirectTransport:
    """Delivers packets to other in-process peer loops through the wire encoding."""

    def __init__(self):
        self.loops = {}

    def send_forward(self, packets, self_id):
        by_next = {}
        for pk in packets:
            t = pk.routing_table
            by_next.setdefault(t[(t.index(self_id) + 1) % len(t)], []).append(pk)
        for nid, group in by_next.items():
            self.loops[nid].on_packets(proto_to_request(request_to_proto(group)))

    def send_abort(self, request_ids, routing_table, self_id):
        for nid in routing_table:
            if nid != self_id:
                self.loops[nid].on_abort(request_ids)


def test_peer_loops_serve_openai_requests_across_two_peers():
    cfg = named_config("tiny")
    tr = _DirectTransport()
    peers = [PeerExecutor(cfg, 0, 2, device="cpu", node_id="a", num_blocks=64),
             PeerExecutor(cfg, 2, 4, device="cpu", node_id="b", num_blocks=64)]
    loops = [PeerLoop(p, tr) for p in peers]
    tr.loops = {"a": loops[0], "b": loops[1]}
    for l in loops:
        l.start()
    try:
        app = create_peer_app(loops[0], TokenizerWrapper(ByteTokenizer(), cfg.vocab_size), "tiny", 512)
        with TestClient(app) as c:
            body = {"prompt": "hello world", "max_tokens": 5, "temperature": 0, "ignore_eos": True,
                    "vllm_xargs": {"parallax_routing_table": ["a", "b"]}}
            r = c.post("/v1/completions", json=body)
            assert r.status_code == 200 and r.json()["usage"]["completion_tokens"] == 5
        with TestClient(create_peer_app(loops[1])) as c2:
            assert c2.get("/health").json()["status"] == "ok"
            assert c2.post("/pp_abort", content=__import__("msgpack").packb({"abort": ["zzz"]})).json()["ok"]
        for _ in range(100):
            if not peers[1].mirror:
                break
            time.sleep(0.01)
        assert not peers[1].mirror and not peers[0].cache.reqs
    finally:
        for l in loops:
            l.stop()


def test_chat_app_forwards_to_backend():
    import httpx

    def handler(request: httpx.Request) -> httpx.Response:
        if request.url.path == "/v1/chat/completions":
            return httpx.Response(200, json={"choices": [{"message": {"content": "pong"}}]})
        return httpx.Response(200, json={"data": {"status": "available"}})

    app = create_chat_app("sched:3001", lambda: httpx.AsyncClient(transport=httpx.MockTransport(handler)))
    with TestClient(app) as c:
        assert c.post("/v1/chat/completions", json={"messages": []}).json()["choices"][0]["message"]["content"] == "pong"
        assert c.get("/cluster/status_json").json()["data"]["status"] == "available"
        assert "parallax chat" in c.get("/").text


def test_node_agent_measures_the_hops_to_its_peers():
    """The scheduler prices a pipeline by the round trips between its nodes, so every node probes the others it
    learns of from the scheduler and sends what it measured with its heartbeats; a peer that does not answer yet
    stays unknown, is tried again, and makes the agent beat faster until then."""

    class Sched:
        def __init__(self):
            self.updates = []

        def node_addresses(self):
            return {"me": "http://me", "b": "http://b", "c": "http://c"}

        def node_update(self, info):
            self.updates.append(info)
            return {}, {}

    up = {"http://b": 1.5}
    sched = Sched()
    agent = NodeAgent(sched, SharedState.create(in_process=True), "http://me", node_id="me",
                      hardware=HardwareInfo(1, "NVIDIA B200", 2250.0, 180.0, 7700.0, "cuda"),
                      probe=lambda url: up.get(url))
    agent.heartbeat_once()
    assert sched.updates[-1]["rtt_to_nodes"] == {"b": 1.5} and agent._rtt_missing
    up["http://c"] = 0.7
    agent.heartbeat_once()
    assert sched.updates[-1]["rtt_to_nodes"] == {"b": 1.5, "c": 0.7} and not agent._rtt_missing
