"""Cluster scheduling: cost model, water-filling / greedy / DP allocation, routing, lifecycle.

Multi-node behaviour is simulated in-process with synthetic nodes (hardware presets and RTTs),
the way the reference tests its scheduler (tests/scheduler_tests/*)."""

from collections import Counter

import pytest

from parallax_b200.scheduling.layer_allocation import DynamicProgrammingLayerAllocator, GreedyLayerAllocator
from parallax_b200.scheduling.model_info import ModelInfo
from parallax_b200.scheduling.node import Node, NodeHardwareInfo, RequestSignal
from parallax_b200.scheduling.node_management import NodeManager, NodeState, Pipeline
from parallax_b200.scheduling.request_routing import (DynamicProgrammingRouting,
                                                      RandomizedOverDynamicPipelinesRouting,
                                                      RoundRobinOverFixedPipelinesRouting, find_turning_points)
from parallax_b200.scheduling.scheduler import Scheduler

HW = {
    "a100-80g": (312.0, 80.0, 2039.0),
    "a100-40g": (312.0, 40.0, 1935.0),
    "rtx5090": (165.0, 32.0, 1792.0),
    "rtx4090": (82.6, 24.0, 1008.0),
    "b200": (2250.0, 180.0, 7700.0),
}


def model(num_layers):
    return ModelInfo(model_name=f"oss-{num_layers}", head_size=64, hidden_dim=2880, intermediate_dim=2880,
                     num_attention_heads=64, num_kv_heads=8, vocab_size=201088, num_layers=num_layers,
                     ffn_num_projections=3, num_local_experts=128, num_experts_per_tok=4,
                     param_bytes_per_element=1, cache_bytes_per_element=2, embedding_bytes_per_element=2)


class _AnyRtt(dict):
    """RTT table that answers 1 ms for every peer (a single NVSwitch box)."""

    def __bool__(self):
        return True

    def __contains__(self, key):
        return True

    def __getitem__(self, key):
        return 1.0


def node(kind, m, nid, **kw):
    tf, mem, bw = HW[kind]
    return Node(node_id=nid, hardware=NodeHardwareInfo(nid, 1, tf, "", mem, bw, "cuda"), model_info=m,
                rtt_to_nodes=_AnyRtt(), **kw)


def test_model_info_costs():
    m = model(36)
    assert m.per_token_per_layer_kv_size == 2 * (8 * 64 + 8 * 64)
    assert m.expected_num_activated_experts(batch_size=1, target_seq_len=1) == 4
    assert m.expected_num_activated_experts(batch_size=64, target_seq_len=1) > 100
    dense = ModelInfo(num_layers=2)
    assert dense.expected_num_activated_experts() is None
    assert m.decoder_layer_io_bytes(roofline=False) > m.decoder_layer_io_bytes(roofline=True, batch_size=1)
    assert m.lm_head_flops(3) == 2 * 3 * 2880 * 201088


def test_capacity_sanity():
    m = model(36)
    caps = {k: node(k, m, k).get_decoder_layer_capacity() for k in ("a100-80g", "a100-40g", "rtx5090", "rtx4090")}
    assert caps == {"a100-80g": 13, "a100-40g": 6, "rtx5090": 5, "rtx4090": 4}
    n = node("rtx4090", m, "x")
    assert n.get_decoder_layer_capacity(include_input_embed=True) == 3


@pytest.mark.parametrize("num_layers,kinds,expected", [
    (21, ["a100-80g", "rtx5090", "rtx4090"], [13, 5, 3]),
    (15, ["a100-80g", "rtx5090"], [11, 4]),
    (20, ["a100-80g", "rtx5090", "rtx4090"], [12, 5, 3]),
    (25, ["a100-80g", "rtx5090", "rtx4090", "rtx4090"], [13, 5, 4, 3]),
    (29, ["rtx4090", "a100-80g", "rtx5090", "rtx5090", "rtx4090"], [3, 13, 5, 5, 3]),
    (8, ["rtx5090", "rtx5090"], [4, 4]),
    (7, ["a100-40g", "rtx5090"], [5, 2]),
])
def test_water_filling(num_layers, kinds, expected):
    m = model(num_layers)
    nodes = [node(k, m, f"{k}-{i}") for i, k in enumerate(kinds)]
    alloc = GreedyLayerAllocator(model_info=m, node_management=NodeManager(initial_nodes=nodes))
    alloc.adjust_pipeline_layers(nodes, assume_sorted=False)
    got = [n.end_layer - n.start_layer for n in nodes]
    assert sum(got) == num_layers
    assert Counter(got) == Counter(expected)
    assert NodeManager(initial_nodes=[]).num_nodes == 0


@pytest.mark.parametrize("strategy", ["greedy", "dp"])
def test_allocators_build_full_pipelines(strategy):
    m = model(12)
    nodes = [node("a100-40g", m, f"n{i}") for i in range(6)]
    cls = GreedyLayerAllocator if strategy == "greedy" else DynamicProgrammingLayerAllocator
    nm = NodeManager(initial_nodes=nodes)
    alloc = cls(model_info=m, node_management=nm)
    assert alloc.allocate_from_standby()
    assert nm.num_full_pipelines(12) >= 2
    # every active node holds a valid range and pipelines tile [0, 12)
    pipes = RandomizedOverDynamicPipelinesRouting.pipeline_discovery(nm.active_nodes, 12)
    assert pipes
    for p in pipes:
        Pipeline.from_node_ids(p, nodes_by_id={n.node_id: n for n in nodes})


def test_dp_prefers_more_pipelines_with_fewer_stages():
    m = model(10)
    nodes = [node("a100-80g", m, "big0"), node("a100-80g", m, "big1")] + [node("rtx4090", m, f"s{i}") for i in range(3)]
    nm = NodeManager(initial_nodes=nodes)
    alloc = DynamicProgrammingLayerAllocator(model_info=m, node_management=nm)
    assert alloc.allocate_from_standby()
    # each 80 GB node can hold the whole 10-layer model: two single-stage pipelines
    assert nm.get("big0").num_current_layers == 10 and nm.get("big1").num_current_layers == 10


def test_b200_box_splits_evenly():
    m = ModelInfo(model_name="qwen3-8b", head_size=128, hidden_dim=4096, intermediate_dim=12288,
                  num_attention_heads=32, num_kv_heads=8, vocab_size=151936, num_layers=36,
                  param_bytes_per_element=2, cache_bytes_per_element=2, embedding_bytes_per_element=2)
    nodes = [node("b200", m, f"gpu{i}") for i in range(8)]
    alloc = GreedyLayerAllocator(model_info=m, node_management=NodeManager(initial_nodes=nodes))
    alloc.adjust_pipeline_layers(nodes)
    got = sorted(n.num_current_layers for n in nodes)
    assert sum(got) == 36 and got[-1] - got[0] <= 1


def _chain(m, spans, lat=None):
    nodes = []
    for i, (s, e) in enumerate(spans):
        n = node("a100-80g", m, f"n{i}", _force_max_concurrent_requests=True)
        n.rtt_to_nodes = {}
        n.set_layer_allocation(s, e)
        n.avg_layer_latency_ms = (lat or {}).get(i, 1.0)
        nodes.append(n)
    nm = NodeManager(initial_nodes=nodes)
    nm.activate([n.node_id for n in nodes])
    for a in nodes:
        for b in nodes:
            if a is not b:
                a.update_rtt(b.node_id, 5.0)
    return nodes, nm


def test_dp_routing_picks_cheapest_chain():
    m = model(8)
    nodes, nm = _chain(m, [(0, 4), (4, 8), (0, 8), (4, 8)], lat={0: 1.0, 1: 1.0, 2: 10.0, 3: 0.5})
    path, cost = DynamicProgrammingRouting(nm, 8).find_optimal_path()
    assert path == ["n0", "n3"]
    assert cost == pytest.approx(1.0 + 5.0 + 0.5, abs=0.1)
    nodes[3].current_requests = nodes[3].max_requests  # overloaded -> infinite latency
    path, _ = DynamicProgrammingRouting(nm, 8).find_optimal_path()
    assert path == ["n0", "n1"]


def test_pipeline_discovery_and_rr_routing():
    m = model(8)
    nodes, nm = _chain(m, [(0, 4), (4, 8), (0, 4), (4, 8)])
    pipes = RandomizedOverDynamicPipelinesRouting.pipeline_discovery(nodes, 8)
    assert len(pipes) == 4
    rr = RoundRobinOverFixedPipelinesRouting(nm, 8)
    reg = rr.bootstrap()
    assert len(reg) == 2
    flat = [x for p in reg.values() for x in p]
    assert len(flat) == len(set(flat)) == 4
    seen = [tuple(rr.find_optimal_path()[0]) for _ in range(4)]
    assert seen[0] != seen[1] and seen[0] == seen[2]
    # a pipeline with an inactive member is skipped
    nm.get(seen[0][0]).is_active = False
    assert all(tuple(rr.find_optimal_path()[0]) == seen[1] for _ in range(3))
    # stale weights after a refit are skipped as well
    nm.get(seen[0][0]).is_active = True
    for nid in seen[1]:
        nm.get(nid).last_refit_time = 10.0
    assert tuple(rr.find_optimal_path(last_refit_time=5.0)[0]) == seen[1]
    assert nm.num_full_pipelines(8) == 4


def test_turning_points():
    m = model(6)
    nodes, _ = _chain(m, [(0, 4), (2, 6)], lat={0: 1.0, 1: 0.1})
    tp = find_turning_points(nodes, 6)
    assert ("n0", 2, "tail") in tp or any(k == "tail" for _, _, k in tp)


def test_scheduler_join_leave_rebalance():
    m = model(12)
    sched = Scheduler(m, [], min_nodes_bootstrapping=2, strategy="greedy", routing_strategy="rr",
                      heartbeat_timeout=0.05)
    for i in range(2):
        sched.enqueue_join(node("a100-40g", m, f"n{i}"))
    sched._process_joins()
    assert sched.bootstrapped and sched.has_full_pipeline()
    sched.receive_request(RequestSignal("r1"))
    rid, path, lat = sched.dispatch_next_request()
    assert rid == "r1" and len(path) == 2 and lat < float("inf")
    assert all(sched.get_node(n).current_requests == 1 for n in path)
    # a third and fourth node join later and form a second pipeline
    for i in range(2, 4):
        sched.enqueue_join(node("a100-40g", m, f"n{i}"))
    sched._process_joins()
    assert len(sched.node_manager.get_registered_pipelines()) == 2
    # heartbeat update path
    sched.enqueue_node_update("n0", current_requests=3, layer_latency_ms=2.5, is_active=True)
    sched._process_node_updates()
    assert sched.get_node("n0").current_requests == 3 and sched.get_node("n0").avg_layer_latency_ms == 2.5
    # node leaves: its pipeline is dissolved, the other one keeps serving
    sched.enqueue_leave(path[0])
    sched._process_leaves()
    assert sched.get_node(path[0]) is None
    assert sched.has_full_pipeline()
    assert sched.node_manager.state_of(path[1]) == NodeState.STANDBY
    # losing a member of the last pipeline triggers a global re-allocation over what is left
    remaining = [n for p in sched.node_manager.get_registered_pipelines().values() for n in p.node_ids]
    sched.enqueue_leave(remaining[0])
    sched._process_leaves()
    assert sched.has_full_pipeline()
    assert sched.node_manager.num_nodes == 2


def test_heartbeat_eviction():
    import time

    m = model(6)
    sched = Scheduler(m, [], min_nodes_bootstrapping=1, strategy="dp", routing_strategy="dp", heartbeat_timeout=0.01)
    sched.enqueue_join(node("a100-80g", m, "solo"))
    sched._process_joins()
    assert sched.bootstrapped
    time.sleep(0.03)
    sched.checking_node_heartbeat()
    sched._process_leaves()
    assert sched.get_node("solo") is None and not sched.has_full_pipeline()


@pytest.mark.parametrize("routing", ["dp", "rr"])
def test_manual_assignment_bootstraps(routing):
    m = model(6)
    sched = Scheduler(m, [], strategy="greedy", routing_strategy=routing)
    a = node("a100-80g", m, "a", manual_layer_assignment=True, start_layer=0, end_layer=3)
    b = node("a100-80g", m, "b", manual_layer_assignment=True, start_layer=3, end_layer=6)
    sched.enqueue_join(a)
    sched.enqueue_join(b)
    sched._process_joins()
    assert sched.bootstrapped
    sched.receive_request(RequestSignal("x"))
    _, path, _ = sched.dispatch_next_request()
    assert path == ["a", "b"]
