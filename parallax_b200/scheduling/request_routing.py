"""Request routing: pick the chain of nodes a request travels through.

Three strategies, as in ``src/scheduling/request_routing.py`` of the reference:

* ``DynamicProgrammingRouting`` - shortest path over node shards; node cost is its effective
  per-layer latency, edge cost the RTT between consecutive nodes;
* ``RandomizedOverDynamicPipelinesRouting`` - enumerate every complete chain once (DFS over
  layer boundaries) and pick a random viable one per request;
* ``RoundRobinOverFixedPipelinesRouting`` - register node-disjoint pipelines at bootstrap
  (one per head node, cheapest first) and dispatch round robin, skipping pipelines that are
  not ready, overloaded, or still serving stale weights after a refit.
"""

from __future__ import annotations

import logging
import random
from abc import ABC, abstractmethod
from typing import Optional

from parallax_b200.scheduling.layer_allocation import (BaseLayerAllocator, layer_level_best_path,
                                                       turning_points_of_path)
from parallax_b200.scheduling.node import Node
from parallax_b200.scheduling.node_management import NodeManager

logger = logging.getLogger(__name__)
INF = float("inf")


def estimate_pipeline_latency(pipeline_node_ids: list[str], *, id_to_node: dict[str, Node]) -> float:
    """Sum of node latencies plus RTT hops; inf if any member is missing or overloaded."""
    total, prev = 0.0, None
    for nid in pipeline_node_ids:
        n = id_to_node.get(nid)
        if n is None or n.is_overloaded:
            return INF
        lat = float(n.layer_latency_ms)
        if lat == INF:
            return INF
        total += lat
        if prev is not None and prev.node_id != n.node_id:
            hop = float(prev.get_rtt_to(n))
            if hop == INF:
                return INF
            total += hop
        prev = n
    return total


def find_turning_points(nodes: list[Node], num_layers: int) -> list[tuple[str, int, str]]:
    """Layers at which the latency-optimal layer-level path switches nodes while the previous
    node still hosts the layer ('tail'), or enters a node after its first layer ('head')."""
    if num_layers <= 0 or not nodes:
        return []
    path = layer_level_best_path(nodes, num_layers)
    return turning_points_of_path(nodes, path) if path else []


def _fmt_lat(x: float) -> str:
    return "inf" if x == INF else f"{x:.2f}"


class RequestRoutingStrategy(ABC):
    def __init__(self, node_manager: NodeManager, total_layers: int = 0):
        self.node_manager = node_manager
        self.total_layers = total_layers

    @abstractmethod
    def find_optimal_path(self, last_refit_time: Optional[float] = None) -> tuple[list[str], float]:
        """(node ids in stage order, estimated latency ms); ([], inf) when nothing is viable."""

    def bootstrap(self):
        return None

    def routing_ready(self) -> bool:
        return True

    def expand_pipelines(self) -> None:
        return None

    def _standby_lines(self) -> list[str]:
        standby = sorted(self.node_manager.standby_nodes, key=lambda n: n.node_id)
        head = f"Standby nodes ({len(standby)})"
        lines = ["", head, "-" * len(head)]
        if not standby:
            lines.append("  (none)")
        for n in standby:
            lines.append("  %-16s load %3d/%-3d | latency %7s ms | active %s"
                         % (n.node_id, n.current_requests, n.max_requests, _fmt_lat(n.layer_latency_ms), n.is_active))
        return lines

    def scheduler_format_snapshot(self) -> str:
        alloc = self.node_manager.list_node_allocations(self.total_layers)
        head = f"Current allocations ({len(alloc)} nodes)"
        lines = [head, "-" * len(head)]
        for nid, s, e in alloc:
            node = self.node_manager.get(nid)
            if node is None:
                raise ValueError(f"Node {nid} not found in node manager")
            hosted = int(self.node_manager.node_assigned_request_count.get(nid, 0))
            lines.append("  %-16s layers [%3d, %3d) | load %3d/%-3d | latency %7s ms | assigned %d | active %s"
                         % (nid, s, e, node.current_requests, node.max_requests,
                            _fmt_lat(node.layer_latency_ms), hosted, node.is_active))
        if len(lines) == 2:
            lines.append("  (none)")
        return "\n".join(lines + self._standby_lines())


class DynamicProgrammingRouting(RequestRoutingStrategy):
    def find_optimal_path(self, last_refit_time: Optional[float] = None) -> tuple[list[str], float]:
        nodes = [n for n in self.node_manager.active_nodes
                 if n.start_layer is not None and n.end_layer is not None and n.is_active is not False]
        L = self.total_layers
        if L <= 0 or not self.node_manager.active_nodes:
            return [], 0.0
        nodes.sort(key=lambda n: (n.start_layer, n.end_layer))
        ends: dict[int, list[int]] = {}
        for i, n in enumerate(nodes):
            ends.setdefault(n.end_layer, []).append(i)
        cost = [INF] * len(nodes)
        parent: list[Optional[int]] = [None] * len(nodes)
        for i, n in enumerate(nodes):
            lat = float(n.layer_latency_ms)
            if n.start_layer == 0:
                cost[i] = lat
                continue
            for j in ends.get(n.start_layer, []):
                if cost[j] == INF:
                    continue
                hop = 0.0 if nodes[j].node_id == n.node_id else float(nodes[j].get_rtt_to(n))
                c = cost[j] + hop + lat
                if c < cost[i]:
                    cost[i], parent[i] = c, j
        terminals = ends.get(L, [])
        if not terminals:
            return [], INF
        end = min(terminals, key=lambda k: cost[k])
        if cost[end] == INF:
            return [], INF
        path, cur = [], end
        while cur is not None:
            path.append(nodes[cur].node_id)
            cur = parent[cur]
        path.reverse()
        return path, cost[end]

    def routing_ready(self) -> bool:
        ids, lat = self.find_optimal_path()
        return bool(ids) and lat != INF


class RandomizedOverDynamicPipelinesRouting(RequestRoutingStrategy):
    def __init__(self, node_manager: NodeManager, total_layers: int = 0):
        super().__init__(node_manager, total_layers)
        self._pipelines: Optional[list[list[str]]] = None
        self._rng = random.Random()

    @staticmethod
    def pipeline_discovery(nodes: list[Node], num_layers: int) -> list[list[str]]:
        """Every chain of nodes whose ranges tile [0, num_layers), depth first, shorter next
        shards first."""
        if not nodes or num_layers <= 0:
            return []
        by_start: dict[int, list[Node]] = {}
        for n in nodes:
            if n.start_layer is not None and n.end_layer is not None:
                by_start.setdefault(n.start_layer, []).append(n)
        found: list[list[str]] = []
        stack: list[tuple[int, list[str]]] = []
        for head in reversed(by_start.get(0, [])):
            stack.append((int(head.end_layer), [head.node_id]))
        while stack:
            end, path = stack.pop()
            if end == num_layers:
                found.append(path)
                continue
            nxt = sorted((n for n in by_start.get(end, []) if n.end_layer > end), key=lambda n: n.end_layer)
            for n in reversed(nxt):
                stack.append((int(n.end_layer), path + [n.node_id]))
        return found

    def find_optimal_path(self, nodes: Optional[list[Node]] = None, num_layers: Optional[int] = None,
                          last_refit_time: Optional[float] = None) -> tuple[list[str], float]:
        nodes = self.node_manager.active_nodes if nodes is None else nodes
        L = self.total_layers if num_layers is None else num_layers
        if not nodes or L <= 0:
            return [], INF
        if self._pipelines is None:
            self._pipelines = self.pipeline_discovery(nodes, L)
        if not self._pipelines:
            return [], INF
        by_id = {n.node_id: n for n in nodes}
        viable = [(p, lat) for p in self._pipelines
                  if (lat := estimate_pipeline_latency(p, id_to_node=by_id)) != INF]
        if not viable:
            return [], INF
        p, lat = self._rng.choice(viable)
        return list(p), float(lat)

    def expand_pipelines(self) -> None:
        raise NotImplementedError("randomized routing discovers pipelines lazily; nothing to expand")


class RoundRobinOverFixedPipelinesRouting(RequestRoutingStrategy):
    def __init__(self, node_manager: NodeManager, total_layers: int,
                 layer_allocator: Optional[BaseLayerAllocator] = None):
        super().__init__(node_manager, total_layers)
        self._rr_cursor = 0
        self.layer_allocator = layer_allocator

    def _select_best_pipelines(self, all_pipelines: list[list[str]], nodes: list[Node]) -> list[list[str]]:
        """One pipeline per head node, cheapest heads first, no node used twice."""
        by_id = {n.node_id: n for n in nodes}
        by_head: dict[str, list[tuple[list[str], float]]] = {}
        for p in all_pipelines:
            if not p or len(set(p)) != len(p):
                continue
            c = estimate_pipeline_latency(p, id_to_node=by_id)
            if c != INF:
                by_head.setdefault(p[0], []).append((p, c))
        used: set[str] = set()
        chosen: list[list[str]] = []
        for head in sorted(by_head, key=lambda h: min(c for _, c in by_head[h])):
            free = [(c, i, p) for i, (p, c) in enumerate(by_head[head]) if not used.intersection(p)]
            if free:
                _, _, p = min(free)
                chosen.append(p)
                used.update(p)
        return chosen

    def bootstrap(self) -> dict[int, list[str]]:
        if self.node_manager.get_registered_pipeline_node_ids():
            self.node_manager.clear_registered_pipelines()
            self._rr_cursor = 0
        nodes = self.node_manager.active_nodes
        if not nodes or self.total_layers <= 0:
            return {}
        every = RandomizedOverDynamicPipelinesRouting.pipeline_discovery(nodes, self.total_layers)
        if not every:
            return {}
        return self.node_manager.register_pipelines(self._select_best_pipelines(every, nodes))

    def clear_registered_pipelines(self) -> None:
        self.node_manager.clear_registered_pipelines()

    def get_registered_pipelines(self) -> dict[int, list[str]]:
        return self.node_manager.get_registered_pipeline_node_ids()

    def routing_ready(self) -> bool:
        return any(p.is_ready for p in self.node_manager.get_registered_pipelines().values())

    def expand_pipelines(self) -> None:
        """Build additional full pipelines out of STANDBY nodes and register them."""
        if self.layer_allocator is None:
            raise NotImplementedError("expand_pipelines requires a layer allocator")
        if not self.node_manager.standby_nodes:
            return
        before = {n.node_id for n in self.node_manager.active_nodes}
        if not self.layer_allocator.allocate_from_standby():
            return
        fresh = [n for n in self.node_manager.active_nodes if n.node_id not in before]
        if not fresh:
            return
        new = RandomizedOverDynamicPipelinesRouting.pipeline_discovery(fresh, self.total_layers)
        new = [p for p in new if all(self.node_manager.pipeline_id_of_node(nid) is None for nid in p)]
        picked, used = [], set()
        for p in new:  # keep them node-disjoint among themselves
            if not used.intersection(p):
                picked.append(p)
                used.update(p)
        if picked:
            try:
                self.node_manager.extend_registered_pipelines(picked)
            except Exception as exc:  # registration is best effort; serving continues
                logger.warning("could not register new pipelines: %s", exc)

    def find_optimal_path(self, nodes=None, num_layers=None,
                          last_refit_time: Optional[float] = None) -> tuple[list[str], float]:
        pipes = self.node_manager.get_registered_pipelines()
        if not pipes:
            self.bootstrap()
            pipes = self.node_manager.get_registered_pipelines()
        by_id = {n.node_id: n for n in self.node_manager.nodes}
        ordered = [pipes[k] for k in sorted(pipes)]
        for _ in range(len(ordered)):
            cand = ordered[self._rr_cursor % len(ordered)]
            self._rr_cursor += 1
            if not cand.is_ready:
                continue
            ids = list(cand.node_ids)
            lat = estimate_pipeline_latency(ids, id_to_node=by_id)
            for nid in ids:
                n = by_id.get(nid)
                if n is None:
                    raise ValueError(f"node {nid} of pipeline {ids} not found in node manager")
                if not n.is_active:
                    lat = INF
                if last_refit_time is not None and n.last_refit_time < last_refit_time:
                    lat = INF  # still serving older weights
            if lat != INF:
                return ids, float(lat)
        return [], INF

    def scheduler_format_snapshot(self) -> str:
        pipes = self.node_manager.get_registered_pipelines()
        head = f"Registered pipelines ({len(pipes)})"
        lines = [head, "-" * len(head)]
        per, total, cur = self.node_manager.report_pipeline_capacity(ready_only=True)
        if per is None:
            lines.append("Capacity: (no registered pipelines)")
        else:
            lines.append(f"Capacity: total={total} current capacity={cur} per_pipeline={per}")
        if not pipes:
            lines.append("  (none)")
        for pid in sorted(pipes):
            p = pipes[pid]
            p.recompute_capacity()
            lines.append("  pipeline %-3d | stages=%d | ready=%s | cap=%d cur=%d"
                         % (pid, p.num_stages, p.is_ready, p.min_node_capacity, p.min_remaining_capacity))
            for i, n in enumerate(p.nodes):
                lines.append("    [%02d] %-16s layers [%3d, %3d) | load %3d/%-3d | latency %7s ms | active %s"
                             % (i, n.node_id, -1 if n.start_layer is None else n.start_layer,
                                -1 if n.end_layer is None else n.end_layer, n.current_requests,
                                n.max_requests, _fmt_lat(n.layer_latency_ms), n.is_active))
        return "\n".join(lines + self._standby_lines())
