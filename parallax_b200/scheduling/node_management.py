"""Thread-safe node registry with ACTIVE / STANDBY lifecycle and fixed-pipeline bookkeeping.

Counterpart of ``src/scheduling/node_management.py:18-520``. A *pipeline* is an ordered list
of nodes whose layer ranges tile ``[0, num_layers)`` without gap or overlap; its request
capacity is that of its tightest stage. When a member leaves, the whole pipeline is dissolved
and the remaining members return to STANDBY with their allocation cleared.
"""

from __future__ import annotations

import logging
import threading
from dataclasses import dataclass, field
from enum import Enum
from typing import Mapping, Optional, Sequence

from parallax_b200.scheduling.node import Node

logger = logging.getLogger(__name__)


class NodeState(str, Enum):
    ACTIVE = "active"
    STANDBY = "standby"


@dataclass
class Pipeline:
    nodes: list[Node]
    min_node_capacity: int = field(init=False, default=0)
    min_remaining_capacity: int = field(init=False, default=0)

    def __post_init__(self):
        if not self.nodes:
            raise ValueError("Pipeline is empty")
        inf = float("inf")
        self.nodes.sort(key=lambda n: (inf if n.start_layer is None else n.start_layer,
                                       inf if n.end_layer is None else n.end_layer))
        total = int(self.nodes[0].model_info.num_layers)
        pos = 0
        for n in self.nodes:
            if int(n.model_info.num_layers) != total:
                raise ValueError(f"Pipeline nodes disagree on model num_layers ({n.node_id})")
            if n.start_layer is None or n.end_layer is None:
                raise ValueError(f"Pipeline node {n.node_id} missing layer allocation")
            s, e = int(n.start_layer), int(n.end_layer)
            if s < 0 or e <= s or e > total:
                raise ValueError(f"Pipeline node {n.node_id} has invalid layer range [{s}, {e})")
            if s != pos:
                if pos == 0:
                    raise ValueError(f"Pipeline must start at layer 0; got {s} on node {n.node_id}")
                raise ValueError(f"Pipeline is not contiguous at node {n.node_id}: expected start {pos}, got {s}")
            pos = e
        if pos != total:
            raise ValueError(f"Pipeline must end at total_layers={total}; got {pos}")
        self.recompute_capacity()

    @property
    def node_ids(self) -> tuple[str, ...]:
        return tuple(n.node_id for n in self.nodes)

    @classmethod
    def from_node_ids(cls, node_ids: Sequence[str], *, nodes_by_id: Mapping[str, Node]) -> "Pipeline":
        nodes = []
        for nid in node_ids:
            n = nodes_by_id.get(nid)
            if n is None:
                raise ValueError(f"Node {nid} not found in registry")
            nodes.append(n)
        return cls(nodes=nodes)

    @property
    def num_stages(self) -> int:
        return len(self.nodes)

    @property
    def is_ready(self) -> bool:
        return all(bool(getattr(n, "is_active", False)) for n in self.nodes)

    def recompute_capacity(self) -> None:
        caps = [int(n.max_requests) for n in self.nodes]
        rem = [max(0, c - int(n.current_requests)) for c, n in zip(caps, self.nodes)]
        self.min_node_capacity = min(caps) if caps else 0
        self.min_remaining_capacity = min(rem) if rem else 0

    def capacity_report(self) -> tuple[int, int]:
        self.recompute_capacity()
        return self.min_node_capacity, self.min_remaining_capacity


class NodeManager:
    def __init__(self, *, initial_nodes: Optional[list[Node]] = None):
        self._lock = threading.RLock()
        self._nodes: dict[str, Node] = {}
        self._state: dict[str, NodeState] = {}
        self._registered_pipelines: dict[int, Pipeline] = {}
        self._node_to_pipeline: dict[str, int] = {}
        self.node_assigned_request_count: dict[str, int] = {}
        for n in initial_nodes or []:
            self.upsert(n, state=NodeState.STANDBY)

    # ---- membership
    def upsert(self, node: Node, *, state: Optional[NodeState] = None) -> None:
        with self._lock:
            self._nodes[node.node_id] = node
            if state is None:
                self._state.setdefault(node.node_id, NodeState.STANDBY)
            else:
                self._state[node.node_id] = state

    def get(self, node_id: str) -> Optional[Node]:
        with self._lock:
            return self._nodes.get(node_id)

    def state_of(self, node_id: str) -> Optional[NodeState]:
        with self._lock:
            return self._state.get(node_id)

    def _standby_locked(self, node_ids, *, allow_missing: bool = False) -> list[Node]:
        out = []
        for nid in node_ids:
            node = self._nodes.get(nid)
            if node is None:
                if allow_missing:
                    continue
                raise ValueError(f"Node {nid} not found in registry")
            prev = self._state.get(nid)
            if prev is not None and prev != NodeState.ACTIVE:
                raise ValueError(f"Node {nid} is not ACTIVE, current state: {prev}")
            self._state[nid] = NodeState.STANDBY
            self.node_assigned_request_count.pop(nid, None)
            out.append(node)
        return out

    def remove(self, node_id: str) -> Optional[Node]:
        """Drop a node; if it belonged to a fixed pipeline the pipeline is dissolved."""
        to_clear: list[Node] = []
        with self._lock:
            self._state.pop(node_id, None)
            removed = self._nodes.pop(node_id, None)
            if removed is None:
                return None
            self.node_assigned_request_count.pop(node_id, None)
            pid = self._node_to_pipeline.pop(node_id, None)
            if pid is not None:
                pipeline = self._registered_pipelines.pop(pid, None)
                if pipeline is not None:
                    members = list(pipeline.node_ids)
                    logger.warning("Node %s left; dissolving pipeline %s with members %s", node_id, pid, members)
                    for nid in members:
                        self._node_to_pipeline.pop(nid, None)
                    rest = [nid for nid in members if nid != node_id]
                    to_clear = self._standby_locked(rest, allow_missing=True)
        for n in to_clear:
            n.clear_serving_state()
        removed.clear_serving_state()
        return removed

    def activate(self, node_ids) -> None:
        with self._lock:
            for nid in node_ids:
                if nid not in self._nodes:
                    raise ValueError(f"Node {nid} not found in registry")
                if self._state.get(nid) != NodeState.STANDBY:
                    raise ValueError(f"Node {nid} is not STANDBY")
                self._state[nid] = NodeState.ACTIVE

    def standby(self, node_ids) -> None:
        with self._lock:
            nodes = self._standby_locked(list(node_ids))
        for n in nodes:
            n.clear_serving_state()

    def ids_to_nodes(self, node_ids) -> list[Node]:
        with self._lock:
            return [self._nodes[nid] for nid in node_ids]

    # ---- views
    @property
    def nodes(self) -> list[Node]:
        with self._lock:
            return list(self._nodes.values())

    @property
    def active_nodes(self) -> list[Node]:
        with self._lock:
            return [n for n in self._nodes.values() if self._state.get(n.node_id) == NodeState.ACTIVE]

    @property
    def standby_nodes(self) -> list[Node]:
        with self._lock:
            return [n for n in self._nodes.values() if self._state.get(n.node_id) == NodeState.STANDBY]

    @property
    def num_nodes(self) -> int:
        return len(self.nodes)

    @property
    def num_active_nodes(self) -> int:
        return len(self.active_nodes)

    @property
    def num_standby_nodes(self) -> int:
        return len(self.standby_nodes)

    def list_node_allocations(self, total_layers: int, ready_only: bool = False) -> list[tuple[str, int, int]]:
        if total_layers <= 0:
            return []
        out = []
        with self._lock:
            for nid, node in self._nodes.items():
                if self._state.get(nid) != NodeState.ACTIVE or (ready_only and not node.is_active):
                    continue
                s, e = node.start_layer, node.end_layer
                if s is None or e is None:
                    continue
                if s < 0 or e <= s or e > total_layers:
                    raise ValueError(f"Invalid layer range: {s}, {e} for node {nid}")
                out.append((nid, int(s), int(e)))
        return out

    def num_full_pipelines(self, total_layers: int, ready_only: bool = False) -> int:
        """Number of distinct node sequences covering [0, total_layers): a path count over
        layer boundaries (each ACTIVE allocation is an edge start -> end)."""
        segs = self.list_node_allocations(total_layers, ready_only)
        if not segs:
            return 0
        ways = {0: 1}
        for s, e in sorted((s, e) for _, s, e in segs):
            w = ways.get(s, 0)
            if w:
                ways[e] = ways.get(e, 0) + w
        return int(ways.get(total_layers, 0))

    def has_full_pipeline(self, num_total_layers: int, ready_only: bool = False) -> bool:
        return self.num_full_pipelines(num_total_layers, ready_only) > 0

    def add_request(self, node_id: str) -> None:
        with self._lock:
            node = self._nodes.get(node_id)
            if node is None:
                raise ValueError(f"Node {node_id} not found in registry")
            if self._state.get(node_id) != NodeState.ACTIVE:
                raise ValueError(f"Node {node_id} is not ACTIVE")
            self.node_assigned_request_count[node_id] = self.node_assigned_request_count.get(node_id, 0) + 1
            node.add_request()

    # ---- fixed pipelines (round-robin routing)
    def _register_locked(self, pid: int, p: Sequence[str], force_active: bool) -> None:
        self._registered_pipelines[pid] = Pipeline.from_node_ids(p, nodes_by_id=self._nodes)
        for nid in p:
            if nid in self._node_to_pipeline:
                raise ValueError(f"Node {nid} is already registered to pipeline {self._node_to_pipeline[nid]}")
            if force_active and self._state.get(nid) != NodeState.ACTIVE:
                logger.warning("Node %s is not ACTIVE.", nid)
                self._state[nid] = NodeState.ACTIVE
            self._node_to_pipeline[nid] = pid

    def register_pipelines(self, pipelines: list[list[str]]) -> dict[int, list[str]]:
        with self._lock:
            self._registered_pipelines, self._node_to_pipeline = {}, {}
            for pid, p in enumerate(pipelines):
                self._register_locked(pid, p, force_active=True)
            return {pid: list(p.node_ids) for pid, p in self._registered_pipelines.items()}

    def extend_registered_pipelines(self, pipelines: list[list[str]]) -> dict[int, list[str]]:
        with self._lock:
            nxt = max(self._registered_pipelines) + 1 if self._registered_pipelines else 0
            for p in pipelines:
                if not p:
                    continue
                self._register_locked(nxt, p, force_active=False)
                nxt += 1
            return {pid: list(p.node_ids) for pid, p in self._registered_pipelines.items()}

    def clear_registered_pipelines(self) -> None:
        with self._lock:
            still_active = [nid for nid in self._node_to_pipeline if self._state.get(nid) == NodeState.ACTIVE]
        self.standby(still_active)
        with self._lock:
            self._registered_pipelines, self._node_to_pipeline = {}, {}

    def get_registered_pipelines(self) -> dict[int, Pipeline]:
        with self._lock:
            return dict(self._registered_pipelines)

    def get_registered_pipeline_node_ids(self) -> dict[int, list[str]]:
        with self._lock:
            return {pid: list(p.node_ids) for pid, p in self._registered_pipelines.items()}

    def pipeline_id_of_node(self, node_id: str) -> Optional[int]:
        with self._lock:
            return self._node_to_pipeline.get(node_id)

    def report_pipeline_capacity(self, ready_only: bool = True):
        """(per-pipeline (capacity, remaining), total capacity, total remaining)."""
        with self._lock:
            if not self._registered_pipelines:
                return None, 0, 0
            per, total, cur = {}, 0, 0
            for pid in sorted(self._registered_pipelines):
                p = self._registered_pipelines[pid]
                p.recompute_capacity()
                remaining = 0 if (ready_only and not p.is_ready) else int(p.min_remaining_capacity)
                per[pid] = (int(p.min_node_capacity), remaining)
                total += int(p.min_node_capacity)
                cur += remaining
            return per, total, cur
