"""Registry of the cluster's nodes and of the fixed pipelines built from them.

A node is either STANDBY (known, hosting nothing) or ACTIVE (hosting a layer span). A *pipeline* is a
chain of nodes whose spans tile ``[0, num_layers)``; it serves as many requests as its tightest member.
Losing one member ends the pipeline: the others drop their layers and wait in STANDBY for the next
allocation. All state sits behind one re-entrant lock; node objects themselves are only touched outside
of it when that cannot race with a lookup (clearing a node that was just removed from every table).

Behavioural counterpart of ``src/scheduling/node_management.py:18-520`` (same states, same pipeline rule,
same capacity report), organised around one record per node instead of parallel tables.
"""

from __future__ import annotations

import logging
import threading
from enum import Enum
from typing import Iterable, Mapping, Optional, Sequence

from parallax_b200.scheduling.node import Node

logger = logging.getLogger(__name__)


class NodeState(str, Enum):
    ACTIVE = "active"
    STANDBY = "standby"


def _span_of(node: Node) -> tuple[int, int]:
    if node.start_layer is None or node.end_layer is None:
        raise ValueError(f"node {node.node_id} hosts no layers and cannot be a pipeline stage")
    return int(node.start_layer), int(node.end_layer)


class Pipeline:
    """Nodes ordered by layer span. Construction checks that the spans tile the model exactly."""

    def __init__(self, nodes: list[Node]):
        if not nodes:
            raise ValueError("a pipeline needs at least one node")
        depth = {int(n.model_info.num_layers) for n in nodes}
        if len(depth) != 1:
            raise ValueError(f"pipeline members were built for models of different depth: {sorted(depth)}")
        total = depth.pop()
        self.nodes = sorted(nodes, key=_span_of)
        cursor = 0
        for n in self.nodes:
            lo, hi = _span_of(n)
            if not 0 <= lo < hi <= total:
                raise ValueError(f"node {n.node_id} hosts [{lo}, {hi}), which is not a span of a {total}-layer model")
            if lo != cursor:
                kind = "gap" if lo > cursor else "overlap"
                raise ValueError(f"{kind} in the pipeline before node {n.node_id}: layers up to {cursor} are "
                                 f"covered, its span starts at {lo}")
            cursor = hi
        if cursor != total:
            raise ValueError(f"the pipeline stops at layer {cursor} of {total}")
        self.min_node_capacity = 0
        self.min_remaining_capacity = 0
        self.recompute_capacity()

    @classmethod
    def from_node_ids(cls, node_ids: Sequence[str], *, nodes_by_id: Mapping[str, Node]) -> "Pipeline":
        missing = [nid for nid in node_ids if nid not in nodes_by_id]
        if missing:
            raise ValueError(f"unknown node(s) {missing}")
        return cls([nodes_by_id[nid] for nid in node_ids])

    @property
    def node_ids(self) -> tuple[str, ...]:
        return tuple(n.node_id for n in self.nodes)

    @property
    def num_stages(self) -> int:
        return len(self.nodes)

    @property
    def is_ready(self) -> bool:
        """Every member reports itself able to serve."""
        return all(getattr(n, "is_active", False) for n in self.nodes)

    def recompute_capacity(self) -> None:
        """The tightest member sets the pipeline's capacity and what is left of it."""
        limits = [int(n.max_requests) for n in self.nodes]
        self.min_node_capacity = min(limits)
        self.min_remaining_capacity = min(max(lim - int(n.current_requests), 0) for lim, n in zip(limits, self.nodes))

    def capacity_report(self) -> tuple[int, int]:
        self.recompute_capacity()
        return self.min_node_capacity, self.min_remaining_capacity


class _Member:
    """Registry record of one node."""

    __slots__ = ("node", "state", "pipeline")

    def __init__(self, node: Node, state: NodeState):
        self.node = node
        self.state = state
        self.pipeline: Optional[int] = None      # id of the fixed pipeline the node belongs to


class NodeManager:
    def __init__(self, *, initial_nodes: Optional[list[Node]] = None):
        self._lock = threading.RLock()
        self._members: dict[str, _Member] = {}
        self._pipelines: dict[int, Pipeline] = {}
        # requests routed through each node since it was last activated (read by the router's log line)
        self.node_assigned_request_count: dict[str, int] = {}
        for n in initial_nodes or []:
            self.upsert(n, state=NodeState.STANDBY)

    # ------------------------------------------------------------------ membership
    def upsert(self, node: Node, *, state: Optional[NodeState] = None) -> None:
        """Add a node or replace its object; the state is kept unless one is given (new nodes start
        in STANDBY)."""
        with self._lock:
            rec = self._members.get(node.node_id)
            if rec is None:
                self._members[node.node_id] = _Member(node, state or NodeState.STANDBY)
            else:
                rec.node = node
                if state is not None:
                    rec.state = state

    def get(self, node_id: str) -> Optional[Node]:
        with self._lock:
            rec = self._members.get(node_id)
            return rec.node if rec else None

    def state_of(self, node_id: str) -> Optional[NodeState]:
        with self._lock:
            rec = self._members.get(node_id)
            return rec.state if rec else None

    def _require(self, node_id: str) -> _Member:
        rec = self._members.get(node_id)
        if rec is None:
            raise ValueError(f"node {node_id} is not registered")
        return rec

    def _to_standby_locked(self, node_ids: Iterable[str], skip_unknown: bool = False) -> list[Node]:
        """ACTIVE -> STANDBY for the given nodes (lock held). Returns the node objects, whose serving
        state the caller clears after releasing the lock."""
        moved = []
        for nid in node_ids:
            rec = self._members.get(nid)
            if rec is None:
                if skip_unknown:
                    continue
                raise ValueError(f"node {nid} is not registered")
            if rec.state is not NodeState.ACTIVE:
                raise ValueError(f"node {nid} cannot go to standby from state {rec.state.value}")
            rec.state = NodeState.STANDBY
            self.node_assigned_request_count.pop(nid, None)
            moved.append(rec.node)
        return moved

    def remove(self, node_id: str) -> Optional[Node]:
        """Forget a node. The fixed pipeline it was part of (if any) ends with it: its other members go
        back to STANDBY without layers."""
        orphans: list[Node] = []
        with self._lock:
            rec = self._members.pop(node_id, None)
            if rec is None:
                return None
            self.node_assigned_request_count.pop(node_id, None)
            if rec.pipeline is not None:
                pipe = self._pipelines.pop(rec.pipeline, None)
                if pipe is not None:
                    others = [nid for nid in pipe.node_ids if nid != node_id]
                    logger.warning("node %s left: pipeline %d (%s) is dissolved", node_id, rec.pipeline,
                                   ", ".join(pipe.node_ids))
                    for nid in others:
                        other = self._members.get(nid)
                        if other is not None:
                            other.pipeline = None
                    orphans = self._to_standby_locked(others, skip_unknown=True)
        for n in orphans:
            n.clear_serving_state()
        rec.node.clear_serving_state()
        return rec.node

    def activate(self, node_ids) -> None:
        with self._lock:
            for nid in node_ids:
                rec = self._require(nid)
                if rec.state is not NodeState.STANDBY:
                    raise ValueError(f"node {nid} is already {rec.state.value}; only standby nodes can be activated")
                rec.state = NodeState.ACTIVE

    def standby(self, node_ids) -> None:
        with self._lock:
            moved = self._to_standby_locked(list(node_ids))
        for n in moved:
            n.clear_serving_state()

    def ids_to_nodes(self, node_ids) -> list[Node]:
        with self._lock:
            return [self._members[nid].node for nid in node_ids]

    # ------------------------------------------------------------------ views
    def _select(self, state: Optional[NodeState]) -> list[Node]:
        with self._lock:
            return [m.node for m in self._members.values() if state is None or m.state is state]

    @property
    def nodes(self) -> list[Node]:
        return self._select(None)

    @property
    def active_nodes(self) -> list[Node]:
        return self._select(NodeState.ACTIVE)

    @property
    def standby_nodes(self) -> list[Node]:
        return self._select(NodeState.STANDBY)

    @property
    def num_nodes(self) -> int:
        with self._lock:
            return len(self._members)

    @property
    def num_active_nodes(self) -> int:
        return len(self.active_nodes)

    @property
    def num_standby_nodes(self) -> int:
        return len(self.standby_nodes)

    def list_node_allocations(self, total_layers: int, ready_only: bool = False) -> list[tuple[str, int, int]]:
        """``(node id, start, end)`` of every ACTIVE node that hosts layers (``ready_only``: and reports
        itself able to serve)."""
        if total_layers <= 0:
            return []
        spans = []
        with self._lock:
            for nid, rec in self._members.items():
                node = rec.node
                if rec.state is not NodeState.ACTIVE or node.start_layer is None or node.end_layer is None:
                    continue
                if ready_only and not node.is_active:
                    continue
                lo, hi = int(node.start_layer), int(node.end_layer)
                if not 0 <= lo < hi <= total_layers:
                    raise ValueError(f"node {nid} hosts [{lo}, {hi}), outside a {total_layers}-layer model")
                spans.append((nid, lo, hi))
        return spans

    def num_full_pipelines(self, total_layers: int, ready_only: bool = False) -> int:
        """How many different chains of ACTIVE nodes cover ``[0, total_layers)``: spans are edges between
        layer boundaries, and the chains are the paths from boundary 0 to boundary ``total_layers``."""
        paths_to = {0: 1}
        for _nid, lo, hi in sorted(self.list_node_allocations(total_layers, ready_only), key=lambda t: (t[1], t[2])):
            reach = paths_to.get(lo)
            if reach:
                paths_to[hi] = paths_to.get(hi, 0) + reach
        return paths_to.get(total_layers, 0) if total_layers > 0 else 0

    def has_full_pipeline(self, num_total_layers: int, ready_only: bool = False) -> bool:
        return self.num_full_pipelines(num_total_layers, ready_only) > 0

    def add_request(self, node_id: str) -> None:
        with self._lock:
            rec = self._require(node_id)
            if rec.state is not NodeState.ACTIVE:
                raise ValueError(f"node {node_id} is {rec.state.value} and takes no requests")
            self.node_assigned_request_count[node_id] = self.node_assigned_request_count.get(node_id, 0) + 1
            rec.node.add_request()

    # ------------------------------------------------------------------ fixed pipelines (round-robin routing)
    def _add_pipeline_locked(self, pid: int, node_ids: Sequence[str], promote: bool) -> None:
        by_id = {nid: m.node for nid, m in self._members.items()}
        pipe = Pipeline.from_node_ids(node_ids, nodes_by_id=by_id)
        taken = [nid for nid in node_ids if self._members[nid].pipeline is not None]
        if taken:
            raise ValueError(f"node(s) {taken} already belong to a pipeline")
        for nid in node_ids:
            rec = self._members[nid]
            if promote and rec.state is not NodeState.ACTIVE:
                logger.warning("node %s joins a pipeline while %s; marking it active", nid, rec.state.value)
                rec.state = NodeState.ACTIVE
            rec.pipeline = pid
        self._pipelines[pid] = pipe

    def _pipeline_ids_locked(self) -> dict[int, list[str]]:
        return {pid: list(p.node_ids) for pid, p in self._pipelines.items()}

    def _forget_pipelines_locked(self) -> None:
        self._pipelines = {}
        for rec in self._members.values():
            rec.pipeline = None

    def register_pipelines(self, pipelines: list[list[str]]) -> dict[int, list[str]]:
        """Replace the set of fixed pipelines (ids 0..n-1). Members are promoted to ACTIVE."""
        with self._lock:
            self._forget_pipelines_locked()
            for pid, ids in enumerate(pipelines):
                self._add_pipeline_locked(pid, ids, promote=True)
            return self._pipeline_ids_locked()

    def extend_registered_pipelines(self, pipelines: list[list[str]]) -> dict[int, list[str]]:
        """Add pipelines (empty ones are skipped) with ids following the existing ones."""
        with self._lock:
            pid = max(self._pipelines, default=-1) + 1
            for ids in pipelines:
                if ids:
                    self._add_pipeline_locked(pid, ids, promote=False)
                    pid += 1
            return self._pipeline_ids_locked()

    def clear_registered_pipelines(self) -> None:
        """Dissolve every fixed pipeline; members that were ACTIVE return to STANDBY without layers."""
        with self._lock:
            to_release = [nid for nid, m in self._members.items()
                          if m.pipeline is not None and m.state is NodeState.ACTIVE]
        self.standby(to_release)
        with self._lock:
            self._forget_pipelines_locked()

    def get_registered_pipelines(self) -> dict[int, Pipeline]:
        with self._lock:
            return dict(self._pipelines)

    def get_registered_pipeline_node_ids(self) -> dict[int, list[str]]:
        with self._lock:
            return self._pipeline_ids_locked()

    def pipeline_id_of_node(self, node_id: str) -> Optional[int]:
        with self._lock:
            rec = self._members.get(node_id)
            return rec.pipeline if rec else None

    def report_pipeline_capacity(self, ready_only: bool = True):
        """``({pipeline id: (capacity, remaining)}, total capacity, total remaining)``; a pipeline that is
        not ready counts with zero remaining when ``ready_only``. ``(None, 0, 0)`` without pipelines."""
        with self._lock:
            if not self._pipelines:
                return None, 0, 0
            report = {}
            for pid in sorted(self._pipelines):
                pipe = self._pipelines[pid]
                cap, left = pipe.capacity_report()
                if ready_only and not pipe.is_ready:
                    left = 0
                report[pid] = (int(cap), int(left))
            return report, sum(c for c, _ in report.values()), sum(r for _, r in report.values())
