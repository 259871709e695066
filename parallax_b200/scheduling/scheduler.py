"""Cluster scheduler: one object that owns the node registry, the layer allocator and the request router.

Everything that changes the cluster arrives as an event - a node joins, a node leaves, a node reports
its load - and is applied by ONE thread in arrival-class order (reports, joins, leaves), so the allocator
never sees a half-applied change. A second thread hands every queued request a routing table as soon as
the router has a pipeline to offer. Nodes whose heartbeat stopped are turned into leave events; when a
departure leaves no complete pipeline (or skews the layer loads beyond the configured threshold) all
automatically placed nodes are sent back to standby and allocated afresh.

The event methods (`join`, `leave`, `apply_pending`) are plain calls, which is how the tests drive the
scheduler without threads. Behavioural counterpart of ``src/scheduling/scheduler.py:29-649``.
"""

from __future__ import annotations

import logging
import queue
import threading
import time
from collections import deque
from dataclasses import dataclass
from typing import Any, Literal, Optional

from parallax_b200.scheduling.layer_allocation import DynamicProgrammingLayerAllocator, GreedyLayerAllocator
from parallax_b200.scheduling.model_info import ModelInfo
from parallax_b200.scheduling.node import Node, RequestSignal
from parallax_b200.scheduling.node_management import NodeManager
from parallax_b200.scheduling.request_routing import (DynamicProgrammingRouting,
                                                      RoundRobinOverFixedPipelinesRouting)

logger = logging.getLogger(__name__)

_REPORT, _JOIN, _LEAVE = "report", "join", "leave"


@dataclass
class _NodeReport:
    """Load / health figures a node sends with its heartbeat; None = field not reported."""

    node_id: str
    current_requests: Optional[int] = None
    layer_latency_ms: Optional[float] = None
    new_rtt_to_nodes: Optional[dict] = None
    is_active: Optional[bool] = None
    last_refit_time: Optional[float] = 0.0


class _Mailbox:
    """Cluster events waiting for the event thread, one FIFO per kind."""

    def __init__(self):
        self._boxes: dict[str, "queue.SimpleQueue[Any]"] = {k: queue.SimpleQueue() for k in (_REPORT, _JOIN, _LEAVE)}
        self.bell = threading.Event()

    def post(self, kind: str, item: Any) -> None:
        self._boxes[kind].put(item)
        self.bell.set()

    def drain(self, kind: str) -> list:
        box, items = self._boxes[kind], []
        while True:
            try:
                items.append(box.get_nowait())
            except queue.Empty:
                return items


class Scheduler:
    def __init__(self, model_info: ModelInfo, nodes: list[Node], min_nodes_bootstrapping: int = 1,
                 enable_weight_refit: bool = False, weight_refit_mode: str = "disk",
                 strategy: Literal["greedy", "dp"] = "dp", routing_strategy: Literal["rr", "dp"] = "rr", *,
                 request_arrival_horizon_sec: float = 600.0, rebalance_threshold: float = float("inf"),
                 water_filling_max_iterations: int = 40, heartbeat_timeout: float = 30.0,
                 trim_layers_on_turning_points: bool = False):
        self.model_info = model_info
        self.num_layers = model_info.num_layers
        self.min_nodes_bootstrapping = min_nodes_bootstrapping
        self.enable_weight_refit = enable_weight_refit
        self.weight_refit_mode = weight_refit_mode
        self.routing_strategy = routing_strategy
        self.dynamic_pipelines_router = routing_strategy == "dp"
        self.request_arrival_horizon_sec = request_arrival_horizon_sec
        self.heartbeat_timeout = heartbeat_timeout
        self.node_manager = NodeManager(initial_nodes=nodes)
        allocator = {"greedy": GreedyLayerAllocator}.get(strategy, DynamicProgrammingLayerAllocator)
        self.layer_allocator = allocator(model_info=model_info, node_management=self.node_manager,
                                         dynamic_pipelines_router=self.dynamic_pipelines_router,
                                         rebalance_threshold=rebalance_threshold,
                                         water_filling_max_iterations=water_filling_max_iterations,
                                         trim_layers_on_turning_points=trim_layers_on_turning_points)
        if self.dynamic_pipelines_router:
            self.request_router = DynamicProgrammingRouting(self.node_manager, self.num_layers)
        else:
            self.request_router = RoundRobinOverFixedPipelinesRouting(self.node_manager, self.num_layers,
                                                                      self.layer_allocator)
        self._mail = _Mailbox()
        self._requests: "queue.Queue[RequestSignal]" = queue.Queue()
        self._recent_arrivals: deque = deque()          # arrival times within the horizon (rate estimate)
        self._ready = threading.Event()                 # a full pipeline has been allocated
        self._halt = threading.Event()
        self._membership_changed = threading.Condition()
        self._workers: list[threading.Thread] = []
        self.alloc_log_snapshot = ""
        # online weight refit (RL): the newest request and which nodes have applied it
        self.refit_request: dict = {}
        self.refit_set: set = set()
        self.last_refit_time = 0.0

    # ------------------------------------------------------------------ views
    def list_node_allocations(self, total_layers: Optional[int] = None):
        return self.node_manager.list_node_allocations(total_layers or self.num_layers)

    def get_node(self, node_id: str) -> Optional[Node]:
        return self.node_manager.get(node_id)

    def has_full_pipeline(self) -> bool:
        return self.node_manager.has_full_pipeline(self.num_layers)

    def report_pipeline_capacity(self, ready_only: bool = True):
        return self.node_manager.report_pipeline_capacity(ready_only=ready_only)

    @property
    def bootstrapped(self) -> bool:
        return self._ready.is_set()

    def need_more_nodes(self) -> bool:
        return not (self.bootstrapped or self.has_full_pipeline())

    def wait_bootstrapped(self, timeout: Optional[float] = None) -> bool:
        return self._ready.wait(timeout)

    def emit_alloc_log_snapshot(self, *, reason: Optional[str] = None) -> str:
        """Refresh (and at debug level log) the router's table of who hosts what."""
        try:
            text = self.request_router.scheduler_format_snapshot()
        except Exception as exc:      # a log line must never break scheduling
            text = f"(no allocation snapshot: {exc})"
        self.alloc_log_snapshot = text
        if reason:
            logger.debug("allocation %s:\n%s", reason, text)
        return text

    # ------------------------------------------------------------------ allocation
    def bootstrap(self, reboot: bool = False) -> bool:
        """Allocate layers to the standby nodes and let the router build its pipelines. Returns whether
        the cluster can serve afterwards. ``reboot`` first dissolves the existing pipelines and ignores
        the minimum node count (used for a global re-allocation)."""
        if reboot:
            self.node_manager.clear_registered_pipelines()
            self._ready.clear()
        else:
            if self.bootstrapped:
                return True
            if self.node_manager.num_nodes < self.min_nodes_bootstrapping:
                return False
        if not self.layer_allocator.allocate_from_standby():
            self._ready.clear()
            return False
        self.request_router.bootstrap()
        self._ready.set()
        self.emit_alloc_log_snapshot(reason="after bootstrap")
        return True

    def _release_layers(self, nodes: list[Node]) -> None:
        """Take the nodes' hosting power out of the allocator's per-layer load table."""
        table = self.layer_allocator.layer_to_load
        for node in nodes:
            if node.start_layer is None or node.end_layer is None:
                continue
            for layer in range(node.start_layer, node.end_layer):
                entry = table.get(layer)
                if entry is not None:
                    entry.remove_node(node)
        self.layer_allocator._update_layer_loads_heap()

    def _reallocate_everything(self) -> None:
        active = self.node_manager.active_nodes
        self._release_layers(active)
        self.node_manager.standby([n.node_id for n in active])
        try:
            self.bootstrap(reboot=True)
        finally:
            self.emit_alloc_log_snapshot(reason="after global re-allocation")

    # ------------------------------------------------------------------ membership (direct calls)
    def join(self, node: Node) -> None:
        """Register a node. Before the first allocation it just waits in standby; afterwards the
        allocator places it (dynamic routing) or the router tries to form one more pipeline with it.
        A node that brings its own layer range is placed there at once."""
        serving = self.bootstrapped
        is_new = self.node_manager.get(node.node_id) is None
        if is_new:
            self.node_manager.upsert(node)
            if serving:
                if self.dynamic_pipelines_router:
                    self.layer_allocator.dynamic_join(node)
                try:
                    self.request_router.expand_pipelines()
                except NotImplementedError:
                    pass
        if node.manual_layer_assignment:
            if node.start_layer is None or node.end_layer is None:
                raise ValueError(f"node {node.node_id} wants a manual placement but names no layer range")
            self.layer_allocator.allocate(node, node.start_layer, node.end_layer)
            if self.has_full_pipeline():
                # the hand-placed nodes cover every layer: a router that works from registered pipelines learns
                # them now (it is only asked for a path once it reports a ready pipeline)
                register = getattr(self.request_router, "bootstrap", None)
                if register is not None:
                    register()
                if not self.bootstrapped:
                    self._ready.set()
        elif serving and not is_new:
            self.node_manager.upsert(node)      # a re-join replaces the node object
        self.emit_alloc_log_snapshot(reason=f"after {node.node_id} joined")
        self._notify_membership()

    def leave(self, node_id: str) -> None:
        """Remove a node and, with it, the fixed pipeline it belonged to: the other members lose their
        layers too (they return to standby), so their share of the layer loads is released as well."""
        node = self.node_manager.get(node_id)
        if node is None:
            raise ValueError(f"cannot remove {node_id}: no such node")
        losing_layers = [node]
        pipeline = self.node_manager.pipeline_id_of_node(node_id)
        if pipeline is not None:
            mates = [nid for nid in self.node_manager.get_registered_pipeline_node_ids().get(pipeline, ())
                     if nid != node_id]
            losing_layers.extend(self.node_manager.ids_to_nodes(mates))
        self._release_layers(losing_layers)
        self.node_manager.remove(node_id)
        self.emit_alloc_log_snapshot(reason=f"after {node_id} left")
        self._notify_membership()

    def _notify_membership(self) -> None:
        with self._membership_changed:
            self._membership_changed.notify_all()

    # ------------------------------------------------------------------ node reports
    def update_node_info(self, node: Node, *, current_requests=None, layer_latency_ms=None,
                         new_rtt_to_nodes=None, is_active=None, last_refit_time: Optional[float] = 0.0) -> None:
        """Apply a heartbeat's figures to the node object and stamp the heartbeat time."""
        if current_requests is not None:
            node.current_requests = current_requests
        if layer_latency_ms is not None:
            node.set_layer_latency_ms(layer_latency_ms)
        if new_rtt_to_nodes is not None:
            node.rtt_to_nodes = new_rtt_to_nodes
        if is_active is not None:
            node.is_active = is_active
        if last_refit_time and last_refit_time > 0.0:
            node.last_refit_time = last_refit_time
        node.last_heartbeat = time.time()

    def update_last_refit_time(self) -> float:
        """The cluster's refit time is that of the node furthest behind among the nodes that are at or
        past the current value."""
        caught_up = [n.last_refit_time for n in self.node_manager.nodes if n.last_refit_time >= self.last_refit_time]
        if caught_up:
            self.last_refit_time = min(caught_up)
        return self.last_refit_time

    def checking_node_heartbeat(self) -> None:
        """Queue a leave for every active node that has been silent for longer than the timeout."""
        now = time.time()
        for node in self.node_manager.active_nodes:
            silent = now - node.last_heartbeat
            if silent > self.heartbeat_timeout:
                logger.warning("no heartbeat from node %s for %.1f s: removing it", node.node_id, silent)
                self.enqueue_leave(node.node_id)

    # ------------------------------------------------------------------ event intake (any thread)
    def enqueue_join(self, node: Node) -> None:
        self._mail.post(_JOIN, node)

    def enqueue_leave(self, node_id: str) -> None:
        self._mail.post(_LEAVE, node_id)

    def enqueue_node_update(self, node_id: str, *, current_requests=None, layer_latency_ms=None,
                            new_rtt_to_nodes=None, is_active=None, last_refit_time: Optional[float] = 0.0) -> None:
        self._mail.post(_REPORT, _NodeReport(node_id, current_requests, layer_latency_ms, new_rtt_to_nodes,
                                             is_active, last_refit_time))

    # ------------------------------------------------------------------ event application (event thread or tests)
    def _apply_reports(self) -> None:
        for rep in self._mail.drain(_REPORT):
            node = self.node_manager.get(rep.node_id)
            if node is None:
                logger.warning("report from unknown node %s dropped", rep.node_id)
                continue
            self.update_node_info(node, current_requests=rep.current_requests, layer_latency_ms=rep.layer_latency_ms,
                                  new_rtt_to_nodes=rep.new_rtt_to_nodes, is_active=rep.is_active,
                                  last_refit_time=rep.last_refit_time)

    def _apply_joins(self) -> None:
        newcomers = self._mail.drain(_JOIN)
        for node in newcomers:
            self.join(node)
        if not newcomers or self.bootstrapped or any(n.manual_layer_assignment for n in newcomers):
            return
        if self.node_manager.num_standby_nodes < self.min_nodes_bootstrapping:
            return
        try:
            if not self.bootstrap():
                logger.info("not enough capacity for a full pipeline yet; waiting for more nodes")
        except Exception as exc:
            logger.warning("allocation after a join failed: %s", exc)

    def _apply_leaves(self) -> None:
        gone = 0
        for node_id in self._mail.drain(_LEAVE):
            try:
                self.leave(node_id)
                gone += 1
            except Exception as exc:
                logger.warning("could not remove node %s: %s", node_id, exc)
        if not gone or not self.layer_allocator.should_global_rebalance():
            return
        remaining = self.node_manager.nodes
        if not remaining or any(n.manual_layer_assignment for n in remaining):
            return      # manually placed nodes are never moved: an operator has to close the gap
        self._reallocate_everything()

    def apply_pending(self) -> None:
        """Apply every queued event: reports first (so decisions see fresh loads), then joins, then leaves."""
        self._apply_reports()
        self._apply_joins()
        self._apply_leaves()

    # names under which the steps are also reachable one by one
    _process_node_updates = _apply_reports
    _process_joins = _apply_joins
    _process_leaves = _apply_leaves

    # ------------------------------------------------------------------ requests
    def receive_request(self, request: RequestSignal) -> None:
        self._requests.put(request)
        self._mail.bell.set()
        now = time.time()
        arrivals = self._recent_arrivals
        arrivals.append(now)
        oldest_kept = now - self.request_arrival_horizon_sec
        while arrivals and arrivals[0] < oldest_kept:
            arrivals.popleft()

    def dispatch_next_request(self, *, timeout: Optional[float] = None):
        """Give the oldest queued request a routing table. Returns ``(request id, path, latency)`` or
        None when the router has no pipeline yet or no request is waiting."""
        if not self.request_router.routing_ready():
            return None
        try:
            request = self._requests.get(timeout=timeout) if timeout is not None else self._requests.get_nowait()
        except queue.Empty:
            return None
        path, latency = self.request_router.find_optimal_path(self.last_refit_time)
        request.routing_table = path
        for node_id in path:
            self.node_manager.add_request(node_id)
        return request.request_id, path, latency

    # ------------------------------------------------------------------ threads
    def _event_worker(self, poll_interval: float) -> None:
        heartbeat_every = max(0.5, poll_interval)
        next_check = 0.0
        while not self._halt.is_set():
            self.apply_pending()
            now = time.time()
            if now >= next_check:
                self.checking_node_heartbeat()
                next_check = now + heartbeat_every
            self._mail.bell.wait(timeout=poll_interval)
            self._mail.bell.clear()

    def _dispatch_worker(self, poll_interval: float) -> None:
        while not self._halt.is_set():
            if self.request_router.routing_ready():
                self.dispatch_next_request(timeout=poll_interval)
            else:
                self._retry_pipeline_registration()
                time.sleep(max(0.0, poll_interval))

    def _retry_pipeline_registration(self, every_s: float = 1.0) -> None:
        """A router that works from registered pipelines found none it could price when the cluster came up
        (the nodes had not measured the hops between them yet): look again until one is ready."""
        router = self.request_router
        if not self.bootstrapped or not hasattr(router, "get_registered_pipelines") or not hasattr(router, "bootstrap"):
            return
        now = time.time()
        if now - getattr(self, "_last_registration_try", 0.0) < every_s or router.get_registered_pipelines():
            return
        self._last_registration_try = now
        try:
            if router.bootstrap():
                logger.info("pipelines registered: %s", router.get_registered_pipelines())
        except Exception as e:
            logger.debug("pipeline registration not possible yet: %s", e)

    def start(self, *, poll_interval: float = 0.05) -> None:
        """Start the event thread and the dispatcher without blocking; dispatching begins by itself
        once the router reports a ready pipeline."""
        self._halt.clear()
        for name, body in (("SchedulerEventLoop", self._event_worker), ("SchedulerDispatcher", self._dispatch_worker)):
            worker = threading.Thread(target=body, args=(poll_interval,), name=name, daemon=True)
            worker.start()
            self._workers.append(worker)

    def run(self, *, poll_interval: float = 0.05, allocation_log_interval: float = 5.0) -> None:
        """Blocking variant of :meth:`start`: refreshes the allocation snapshot until :meth:`stop`."""
        self.start(poll_interval=poll_interval)
        try:
            while not self._halt.wait(timeout=max(1.0, allocation_log_interval)):
                self.emit_alloc_log_snapshot()
        finally:
            for worker in self._workers:
                worker.join(timeout=2.0)
            self._workers.clear()

    def stop(self) -> None:
        self._halt.set()
        self._mail.bell.set()
        self._notify_membership()
