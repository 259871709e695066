"""Cluster scheduler: owns the node registry, the layer allocator and the request router.

Event-driven like ``src/scheduling/scheduler.py:29-649`` of the reference: joins, leaves and
heartbeat updates are queued and applied by one event thread; a dispatcher thread assigns a
routing table to every queued request signal; nodes silent for ``heartbeat_timeout`` seconds
are evicted; after a leave the cluster is globally re-allocated when no full pipeline is left
(or layer loads became too uneven). The ``_process_*`` methods can be called directly, which
is how the tests drive it without threads.
"""

from __future__ import annotations

import logging
import queue
import threading
import time
from collections import deque
from typing import Literal, Optional

from parallax_b200.scheduling.layer_allocation import DynamicProgrammingLayerAllocator, GreedyLayerAllocator
from parallax_b200.scheduling.model_info import ModelInfo
from parallax_b200.scheduling.node import Node, RequestSignal
from parallax_b200.scheduling.node_management import NodeManager
from parallax_b200.scheduling.request_routing import (DynamicProgrammingRouting,
                                                      RoundRobinOverFixedPipelinesRouting)

logger = logging.getLogger(__name__)


class Scheduler:
    def __init__(self, model_info: ModelInfo, nodes: list[Node], min_nodes_bootstrapping: int = 1,
                 enable_weight_refit: bool = False, weight_refit_mode: str = "disk",
                 strategy: Literal["greedy", "dp"] = "dp", routing_strategy: Literal["rr", "dp"] = "rr", *,
                 request_arrival_horizon_sec: float = 600.0, rebalance_threshold: float = float("inf"),
                 water_filling_max_iterations: int = 40, heartbeat_timeout: float = 30.0,
                 trim_layers_on_turning_points: bool = False):
        self.model_info = model_info
        self.num_layers = model_info.num_layers
        self.routing_strategy = routing_strategy
        self.enable_weight_refit = enable_weight_refit
        self.weight_refit_mode = weight_refit_mode
        self.node_manager = NodeManager(initial_nodes=nodes)
        self.dynamic_pipelines_router = routing_strategy == "dp"
        alloc_cls = GreedyLayerAllocator if strategy == "greedy" else DynamicProgrammingLayerAllocator
        self.layer_allocator = alloc_cls(
            model_info=model_info, node_management=self.node_manager,
            dynamic_pipelines_router=self.dynamic_pipelines_router, rebalance_threshold=rebalance_threshold,
            water_filling_max_iterations=water_filling_max_iterations,
            trim_layers_on_turning_points=trim_layers_on_turning_points)
        self.min_nodes_bootstrapping = min_nodes_bootstrapping
        if routing_strategy == "dp":
            self.request_router = DynamicProgrammingRouting(self.node_manager, self.num_layers)
        else:
            self.request_router = RoundRobinOverFixedPipelinesRouting(self.node_manager, self.num_layers,
                                                                      self.layer_allocator)
        self._request_queue: "queue.Queue[RequestSignal]" = queue.Queue()
        self.request_arrival_horizon_sec = request_arrival_horizon_sec
        self.heartbeat_timeout = heartbeat_timeout
        self._arrival_ts: deque = deque()
        self._pending_joins: "queue.Queue[Node]" = queue.Queue()
        self._pending_leaves: "queue.Queue[str]" = queue.Queue()
        self._pending_node_updates: queue.Queue = queue.Queue()
        self._stop_event = threading.Event()
        self._wake_event = threading.Event()
        self._bootstrapped_event = threading.Event()
        self._node_count_cv = threading.Condition()
        self._threads: list[threading.Thread] = []
        self.alloc_log_snapshot = ""
        # online weight refit (RL): the newest request and which nodes have applied it
        self.refit_request: dict = {}
        self.refit_set: set = set()
        self.last_refit_time = 0.0

    # ---- views
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
        return self._bootstrapped_event.is_set()

    def need_more_nodes(self) -> bool:
        return not self._bootstrapped_event.is_set() and not self.has_full_pipeline()

    # ---- allocation
    def bootstrap(self, reboot: bool = False) -> bool:
        if reboot:
            self.node_manager.clear_registered_pipelines()
            self._bootstrapped_event.clear()
        elif self._bootstrapped_event.is_set():
            return True
        if self.node_manager.num_nodes < self.min_nodes_bootstrapping and not reboot:
            return False
        if not self.layer_allocator.allocate_from_standby():
            self._bootstrapped_event.clear()
            return False
        self.request_router.bootstrap()
        self._bootstrapped_event.set()
        self.emit_alloc_log_snapshot(reason="Post Bootstrap")
        return True

    def update_last_refit_time(self) -> float:
        times = [n.last_refit_time for n in self.node_manager.nodes if n.last_refit_time >= self.last_refit_time]
        if times:
            self.last_refit_time = min(times)
        return self.last_refit_time

    def update_node_info(self, node: Node, *, current_requests=None, layer_latency_ms=None,
                         new_rtt_to_nodes=None, is_active=None, last_refit_time: Optional[float] = 0.0) -> None:
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

    # ---- event intake
    def enqueue_join(self, node: Node) -> None:
        self._pending_joins.put(node)
        self._wake_event.set()

    def enqueue_leave(self, node_id: str) -> None:
        self._pending_leaves.put(node_id)
        self._wake_event.set()

    def enqueue_node_update(self, node_id: str, *, current_requests=None, layer_latency_ms=None,
                            new_rtt_to_nodes=None, is_active=None, last_refit_time: Optional[float] = 0.0) -> None:
        self._pending_node_updates.put((node_id, current_requests, layer_latency_ms, new_rtt_to_nodes,
                                        is_active, last_refit_time))
        self._wake_event.set()

    def checking_node_heartbeat(self) -> None:
        now = time.time()
        for node in self.node_manager.active_nodes:
            if now - node.last_heartbeat > self.heartbeat_timeout:
                logger.warning("node %s missed heartbeats for %.1fs; evicting", node.node_id,
                               now - node.last_heartbeat)
                self.enqueue_leave(node.node_id)

    def join(self, node: Node) -> None:
        booted = self._bootstrapped_event.is_set()
        if self.node_manager.get(node.node_id) is None:
            self.node_manager.upsert(node)
            if booted:
                if self.dynamic_pipelines_router:
                    self.layer_allocator.dynamic_join(node)
                try:
                    self.request_router.expand_pipelines()
                except NotImplementedError:
                    pass
        if node.manual_layer_assignment:
            if node.start_layer is None or node.end_layer is None:
                raise ValueError(f"node {node.node_id} asks for manual assignment without a layer range")
            self.layer_allocator.allocate(node, node.start_layer, node.end_layer)
            if self.has_full_pipeline() and not self._bootstrapped_event.is_set():
                self._bootstrapped_event.set()
        elif booted:
            self.node_manager.upsert(node)
        self.emit_alloc_log_snapshot(reason=f"after join {node.node_id}")
        with self._node_count_cv:
            self._node_count_cv.notify_all()

    def _drop_layer_loads(self, node: Node) -> None:
        if node.start_layer is None or node.end_layer is None:
            return
        for l in range(node.start_layer, node.end_layer):
            ll = self.layer_allocator.layer_to_load.get(l)
            if ll is not None:
                ll.remove_node(node)

    def leave(self, node_id: str) -> None:
        """Remove a node. A fixed pipeline it belonged to is dissolved: the other members go
        back to STANDBY with their allocation cleared, so their hosting power is dropped too."""
        node = self.node_manager.get(node_id)
        if node is None:
            raise ValueError(f"Node {node_id} not found in nodes")
        affected = [node]
        pid = self.node_manager.pipeline_id_of_node(node_id)
        if pid is not None:
            members = self.node_manager.get_registered_pipeline_node_ids().get(pid, [])
            affected += [m for m in self.node_manager.ids_to_nodes([x for x in members if x != node_id])]
        for n in affected:
            self._drop_layer_loads(n)
        self.layer_allocator._update_layer_loads_heap()
        self.node_manager.remove(node_id)
        self.emit_alloc_log_snapshot(reason=f"after leave {node_id}")
        with self._node_count_cv:
            self._node_count_cv.notify_all()

    # ---- requests
    def receive_request(self, request: RequestSignal) -> None:
        self._request_queue.put(request)
        self._wake_event.set()
        now = time.time()
        self._arrival_ts.append(now)
        while self._arrival_ts and now - self._arrival_ts[0] > self.request_arrival_horizon_sec:
            self._arrival_ts.popleft()

    def dispatch_next_request(self, *, timeout: Optional[float] = None):
        """Pop one request signal and give it a routing table: (request_id, path, latency)."""
        if not self.request_router.routing_ready():
            return None
        try:
            req = self._request_queue.get(timeout=timeout) if timeout is not None else self._request_queue.get_nowait()
        except queue.Empty:
            return None
        path, latency = self.request_router.find_optimal_path(self.last_refit_time)
        req.routing_table = path
        for nid in path:
            self.node_manager.add_request(nid)
        return req.request_id, path, latency

    def emit_alloc_log_snapshot(self, *, reason: Optional[str] = None) -> str:
        try:
            snap = self.request_router.scheduler_format_snapshot()
        except Exception as exc:
            snap = f"(failed to build allocation snapshot: {exc})"
        self.alloc_log_snapshot = snap
        if reason:
            logger.debug("allocation snapshot (%s)\n%s", reason, snap)
        return snap

    # ---- queued-event processing (also called directly by tests)
    def _process_node_updates(self) -> None:
        while True:
            try:
                nid, cur, lat, rtts, active, refit = self._pending_node_updates.get_nowait()
            except queue.Empty:
                return
            node = self.node_manager.get(nid)
            if node is None:
                logger.warning("update for unknown node %s ignored", nid)
                continue
            self.update_node_info(node, current_requests=cur, layer_latency_ms=lat, new_rtt_to_nodes=rtts,
                                  is_active=active, last_refit_time=refit)

    def _process_joins(self) -> None:
        joined = manual = False
        while True:
            try:
                node = self._pending_joins.get_nowait()
            except queue.Empty:
                break
            self.join(node)
            joined = True
            manual = manual or node.manual_layer_assignment
        if joined and not self._bootstrapped_event.is_set() and not manual:
            if self.node_manager.num_standby_nodes >= self.min_nodes_bootstrapping:
                try:
                    if not self.bootstrap():
                        logger.info("bootstrap after join produced no full pipeline yet; waiting for more nodes")
                except Exception as exc:
                    logger.warning("bootstrap attempt failed: %s", exc)

    def _process_leaves(self) -> None:
        removed = False
        while True:
            try:
                nid = self._pending_leaves.get_nowait()
            except queue.Empty:
                break
            try:
                self.leave(nid)
                removed = True
            except Exception as exc:
                logger.warning("leave of %s failed: %s", nid, exc)
        if not removed or not self.layer_allocator.should_global_rebalance():
            return
        nodes = self.node_manager.nodes
        manual = sum(1 for n in nodes if n.manual_layer_assignment)
        if not nodes or manual:
            # manually placed nodes are never moved; an operator has to fix the gap
            return
        for n in self.node_manager.active_nodes:
            self._drop_layer_loads(n)
        self.layer_allocator._update_layer_loads_heap()
        self.node_manager.standby([n.node_id for n in self.node_manager.active_nodes])
        try:
            self.bootstrap(reboot=True)
        finally:
            self.emit_alloc_log_snapshot(reason="after global rebalance")

    # ---- threads
    def _event_loop(self, poll_interval: float) -> None:
        last_hb = 0.0
        while not self._stop_event.is_set():
            self._process_node_updates()
            self._process_joins()
            self._process_leaves()
            now = time.time()
            if now - last_hb >= max(0.5, poll_interval):
                self.checking_node_heartbeat()
                last_hb = now
            self._wake_event.wait(timeout=poll_interval)
            self._wake_event.clear()

    def _dispatch_loop(self, poll_interval: float) -> None:
        while not self._stop_event.is_set():
            if not self.request_router.routing_ready():
                time.sleep(max(0.0, poll_interval))
                continue
            self.dispatch_next_request(timeout=poll_interval)

    def start(self, *, poll_interval: float = 0.05) -> None:
        """Start the event and dispatcher threads without blocking (dispatch waits for bootstrap
        through ``routing_ready``)."""
        self._stop_event.clear()
        for name, fn in (("SchedulerEventLoop", self._event_loop), ("SchedulerDispatcher", self._dispatch_loop)):
            t = threading.Thread(target=fn, args=(poll_interval,), name=name, daemon=True)
            t.start()
            self._threads.append(t)

    def run(self, *, poll_interval: float = 0.05, allocation_log_interval: float = 5.0) -> None:
        """Blocking variant: start the threads and log allocation snapshots until ``stop()``."""
        self.start(poll_interval=poll_interval)
        try:
            while not self._stop_event.is_set():
                self.emit_alloc_log_snapshot()
                self._stop_event.wait(timeout=max(1.0, allocation_log_interval))
        finally:
            for t in self._threads:
                t.join(timeout=2.0)
            self._threads.clear()

    def wait_bootstrapped(self, timeout: Optional[float] = None) -> bool:
        return self._bootstrapped_event.wait(timeout)

    def stop(self) -> None:
        self._stop_event.set()
        self._wake_event.set()
        with self._node_count_cv:
            self._node_count_cv.notify_all()
