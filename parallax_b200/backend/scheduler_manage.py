"""Glue between the cluster backend's HTTP surface and the cluster scheduler.

``SchedulerManage`` owns the :class:`Scheduler` threads, answers cluster-status queries,
hands out routing tables, and keeps the node -> call URL map used to reach the first hop of a
pipeline. ``NodeRPCHandler`` implements the three node-facing calls (join, heartbeat update,
leave). In the reference these travel over a libp2p RPC layer
(``src/backend/server/scheduler_manage.py:19-336``, ``rpc_connection_handler.py:33-228``);
here they are plain JSON over the backend's own HTTP port, which is all a single box or a
rack needs.
"""

from __future__ import annotations

import logging
import os
import time
from typing import Optional

from parallax_b200.backend.static_config import get_model_info, get_node_join_command
from parallax_b200.scheduling.node import Node, NodeHardwareInfo, RequestSignal
from parallax_b200.scheduling.scheduler import Scheduler

logger = logging.getLogger(__name__)

NODE_STATUS_AVAILABLE = "available"
NODE_STATUS_WAITING = "waiting"


class NodeRPCHandler:
    def __init__(self, scheduler: Scheduler, call_urls: dict[str, str]):
        self.scheduler = scheduler
        self.call_urls = call_urls

    # ---- message -> Node
    @staticmethod
    def build_hardware(h: dict) -> NodeHardwareInfo:
        return NodeHardwareInfo(node_id=h.get("node_id"), num_gpus=h.get("num_gpus"), tflops_fp16=h.get("tflops_fp16"),
                                gpu_name=h.get("gpu_name"), memory_gb=h.get("memory_gb"),
                                memory_bandwidth_gbps=h.get("memory_bandwidth_gbps"), device=h.get("device"))

    def build_node(self, msg: dict) -> Node:
        kw = {}
        for k in ("kvcache_mem_ratio", "param_mem_ratio", "max_concurrent_requests", "max_sequence_length"):
            if msg.get(k) is not None:
                kw[k] = msg[k]
        node = Node(node_id=msg.get("node_id"), hardware=self.build_hardware(msg.get("hardware") or {}),
                    model_info=self.scheduler.model_info, is_active=msg.get("is_active", True),
                    manual_layer_assignment=msg.get("manual_layer_assignment", False),
                    last_refit_time=msg.get("last_refit_time", 0.0), **kw)
        for src, dst in (("start_layer", "start_layer"), ("end_layer", "end_layer"),
                         ("current_requests", "current_requests"), ("layer_latency_ms", "avg_layer_latency_ms"),
                         ("rtt_to_nodes", "rtt_to_nodes")):
            if msg.get(src) is not None:
                setattr(node, dst, msg[src])
        if msg.get("http_addr"):
            self.call_urls[node.node_id] = str(msg["http_addr"]).rstrip("/")
        return node

    # ---- allocation view
    def get_layer_allocation(self, node_id: str) -> dict:
        for nid, s, e in self.scheduler.list_node_allocations():
            if nid == node_id:
                node = self.scheduler.get_node(nid)
                if node is not None:
                    return {"node_id": nid, "model_name": node.model_info.model_name, "start_layer": s,
                            "end_layer": e, "tp_size": node.hardware.num_gpus,
                            "enable_weight_refit": self.scheduler.enable_weight_refit,
                            "weight_refit_mode": self.scheduler.weight_refit_mode}
        return {}

    def wait_layer_allocation(self, node_id: str, wait_seconds: float, poll: float = 0.05) -> dict:
        t0 = time.time()
        while True:
            alloc = self.get_layer_allocation(node_id)
            if alloc or time.time() - t0 > wait_seconds:
                return alloc
            time.sleep(poll)

    # ---- calls
    def node_join(self, msg: dict, wait_seconds: float = 300) -> dict:
        try:
            node = self.build_node(msg)
            self.scheduler.enqueue_join(node)
            return self.wait_layer_allocation(node.node_id, wait_seconds)
        except Exception as e:
            logger.exception("node_join failed: %s", e)
            return {}

    def node_leave(self, msg: dict) -> dict:
        try:
            nid = msg.get("node_id")
            self.scheduler.enqueue_leave(nid)
            self.call_urls.pop(nid, None)
        except Exception as e:
            logger.exception("node_leave failed: %s", e)
        return {}

    def node_update(self, msg: dict) -> tuple[dict, dict]:
        """Heartbeat. Returns (layer allocation, refit request to apply or {}). Unknown nodes are
        joined on the fly, which is how a node survives a scheduler restart."""
        try:
            node = self.build_node(msg)
            if self.scheduler.get_node(node.node_id) is None:
                self.scheduler.enqueue_join(node)
                return self.wait_layer_allocation(node.node_id, wait_seconds=5), {}
            self.scheduler.enqueue_node_update(
                node.node_id, current_requests=node.current_requests, layer_latency_ms=node.avg_layer_latency_ms,
                new_rtt_to_nodes=node.rtt_to_nodes or None, is_active=node.is_active,
                last_refit_time=node.last_refit_time)
            refit = {}
            if self.scheduler.refit_request and node.node_id not in self.scheduler.refit_set and node.is_active:
                refit = self.scheduler.refit_request
                self.scheduler.refit_set.add(node.node_id)
            return self.get_layer_allocation(node.node_id), refit
        except Exception as e:
            logger.exception("node_update failed: %s", e)
            return {}, {}


class SchedulerManage:
    def __init__(self, http_port: int = 3001, use_hfcache: bool = False, enable_weight_refit: bool = False,
                 weight_refit_mode: str = "disk", advertise_addr: Optional[str] = None,
                 scheduler_kwargs: Optional[dict] = None):
        self.http_port = http_port
        self.use_hfcache = use_hfcache
        self.enable_weight_refit = enable_weight_refit
        self.weight_refit_mode = weight_refit_mode
        self.advertise_addr = advertise_addr or f"127.0.0.1:{http_port}"
        self.scheduler_kwargs = scheduler_kwargs or {}
        self.model_name: Optional[str] = None
        self.init_nodes_num: Optional[int] = None
        self.is_local_network = True
        self.scheduler: Optional[Scheduler] = None
        self.call_urls: dict[str, str] = {}
        self.connection_handler: Optional[NodeRPCHandler] = None

    # ---- lifecycle
    def run(self, model_name: str, init_nodes_num: int, is_local_network: bool = True, model_info=None) -> None:
        if self.scheduler is not None:
            self.stop()
        self.is_local_network = is_local_network
        self.model_name, self.init_nodes_num = model_name, init_nodes_num
        info = model_info or get_model_info(model_name, self.use_hfcache)
        kw = dict(self.scheduler_kwargs)
        if "heartbeat_timeout" not in kw and os.environ.get("PARALLAX_HEARTBEAT_TIMEOUT_S"):
            # seconds of silence after which a node is dropped from the cluster (default 30)
            kw["heartbeat_timeout"] = float(os.environ["PARALLAX_HEARTBEAT_TIMEOUT_S"])
        self.scheduler = Scheduler(info, [], min_nodes_bootstrapping=init_nodes_num,
                                   enable_weight_refit=self.enable_weight_refit,
                                   weight_refit_mode=self.weight_refit_mode, **kw)
        self.connection_handler = NodeRPCHandler(self.scheduler, self.call_urls)
        self.scheduler.start(poll_interval=0.05)

    def is_running(self) -> bool:
        return self.scheduler is not None

    def stop(self) -> None:
        if self.scheduler is not None:
            self.scheduler.stop()
            time.sleep(0.1)
            self.scheduler = None

    # ---- queries
    def get_model_name(self):
        return self.model_name

    def get_init_nodes_num(self):
        return self.init_nodes_num

    def get_is_local_network(self) -> bool:
        return self.is_local_network

    def get_peer_id(self) -> str:
        return self.advertise_addr

    def need_more_nodes(self) -> bool:
        return self.scheduler.need_more_nodes() if self.scheduler else False

    def get_schedule_status(self) -> str:
        if self.scheduler is None:
            return NODE_STATUS_WAITING
        return NODE_STATUS_AVAILABLE if self.scheduler.has_full_pipeline() else NODE_STATUS_WAITING

    def build_node_info(self, node: Node) -> dict:
        return {"node_id": node.node_id, "status": NODE_STATUS_AVAILABLE if node.is_active else NODE_STATUS_WAITING,
                "gpu_num": node.hardware.num_gpus, "gpu_name": node.hardware.gpu_name,
                "gpu_memory": node.hardware.memory_gb, "start_layer": node.start_layer, "end_layer": node.end_layer}

    def get_node_list(self) -> list[dict]:
        return [self.build_node_info(n) for n in self.scheduler.node_manager.nodes] if self.scheduler else []

    def get_cluster_status(self) -> dict:
        return {"type": "cluster_status", "data": {
            "status": self.get_schedule_status(), "model_name": self.model_name, "init_nodes_num": self.init_nodes_num,
            "node_join_command": get_node_join_command(self.get_peer_id(), self.is_local_network),
            "node_list": self.get_node_list(), "need_more_nodes": self.need_more_nodes(),
            "max_running_request": self.scheduler.report_pipeline_capacity()[1] if self.scheduler else 0,
        }}

    # ---- refit
    def weight_refit(self, request_data: dict) -> bool:
        if self.scheduler is None:
            return False
        self.scheduler.refit_request = request_data
        self.scheduler.refit_set = set()
        return True

    def get_last_refit_time(self) -> float:
        return self.scheduler.update_last_refit_time() if self.scheduler else 0.0

    # ---- routing
    def get_routing_table(self, request_id, received_ts, wait_s: float = 5.0) -> Optional[list[str]]:
        """None: no routing possible yet; []: every pipeline is busy; otherwise the node path."""
        sig = RequestSignal(str(request_id), received_ts)
        self.scheduler.receive_request(sig)
        t0 = time.time()
        while sig.routing_table is None and time.time() - t0 < wait_s:
            time.sleep(0.005)
        return sig.routing_table

    def get_call_url_by_node_id(self, node_id: str) -> Optional[str]:
        return self.call_urls.get(node_id)

    def release_request(self, routing_table: list[str]) -> None:
        """A request finished: give its slots back on every node of its path."""
        if self.scheduler is None:
            return
        for nid in routing_table:
            node = self.scheduler.get_node(nid)
            if node is not None and node.current_requests > 0:
                node.remove_request()
