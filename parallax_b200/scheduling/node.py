"""Scheduling primitives: hardware description, request signal, roofline model, node state.

Behavioural counterpart of ``src/scheduling/node.py:24-427``: a node's request capacity comes
from its KV budget, its layer capacity from its parameter-memory budget (with reservations
for the embedding table / lm_head at the pipeline ends), and its effective per-layer latency
is the measured EWMA plus a load term, or a roofline estimate when nothing was measured yet.
"""

from __future__ import annotations

import logging
import time
from dataclasses import dataclass, field
from math import floor
from typing import Optional

from parallax_b200.scheduling.model_info import ModelInfo

logger = logging.getLogger(__name__)

GiB = 1024 ** 3


@dataclass
class NodeHardwareInfo:
    node_id: str
    num_gpus: int
    tflops_fp16: float
    gpu_name: str
    memory_gb: float
    memory_bandwidth_gbps: float
    device: str


@dataclass
class RequestSignal:
    """routing_table: None = not assigned yet; [] = every pipeline is full right now."""

    request_id: str
    received_ts: float = field(default_factory=time.time)
    routing_table: Optional[list[str]] = None


def max_requests_for_kv_budget(requested: Optional[int], max_sequence_len: Optional[int], kv_bytes: int,
                               num_layers: int, num_kv_heads: int, head_dim_k: int, head_dim_v: int,
                               elem_bytes: int) -> int:
    """Concurrent requests that fit a KV budget at full sequence length (>= 1)."""
    per_token = num_layers * num_kv_heads * (head_dim_k + head_dim_v) * elem_bytes
    max_tokens = max(0, kv_bytes // per_token) if per_token > 0 else 0
    cap = None
    if max_sequence_len and max_tokens:
        cap = max(1, max_tokens // int(max_sequence_len))
    if requested is None:
        return 16 if cap is None else cap
    return min(requested, cap) if cap is not None else requested


class RooflinePerformanceModel:
    def __init__(self, hardware: NodeHardwareInfo, model_info: ModelInfo, quantization_speedup: float = 1.0, *,
                 batch_size: int = 1, target_seq_len: int = 1, source_seq_len: int = 256):
        self.tflops = hardware.tflops_fp16
        self.io_bandwidth = hardware.memory_bandwidth_gbps
        self.model_info = model_info
        self.quantization_speedup = quantization_speedup
        self.batch_size = batch_size
        self.target_seq_len = target_seq_len
        self.source_seq_len = source_seq_len

    def get_compute_roofline_latency_ms(self, flops: float) -> float:
        return flops / (self.quantization_speedup * self.tflops * 1e9)

    def get_io_roofline_latency_ms(self, io_bytes: float) -> float:
        return io_bytes / (self.io_bandwidth * 1e6)

    def set_sequence_shape(self, *, batch_size=None, target_seq_len=None, source_seq_len=None) -> None:
        if batch_size is not None:
            self.batch_size = batch_size
        if target_seq_len is not None:
            self.target_seq_len = target_seq_len
        if source_seq_len is not None:
            self.source_seq_len = source_seq_len

    def roofline_layer_latency_ms(self, include_input_embed: bool = False, include_lm_head: bool = False,
                                  num_current_layers: int = 1) -> float:
        """Average per-layer latency of a node hosting ``num_current_layers`` layers."""
        if num_current_layers <= 0:
            return float("inf")
        shape = dict(batch_size=self.batch_size, target_seq_len=self.target_seq_len,
                     source_seq_len=self.source_seq_len)
        layer_compute = self.get_compute_roofline_latency_ms(self.model_info.decoder_layer_flops(**shape))
        layer_io = self.get_io_roofline_latency_ms(self.model_info.decoder_layer_io_bytes(roofline=True, **shape))
        flops = io = 0
        if include_input_embed:
            io += self.model_info.embedding_io_bytes
        if include_lm_head:
            flops += self.model_info.lm_head_flops(self.target_seq_len)
            io += self.model_info.embedding_io_bytes
        ends = max(self.get_compute_roofline_latency_ms(flops), self.get_io_roofline_latency_ms(io))
        return (num_current_layers * max(layer_compute, layer_io) + ends) / num_current_layers


@dataclass
class Node:
    node_id: str
    hardware: NodeHardwareInfo
    model_info: ModelInfo
    kvcache_mem_ratio: float = 0.3
    param_mem_ratio: float = 0.5
    max_concurrent_requests: int = 16
    max_sequence_length: int = 4096
    manual_layer_assignment: bool = False
    start_layer: Optional[int] = None
    end_layer: Optional[int] = None
    current_requests: int = 0
    last_refit_time: float = 0.0
    is_active: bool = True
    last_heartbeat: float = 0.0
    avg_layer_latency_ms: Optional[float] = None
    load_compensator: float = 0.05
    rtt_to_nodes: Optional[dict[str, float]] = None
    _force_max_concurrent_requests: bool = False

    def __post_init__(self):
        if self.last_heartbeat == 0.0:
            self.last_heartbeat = time.time()
        if self.rtt_to_nodes is None:
            self.rtt_to_nodes = {}

    # ---- capacity
    @property
    def num_current_layers(self) -> int:
        if self.start_layer is None or self.end_layer is None:
            return 0
        return self.end_layer - self.start_layer

    @property
    def max_requests(self) -> int:
        if self._force_max_concurrent_requests or self.start_layer is None or self.end_layer is None:
            return self.max_concurrent_requests
        elem = int(getattr(self.model_info, "cache_bytes_per_element", 2) or 2)
        derived = max_requests_for_kv_budget(
            self.max_concurrent_requests, self.max_sequence_length,
            int(self.hardware.memory_gb * GiB * self.kvcache_mem_ratio), self.num_current_layers,
            self.model_info.num_kv_heads, self.model_info.head_size_k, self.model_info.head_size_v, elem)
        if derived <= 0:
            raise ValueError(f"Node {self.node_id} has invalid max concurrent requests: {derived}")
        if self.max_concurrent_requests is None:
            return derived
        return max(self.max_concurrent_requests, derived)

    @property
    def has_embedding(self) -> bool:
        return self.start_layer == 0 if self.start_layer is not None else False

    @property
    def has_lm_head(self) -> bool:
        return self.end_layer == self.model_info.num_layers if self.end_layer is not None else False

    @property
    def is_overloaded(self) -> bool:
        return self.current_requests >= self.max_requests

    def _param_budget_bytes(self) -> int:
        return floor(self.hardware.num_gpus * self.hardware.memory_gb * GiB * self.param_mem_ratio)

    def get_decoder_layer_capacity(self, include_input_embed: bool = False, include_lm_head: bool = False) -> int:
        """Decoder layers whose parameters fit this node's parameter-memory budget."""
        avail = self._param_budget_bytes()
        if include_input_embed:
            avail -= self.model_info.embedding_io_bytes
        if include_lm_head and not (include_input_embed and self.model_info.tie_embedding):
            avail -= self.model_info.embedding_io_bytes
        per_layer = self.model_info.decoder_layer_io_bytes(roofline=False)
        if self.hardware.device == "mlx":
            per_layer *= self.model_info.mlx_bit_factor
        return floor(avail / per_layer)

    @property
    def per_decoder_layer_kv_cache_memory(self) -> Optional[int]:
        if self.num_current_layers == 0:
            return None
        return floor(self.hardware.num_gpus * self.hardware.memory_gb * GiB * self.kvcache_mem_ratio
                     / self.num_current_layers)

    # ---- allocation state
    def set_layer_allocation(self, start_layer: int, end_layer: int) -> None:
        self.start_layer, self.end_layer = start_layer, end_layer

    def clear_layer_allocation(self) -> None:
        self.start_layer = self.end_layer = None

    def clear_serving_state(self) -> None:
        self.clear_layer_allocation()
        self.current_requests = 0
        self.avg_layer_latency_ms = None

    def hosts_layer(self, layer_id: int) -> bool:
        if self.start_layer is None or self.end_layer is None:
            return False
        return self.start_layer <= layer_id < self.end_layer

    def add_request(self) -> None:
        self.current_requests += 1

    def remove_request(self) -> None:
        self.current_requests -= 1

    # ---- latency
    def set_layer_latency_ms(self, latency_ms: float) -> None:
        self.avg_layer_latency_ms = latency_ms

    def roofline_layer_latency_ms(self) -> float:
        pb = float(self.model_info.param_bytes_per_element)
        base = 1.0 if pb <= 0 else 2.0 / pb
        eff = 0.8 if pb < 2.0 else 1.0  # sub-16-bit weights reach ~80 % of the ideal speed-up
        model = RooflinePerformanceModel(self.hardware, self.model_info, max(0.1, base * eff),
                                         batch_size=self.current_requests, target_seq_len=1,
                                         source_seq_len=self.max_sequence_length)
        return model.roofline_layer_latency_ms(include_input_embed=self.has_embedding,
                                               include_lm_head=self.has_lm_head,
                                               num_current_layers=self.num_current_layers)

    @property
    def layer_latency_ms(self) -> float:
        if self.is_overloaded:
            return float("inf")
        if self.avg_layer_latency_ms is None:
            return self.roofline_layer_latency_ms()
        return self.avg_layer_latency_ms + self.load_compensator * (self.current_requests / self.max_requests)

    # ---- network
    def update_rtt(self, target_node_id: str, rtt_ms: float) -> None:
        self.rtt_to_nodes[target_node_id] = rtt_ms

    def get_rtt_to(self, other: "Node") -> float:
        """Cached RTT in ms; falls back to the reverse direction; inf when unknown."""
        if self is other or self.node_id == other.node_id:
            return 0.0
        if self.rtt_to_nodes and other.node_id in self.rtt_to_nodes:
            return self.rtt_to_nodes[other.node_id]
        if other.rtt_to_nodes and self.node_id in other.rtt_to_nodes:
            return other.rtt_to_nodes[self.node_id]
        return float("inf")
