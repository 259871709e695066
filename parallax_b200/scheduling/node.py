"""What the cluster scheduler knows about one serving node.

Three questions are answered here, each by its own small piece:

* **How many requests fit?**  :func:`max_requests_for_kv_budget` turns a KV-cache byte budget into a
  number of full-length sequences.
* **How many layers fit?**  :class:`_MemoryPlan` splits a node's device memory into a parameter share
  and a KV share and prices a decoder layer, the embedding table and the lm_head against it.
* **How fast is a layer?**  :class:`RooflinePerformanceModel` gives the slower of compute time and
  memory time for one decode step; a node that has reported measurements uses those plus a load term.

Same behaviour as the reference's node model (``src/scheduling/node.py:24-427``): capacities and
latencies computed from the same quantities, so that the allocator and the router make the same
decisions; the public names (``Node.max_requests``, ``layer_latency_ms``, ``get_decoder_layer_capacity``,
``get_rtt_to`` ...) are the interface the allocator, router and backend are written against.
"""

from __future__ import annotations

import logging
import math
import time
from dataclasses import dataclass, field
from typing import Optional

from parallax_b200.scheduling.model_info import ModelInfo

logger = logging.getLogger(__name__)

_BYTES_PER_GIB = float(1 << 30)
_DEFAULT_REQUESTS_WITHOUT_BUDGET = 16


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
    """A request as the router sees it. ``routing_table`` is None until a path was chosen and an
    empty list when every pipeline was full at that moment."""

    request_id: str
    received_ts: float = field(default_factory=time.time)
    routing_table: Optional[list[str]] = None


def max_requests_for_kv_budget(requested: Optional[int], max_sequence_len: Optional[int], kv_bytes: int,
                               num_layers: int, num_kv_heads: int, head_dim_k: int, head_dim_v: int,
                               elem_bytes: int) -> int:
    """Full-length sequences whose K and V fit ``kv_bytes`` on ``num_layers`` layers, never below one;
    bounded by ``requested`` when the caller asked for a specific number. Without a usable budget
    (zero bytes per token, unknown sequence length) the request count asked for stands, or 16."""
    bytes_per_token = num_layers * num_kv_heads * (head_dim_k + head_dim_v) * elem_bytes
    fits = None
    if bytes_per_token > 0 and max_sequence_len:
        tokens = kv_bytes // bytes_per_token
        if tokens > 0:
            fits = max(tokens // int(max_sequence_len), 1)
    if fits is None:
        return _DEFAULT_REQUESTS_WITHOUT_BUDGET if requested is None else requested
    return fits if requested is None else min(requested, fits)


class RooflinePerformanceModel:
    """Latency of one decode step of one layer as max(FLOPs / peak, bytes / bandwidth).

    ``quantization_speedup`` scales the compute peak (weights below 16 bit run the GEMMs faster). The
    sequence shape (batch, new tokens per sequence, context length) can be changed between queries."""

    def __init__(self, hardware: NodeHardwareInfo, model_info: ModelInfo, quantization_speedup: float = 1.0, *,
                 batch_size: int = 1, target_seq_len: int = 1, source_seq_len: int = 256):
        self.model_info = model_info
        self.tflops = hardware.tflops_fp16
        self.io_bandwidth = hardware.memory_bandwidth_gbps
        self.quantization_speedup = quantization_speedup
        self.batch_size, self.target_seq_len, self.source_seq_len = batch_size, target_seq_len, source_seq_len

    # unit bookkeeping: TFLOP/s * 1e9 = FLOP per millisecond; GB/s * 1e6 = bytes per millisecond
    def get_compute_roofline_latency_ms(self, flops: float) -> float:
        flop_per_ms = self.tflops * self.quantization_speedup * 1e9
        return flops / flop_per_ms

    def get_io_roofline_latency_ms(self, io_bytes: float) -> float:
        return io_bytes / (self.io_bandwidth * 1e6)

    def set_sequence_shape(self, *, batch_size=None, target_seq_len=None, source_seq_len=None) -> None:
        for name, value in (("batch_size", batch_size), ("target_seq_len", target_seq_len),
                            ("source_seq_len", source_seq_len)):
            if value is not None:
                setattr(self, name, value)

    def _bound(self, flops: float, io_bytes: float) -> float:
        return max(self.get_compute_roofline_latency_ms(flops), self.get_io_roofline_latency_ms(io_bytes))

    def roofline_layer_latency_ms(self, include_input_embed: bool = False, include_lm_head: bool = False,
                                  num_current_layers: int = 1) -> float:
        """Mean per-layer latency of a node that hosts ``num_current_layers`` layers; the cost of the
        embedding lookup and the lm_head (pipeline ends) is spread over those layers."""
        if num_current_layers <= 0:
            return math.inf
        mi = self.model_info
        shape = {"batch_size": self.batch_size, "target_seq_len": self.target_seq_len,
                 "source_seq_len": self.source_seq_len}
        one_layer = self._bound(mi.decoder_layer_flops(**shape), mi.decoder_layer_io_bytes(roofline=True, **shape))
        end_flops = mi.lm_head_flops(self.target_seq_len) if include_lm_head else 0
        end_bytes = mi.embedding_io_bytes * (int(include_input_embed) + int(include_lm_head))
        total = one_layer * num_current_layers + self._bound(end_flops, end_bytes)
        return total / num_current_layers


class _MemoryPlan:
    """Byte budgets of a node: a share of device memory for parameters, a share for the KV cache."""

    def __init__(self, hardware: NodeHardwareInfo, param_ratio: float, kv_ratio: float):
        self.hardware, self.param_ratio, self.kv_ratio = hardware, param_ratio, kv_ratio

    def _device_bytes(self, all_gpus: bool = True) -> float:
        gpus = max(self.hardware.num_gpus, 1) if all_gpus else 1      # a CPU-only node counts as one device
        return gpus * self.hardware.memory_gb * _BYTES_PER_GIB

    @property
    def param_bytes(self) -> int:
        return math.floor(self._device_bytes() * self.param_ratio)

    @property
    def kv_bytes(self) -> int:
        return math.floor(self._device_bytes() * self.kv_ratio)

    @property
    def kv_bytes_one_gpu(self) -> int:
        return int(self._device_bytes(all_gpus=False) * self.kv_ratio)

    def layers_that_fit(self, model: ModelInfo, with_embedding: bool, with_lm_head: bool) -> int:
        left = self.param_bytes
        tables = int(with_embedding)
        if with_lm_head and not (with_embedding and model.tie_embedding):
            tables += 1          # a tied lm_head shares the embedding table that is already counted
        left -= tables * model.embedding_io_bytes
        layer_bytes = model.decoder_layer_io_bytes(roofline=False)
        if self.hardware.device == "mlx":
            layer_bytes *= model.mlx_bit_factor
        return math.floor(left / layer_bytes)


class Node:
    """A serving node: hardware, the layer span it hosts, its load and its measured speed."""

    def __init__(self, node_id: str, hardware: NodeHardwareInfo, model_info: ModelInfo, kvcache_mem_ratio: float = 0.3,
                 param_mem_ratio: float = 0.5, max_concurrent_requests: int = 16, max_sequence_length: int = 4096,
                 manual_layer_assignment: bool = False, start_layer: Optional[int] = None,
                 end_layer: Optional[int] = None, current_requests: int = 0, last_refit_time: float = 0.0,
                 is_active: bool = True, last_heartbeat: float = 0.0, avg_layer_latency_ms: Optional[float] = None,
                 load_compensator: float = 0.05, rtt_to_nodes: Optional[dict[str, float]] = None,
                 _force_max_concurrent_requests: bool = False):
        self.node_id = node_id
        self.hardware = hardware
        self.model_info = model_info
        self.kvcache_mem_ratio = kvcache_mem_ratio
        self.param_mem_ratio = param_mem_ratio
        self.max_concurrent_requests = max_concurrent_requests
        self.max_sequence_length = max_sequence_length
        self.manual_layer_assignment = manual_layer_assignment
        self.start_layer, self.end_layer = start_layer, end_layer
        self.current_requests = current_requests
        self.last_refit_time = last_refit_time
        self.is_active = is_active
        self.last_heartbeat = last_heartbeat or time.time()
        self.avg_layer_latency_ms = avg_layer_latency_ms
        self.load_compensator = load_compensator
        self.rtt_to_nodes = rtt_to_nodes if rtt_to_nodes is not None else {}      # any mapping: node id -> ms
        # take max_concurrent_requests as given instead of deriving the capacity from the KV budget
        self._force_max_concurrent_requests = _force_max_concurrent_requests

    def __repr__(self) -> str:
        return (f"Node({self.node_id}, layers=[{self.start_layer}, {self.end_layer}), "
                f"requests={self.current_requests}, active={self.is_active})")

    def _memory(self) -> _MemoryPlan:
        return _MemoryPlan(self.hardware, self.param_mem_ratio, self.kvcache_mem_ratio)

    # ------------------------------------------------------------------ layer span
    @property
    def _has_span(self) -> bool:
        return self.start_layer is not None and self.end_layer is not None

    @property
    def num_current_layers(self) -> int:
        return self.end_layer - self.start_layer if self._has_span else 0

    @property
    def has_embedding(self) -> bool:
        return self.start_layer is not None and self.start_layer == 0

    @property
    def has_lm_head(self) -> bool:
        return self.end_layer is not None and self.end_layer == self.model_info.num_layers

    def set_layer_allocation(self, start_layer: int, end_layer: int) -> None:
        self.start_layer, self.end_layer = start_layer, end_layer

    def clear_layer_allocation(self) -> None:
        self.start_layer = self.end_layer = None

    def clear_serving_state(self) -> None:
        """Back to a blank standby node: no layers, no load, no measurements."""
        self.clear_layer_allocation()
        self.current_requests = 0
        self.avg_layer_latency_ms = None

    def hosts_layer(self, layer_id: int) -> bool:
        return self._has_span and self.start_layer <= layer_id < self.end_layer

    # ------------------------------------------------------------------ capacity
    @property
    def max_requests(self) -> int:
        """Concurrent requests this node takes: what the KV share holds at full sequence length on the
        hosted layers, but never less than the configured ``max_concurrent_requests``."""
        configured = self.max_concurrent_requests
        if self._force_max_concurrent_requests or not self._has_span:
            return configured
        elem = int(getattr(self.model_info, "cache_bytes_per_element", 2) or 2)
        fits = max_requests_for_kv_budget(configured, self.max_sequence_length, self._memory().kv_bytes_one_gpu,
                                          self.num_current_layers, self.model_info.num_kv_heads,
                                          self.model_info.head_size_k, self.model_info.head_size_v, elem)
        if fits <= 0:
            raise ValueError(f"node {self.node_id}: the KV budget holds no request ({fits})")
        return fits if configured is None else max(configured, fits)

    @property
    def is_overloaded(self) -> bool:
        return self.current_requests >= self.max_requests

    def get_decoder_layer_capacity(self, include_input_embed: bool = False, include_lm_head: bool = False) -> int:
        """Decoder layers whose parameters fit the parameter share of this node's memory, after setting
        aside the embedding table and / or the lm_head when the node sits at a pipeline end."""
        return self._memory().layers_that_fit(self.model_info, include_input_embed, include_lm_head)

    @property
    def per_decoder_layer_kv_cache_memory(self) -> Optional[int]:
        n = self.num_current_layers
        return math.floor(self._memory().kv_bytes / n) if n else None

    def add_request(self) -> None:
        self.current_requests += 1

    def remove_request(self) -> None:
        self.current_requests -= 1

    # ------------------------------------------------------------------ speed
    def set_layer_latency_ms(self, latency_ms: float) -> None:
        self.avg_layer_latency_ms = latency_ms

    def _quantization_speedup(self) -> float:
        """16-bit weights are the baseline; narrower weights scale the peak by 2 / bytes, of which
        about 80 % is reached in practice. Never below a tenth of the baseline."""
        width = float(self.model_info.param_bytes_per_element)
        if width <= 0:
            return 1.0
        gain = 2.0 / width
        if width < 2.0:
            gain *= 0.8
        return max(gain, 0.1)

    def roofline_layer_latency_ms(self) -> float:
        model = RooflinePerformanceModel(self.hardware, self.model_info, self._quantization_speedup(),
                                         batch_size=self.current_requests, target_seq_len=1,
                                         source_seq_len=self.max_sequence_length)
        return model.roofline_layer_latency_ms(include_input_embed=self.has_embedding, include_lm_head=self.has_lm_head,
                                               num_current_layers=self.num_current_layers)

    @property
    def layer_latency_ms(self) -> float:
        """What the router charges per layer on this node: infinite when full, the roofline estimate
        until a measurement arrived, then the measurement plus a term that grows with the load."""
        if self.is_overloaded:
            return math.inf
        measured = self.avg_layer_latency_ms
        if measured is None:
            return self.roofline_layer_latency_ms()
        load = self.current_requests / self.max_requests
        return measured + load * self.load_compensator

    # ------------------------------------------------------------------ network
    def update_rtt(self, target_node_id: str, rtt_ms: float) -> None:
        self.rtt_to_nodes[target_node_id] = rtt_ms

    def get_rtt_to(self, other: "Node") -> float:
        """Round-trip time to ``other`` in ms: zero to itself, else what either side has measured
        (this node's figure first), else infinity."""
        if other is self or other.node_id == self.node_id:
            return 0.0
        for table, key in ((self.rtt_to_nodes, other.node_id), (other.rtt_to_nodes, self.node_id)):
            if table is not None and key in table:
                return table[key]
        return math.inf
