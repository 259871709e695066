"""Stage worker: one pipeline stage's model + paged KV tensors on one device."""

from __future__ import annotations

import logging
from typing import Optional

import torch

from parallax_b200.cache.kv_pool import KVPool, bytes_per_block
from parallax_b200.engine.batch import ForwardBatch
from parallax_b200.models.config import ModelConfig
from parallax_b200.models.registry import build_stage
from parallax_b200.utils.trace import nvtx_enabled, nvtx_range

logger = logging.getLogger(__name__)


def plan_kv_blocks(cfg: ModelConfig, start: int, end: int, page_size: int, device: torch.device,
                   fraction: float, dtype: torch.dtype, tp: int = 1,
                   max_tokens: Optional[int] = None, cpu_default_blocks: int = 256,
                   kv_cache_dtype: Optional[str] = None) -> int:
    """KV blocks for a stage: ``fraction`` of the memory left after the weights are loaded."""
    from parallax_b200.cache.kv_pool import kv_cache_torch_dtype

    kv_elem = torch.empty(0, dtype=kv_cache_torch_dtype(kv_cache_dtype, dtype)).element_size()
    per_block = bytes_per_block(cfg, start, end, page_size, torch.empty(0, dtype=dtype).element_size(), tp, kv_elem)
    if per_block == 0:
        return 0
    if device.type != "cuda":
        n = cpu_default_blocks
    else:
        free, _total = torch.cuda.mem_get_info(device)
        n = int(free * fraction) // per_block
    if max_tokens is not None:
        n = min(n, (max_tokens + page_size - 1) // page_size)
    return max(int(n), 1)


class StageWorker:
    def __init__(self, cfg: ModelConfig, start_layer: int, end_layer: int, device, dtype=None,
                 page_size: int = 16, num_blocks: Optional[int] = None, kv_fraction: float = 0.8,
                 max_kv_tokens: Optional[int] = None, seed: int = 0, weights: Optional[dict] = None,
                 max_positions: Optional[int] = None, tp_rank: int = 0, tp_size: int = 1,
                 tp_group=None, num_linear_slots: int = 0, comm=None, ep_rank: int = 0, ep_size: int = 1,
                 ep_comm=None, ep_local_init: bool = False, kv_cache_dtype: Optional[str] = None,
                 kv_scale: tuple = (1.0, 1.0)):
        self.cfg = cfg
        self.device = torch.device(device)
        self.dtype = dtype or (torch.bfloat16 if self.device.type == "cuda" else torch.float32)
        self.start_layer, self.end_layer = start_layer, end_layer
        self.page_size = page_size
        self.model = build_stage(cfg, start_layer, end_layer, self.device, self.dtype,
                                 max_positions=max_positions, tp_rank=tp_rank, tp_size=tp_size,
                                 tp_group=tp_group, comm=comm, ep_rank=ep_rank, ep_size=ep_size, ep_comm=ep_comm,
                                 ep_local_init=ep_local_init)
        if weights is not None:
            self.model.load_weights(weights)
        else:
            self.model.init_random(seed)
        if num_blocks is None:
            num_blocks = plan_kv_blocks(cfg, start_layer, end_layer, page_size, self.device,
                                        kv_fraction, self.dtype, tp_size, max_kv_tokens,
                                        kv_cache_dtype=kv_cache_dtype)
        self.num_blocks = num_blocks
        self.pool = KVPool(cfg, start_layer, end_layer, num_blocks, page_size, self.device, self.dtype,
                           tp=tp_size, num_linear_slots=num_linear_slots, kv_cache_dtype=kv_cache_dtype,
                           kv_scale=kv_scale)
        self.model.attach_kv(self.pool.layers)
        logger.info("stage [%d,%d) on %s: %.2f GB weights, %d KV blocks (%.2f GB)", start_layer,
                    end_layer, self.device, self.model.weight_bytes() / 1e9, num_blocks,
                    self.pool.nbytes() / 1e9)

    @property
    def is_first(self) -> bool:
        return self.model.is_first

    @property
    def is_last(self) -> bool:
        return self.model.is_last

    @torch.inference_mode()
    def run(self, fb: ForwardBatch, hidden: Optional[torch.Tensor] = None) -> torch.Tensor:
        if nvtx_enabled():
            m = self.model
            with nvtx_range(f"stage [{m.start_layer},{m.end_layer}) T={fb.num_tokens}"):
                return m.forward(fb, hidden)
        return self.model.forward(fb, hidden)
