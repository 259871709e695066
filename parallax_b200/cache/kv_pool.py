"""Device tensors of the paged caches of one pipeline stage.

One cache object per decoder layer, chosen by layer kind (same taxonomy as the reference's
hybrid cache, ``src/parallax/server/cache_manager.py:188-259``):

* ``attention``      K, V            ``[blocks, Hkv, page, D]``
* ``mla_attention``  latent | rope   ``[blocks, 1, page, kv_lora + rope]`` (one tensor)
* ``dsa_attention``  MLA cache + lightning-indexer keys ``[blocks, 1, page, index_dim]``
* ``linear``         conv state ``[slots, conv_dim, k-1]`` + recurrent state
                     ``[slots, Hv, Dv, Dk]`` (per request slot, not paged)

Layouts are chosen for the sm_100a kernels (whole pages of one head are contiguous), not
for compatibility with the reference's Metal layouts.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from parallax_b200.models.config import (ATTENTION, DSA_ATTENTION, LINEAR, MLA_ATTENTION,
                                         MSA_ATTENTION, ModelConfig)


@dataclass
class LayerCache:
    kind: str
    k: Optional[torch.Tensor] = None        # attention K / MLA latent+rope
    v: Optional[torch.Tensor] = None        # attention V
    index_k: Optional[torch.Tensor] = None  # DSA / MSA indexer keys
    conv_state: Optional[torch.Tensor] = None
    rec_state: Optional[torch.Tensor] = None
    # e4m3 K / V caches hold value / scale; the attention kernels multiply by the scale again
    k_scale: float = 1.0
    v_scale: float = 1.0

    @property
    def kv_scale(self) -> tuple:
        return (self.k_scale, self.v_scale)

    def __iter__(self):  # lets attention layers unpack ``k, v = cache``
        yield self.k
        yield self.v


def kv_cache_torch_dtype(name: Optional[str], model_dtype):
    """Storage dtype of the K / V pages for a ``--kv-cache-dtype`` value."""
    if name in (None, "", "auto"):
        return model_dtype
    if name in ("fp8", "fp8_e4m3", "float8_e4m3fn"):
        return torch.float8_e4m3fn
    if name in ("bf16", "bfloat16"):
        return torch.bfloat16
    raise ValueError(f"unknown KV cache dtype {name!r} (auto, bf16, fp8_e4m3)")


def linear_dims(cfg: ModelConfig, tp: int = 1) -> tuple[int, int, int, int, int]:
    """(conv_dim, conv_kernel-1, num_v_heads, v_head_dim, k_head_dim) of a gated-delta layer."""
    hk, hv = cfg.linear_num_key_heads // tp, cfg.linear_num_value_heads // tp
    dk, dv = cfg.linear_key_head_dim, cfg.linear_value_head_dim
    conv_dim = 2 * hk * dk + hv * dv
    return conv_dim, max(cfg.linear_conv_kernel_dim - 1, 0), hv, dv, dk


def bytes_per_block(cfg: ModelConfig, start: int, end: int, page: int, elem: int = 2, tp: int = 1,
                    kv_elem: Optional[int] = None) -> int:
    """``kv_elem``: bytes per element of the K / V pages when they differ from the model's (e4m3: 1)."""
    total = 0
    kv_elem = kv_elem or elem
    for li in range(start, end):
        kind = cfg.layer_kind(li)
        if kind in (ATTENTION, MSA_ATTENTION):
            hkv = max(1, cfg.num_key_value_heads // tp)
            total += 2 * hkv * page * cfg.head_dim * kv_elem
            if kind == MSA_ATTENTION:
                total += page * int(cfg.raw.get("index_head_dim") or 0) * elem
        elif kind in (MLA_ATTENTION, DSA_ATTENTION):
            total += page * (cfg.kv_lora_rank + cfg.qk_rope_head_dim) * elem
            if kind == DSA_ATTENTION:
                total += page * cfg.index_head_dim * elem
    return total


def bytes_per_linear_slot(cfg: ModelConfig, start: int, end: int, elem: int = 2, tp: int = 1) -> int:
    total = 0
    for li in range(start, end):
        if cfg.layer_kind(li) == LINEAR:
            conv_dim, km1, hv, dv, dk = linear_dims(cfg, tp)
            total += conv_dim * km1 * elem + hv * dv * dk * 4
    return total


class KVPool:
    def __init__(self, cfg: ModelConfig, start_layer: int, end_layer: int, num_blocks: int,
                 page_size: int, device, dtype, tp: int = 1, num_linear_slots: int = 0,
                 kv_cache_dtype: Optional[str] = None, kv_scale: tuple = (1.0, 1.0)):
        """``kv_cache_dtype="fp8_e4m3"`` keeps the K / V pages of the softmax-attention layers as e4m3 bytes
        (half the memory and half the bytes a decode step reads); latent, indexer and recurrent caches stay in
        the model's dtype."""
        kv_dt = kv_cache_torch_dtype(kv_cache_dtype, dtype)
        self.kv_cache_dtype = kv_dt
        self.cfg = cfg
        self.num_blocks = num_blocks
        self.page_size = page_size
        self.device = torch.device(device)
        self.dtype = dtype
        self.layers: list[LayerCache] = []
        for li in range(start_layer, end_layer):
            kind = cfg.layer_kind(li)
            lc = LayerCache(kind)
            if kind in (ATTENTION, MSA_ATTENTION):
                hkv = max(1, cfg.num_key_value_heads // tp)
                shape = (num_blocks, hkv, page_size, cfg.head_dim)
                lc.k = torch.zeros(shape, device=self.device, dtype=kv_dt)
                lc.v = torch.zeros(shape, device=self.device, dtype=kv_dt)
                if kv_dt == torch.float8_e4m3fn:
                    lc.k_scale, lc.v_scale = float(kv_scale[0]), float(kv_scale[1])
                if kind == MSA_ATTENTION:
                    lc.index_k = torch.zeros((num_blocks, 1, page_size, int(cfg.raw.get("index_head_dim") or 0)),
                                             device=self.device, dtype=dtype)
            elif kind in (MLA_ATTENTION, DSA_ATTENTION):
                lc.k = torch.zeros((num_blocks, 1, page_size, cfg.kv_lora_rank + cfg.qk_rope_head_dim),
                                   device=self.device, dtype=dtype)
                if kind == DSA_ATTENTION:
                    lc.index_k = torch.zeros((num_blocks, 1, page_size, cfg.index_head_dim),
                                             device=self.device, dtype=dtype)
            elif kind == LINEAR:
                conv_dim, km1, hv, dv, dk = linear_dims(cfg, tp)
                lc.conv_state = torch.zeros((num_linear_slots, conv_dim, km1), device=self.device, dtype=dtype)
                lc.rec_state = torch.zeros((num_linear_slots, hv, dv, dk), device=self.device,
                                           dtype=torch.float32)
            self.layers.append(lc)

    def zero_slot(self, slot: int) -> None:
        for lc in self.layers:
            if lc.kind == LINEAR:
                lc.conv_state[slot].zero_()
                lc.rec_state[slot].zero_()

    def copy_slot(self, dst: int, src: int) -> None:
        for lc in self.layers:
            if lc.kind == LINEAR:
                lc.conv_state[dst].copy_(lc.conv_state[src])
                lc.rec_state[dst].copy_(lc.rec_state[src])

    def nbytes(self) -> int:
        n = 0
        for lc in self.layers:
            for t in (lc.k, lc.v, lc.index_k, lc.conv_state, lc.rec_state):
                if t is not None:
                    n += t.numel() * t.element_size()
        return n


def plan_num_blocks(cfg: ModelConfig, start: int, end: int, page: int, free_bytes: int,
                    fraction: float, elem: int = 2, tp: int = 1, max_tokens: Optional[int] = None,
                    kv_elem: Optional[int] = None) -> int:
    """Number of KV blocks that fit into ``fraction`` of the free device memory."""
    per_block = bytes_per_block(cfg, start, end, page, elem, tp, kv_elem)
    if per_block == 0:
        return 0
    n = int(free_bytes * fraction) // per_block
    if max_tokens is not None:
        n = min(n, (max_tokens + page - 1) // page)
    return max(n, 0)
