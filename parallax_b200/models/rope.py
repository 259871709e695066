"""Rotary-embedding tables (cos | sin per position, fp32) incl. the common scaling rules."""

from __future__ import annotations

import math

import torch

from parallax_b200.models.config import ModelConfig
from parallax_b200.ops import build_cos_sin


def _yarn_find_dim(num_rot: float, dim: int, base: float, max_pos: int) -> float:
    return (dim * math.log(max_pos / (num_rot * 2 * math.pi))) / (2 * math.log(base))


def rope_inv_freq(cfg: ModelConfig) -> tuple[torch.Tensor, float]:
    """Returns (inv_freq [rot_dim/2] float64, attention scaling factor for cos/sin)."""
    rot = cfg.rot_dim
    base = cfg.rope_theta
    inv = 1.0 / (base ** (torch.arange(0, rot, 2, dtype=torch.float64) / rot))
    sc = cfg.rope_scaling or {}
    kind = sc.get("rope_type") or sc.get("type") or "default"
    factor = float(sc.get("factor", 1.0))
    if kind in ("default", None) or not sc:
        return inv, 1.0
    if kind == "linear":
        return inv / factor, 1.0
    if kind == "llama3":
        low = float(sc.get("low_freq_factor", 1.0))
        high = float(sc.get("high_freq_factor", 4.0))
        old = float(sc.get("original_max_position_embeddings", 8192))
        wavelen = 2 * math.pi / inv
        smooth = (old / wavelen - low) / (high - low)
        scaled = torch.where(wavelen > old / low, inv / factor, inv)
        mid = (1 - smooth) * inv / factor + smooth * inv
        is_mid = (wavelen <= old / low) & (wavelen >= old / high)
        return torch.where(is_mid, mid, scaled), 1.0
    if kind == "yarn":
        old = float(sc.get("original_max_position_embeddings", cfg.max_position_embeddings))
        beta_fast = float(sc.get("beta_fast", 32))
        beta_slow = float(sc.get("beta_slow", 1))
        lo, hi = _yarn_find_dim(beta_fast, rot, base, int(old)), _yarn_find_dim(beta_slow, rot, base, int(old))
        if sc.get("truncate", True):
            lo, hi = math.floor(lo), math.ceil(hi)
        lo, hi = max(lo, 0), min(hi, rot - 1)
        ramp = ((torch.arange(rot // 2, dtype=torch.float64) - lo) / max(hi - lo, 1e-3)).clamp(0, 1)
        extrap = 1.0 - ramp
        inv_y = inv / factor * (1 - extrap) + inv * extrap
        mscale = float(sc.get("mscale", 1.0))
        mscale_all = float(sc.get("mscale_all_dim", 0.0))

        def get_mscale(s, m):
            return 1.0 if s <= 1 else 0.1 * m * math.log(s) + 1.0

        if mscale_all:
            att = get_mscale(factor, mscale) / get_mscale(factor, mscale_all)
        else:
            att = sc.get("attention_factor") or get_mscale(factor, 1.0)
        return inv_y, float(att)
    # unknown rule: plain frequencies
    return inv, 1.0


def build_rope_table(cfg: ModelConfig, max_pos: int, device) -> torch.Tensor:
    if cfg.rot_dim <= 0:
        return None
    inv, att = rope_inv_freq(cfg)
    return build_cos_sin(max_pos, cfg.rot_dim, cfg.rope_theta, device=device, inv_freq=inv,
                         attention_factor=att)
