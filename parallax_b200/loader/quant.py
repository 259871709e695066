"""Block-scaled fp8 (e4m3) weights: 128x128 weight blocks with one fp32 scale each, the format
of the DeepSeek-V3 family checkpoints (``weight`` in float8_e4m3fn + ``weight_scale_inv``).

The reference hands such checkpoints to its backends with ``quantization=quant_method``
(``src/parallax/sglang/model_runner.py:358-366``) or repacks them for MLX
(``src/parallax/models/minimax_m3.py:920-1016``). Here they are either kept in fp8 for the
block-scaled tcgen05 GEMM or expanded to bf16 at load time.
"""

from __future__ import annotations

from typing import Optional

import torch

FP8_MAX = 448.0


def quantize_fp8_block(w: torch.Tensor, block: tuple[int, int] = (128, 128)):
    """``w [N, K]`` -> (fp8 e4m3 ``[N, K]``, fp32 ``scale_inv [ceil(N/bn), ceil(K/bk)]``) with
    ``w ~= fp8 * scale_inv`` per block."""
    N, K = w.shape
    bn, bk = block
    nb, kb = (N + bn - 1) // bn, (K + bk - 1) // bk
    wp = torch.zeros((nb * bn, kb * bk), dtype=torch.float32, device=w.device)
    wp[:N, :K] = w.float()
    blocks = wp.view(nb, bn, kb, bk)
    amax = blocks.abs().amax(dim=(1, 3)).clamp_min(1e-12)
    scale_inv = amax / FP8_MAX
    q = (blocks / scale_inv[:, None, :, None]).clamp(-FP8_MAX, FP8_MAX)
    q = q.view(nb * bn, kb * bk)[:N, :K].to(torch.float8_e4m3fn)
    return q.contiguous(), scale_inv.contiguous()


def dequant_fp8_block(q: torch.Tensor, scale_inv: torch.Tensor, block: tuple[int, int] = (128, 128),
                      dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    N, K = q.shape
    bn, bk = block
    s = scale_inv.float().repeat_interleave(bn, dim=0)[:N].repeat_interleave(bk, dim=1)[:, :K]
    return (q.float() * s).to(dtype)


def quantize_fp8_rows(x: torch.Tensor, group: int = 128):
    """Activations: one scale per row and ``group`` consecutive columns (1 x 128 groups)."""
    T, K = x.shape
    kg = (K + group - 1) // group
    xp = torch.zeros((T, kg * group), dtype=torch.float32, device=x.device)
    xp[:, :K] = x.float()
    g = xp.view(T, kg, group)
    scale = g.abs().amax(dim=-1).clamp_min(1e-12) / FP8_MAX
    q = (g / scale[..., None]).clamp(-FP8_MAX, FP8_MAX).view(T, kg * group)[:, :K].to(torch.float8_e4m3fn)
    return q.contiguous(), scale.contiguous()


def dequant_if_needed(tensors: dict, name: str, cfg=None, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """Return ``tensors[name]`` expanded to a floating tensor if it is stored block-scaled."""
    t = tensors[name]
    if t.dtype != torch.float8_e4m3fn:
        return t
    scale = tensors.get(name + "_scale_inv")
    if scale is None:
        scale = tensors.get(name.replace(".weight", ".weight_scale_inv"))
    if scale is None:
        return t.to(dtype or torch.bfloat16)
    block = tuple((getattr(cfg, "weight_block_size", None) or [128, 128]))
    return dequant_fp8_block(t, scale, block, dtype or torch.bfloat16)
