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


# ------------------------------------------------------------------------------------ mxfp4
# GPT-OSS checkpoints store the expert matrices as MXFP4: groups of 32 values along the input
# dimension share one power-of-two scale (e8m0, bias 127) and each value is a 4-bit e2m1 float,
# two per byte with the low nibble first (``<name>_blocks`` uint8 [..., rows, K/32, 16] and
# ``<name>_scales`` uint8 [..., rows, K/32]). The reference passes these checkpoints to its
# backends untouched (``src/parallax/sglang/model_runner.py:358-366``); here they are expanded
# to bf16 when the shard is loaded.
_FP4_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0)


def dequant_mxfp4(blocks: torch.Tensor, scales: torch.Tensor, dtype: torch.dtype = torch.bfloat16,
                  rows_per_chunk: int = 1 << 16) -> torch.Tensor:
    """``blocks [..., rows, G, 16]`` + ``scales [..., rows, G]`` -> ``[..., rows, G * 32]``."""
    assert blocks.dtype == torch.uint8 and scales.dtype == torch.uint8
    assert blocks.shape[:-1] == scales.shape, (blocks.shape, scales.shape)
    *prefix, G, B = blocks.shape
    lut = torch.tensor(_FP4_VALUES, dtype=torch.float32, device=blocks.device)
    flat_b = blocks.reshape(-1, B)
    flat_s = scales.reshape(-1, 1).to(torch.int32) - 127
    out = torch.empty((flat_b.shape[0], 2 * B), dtype=dtype, device=blocks.device)
    for r0 in range(0, flat_b.shape[0], rows_per_chunk):      # bounded temporaries for 100-GB checkpoints
        blk = flat_b[r0:r0 + rows_per_chunk]
        sub = torch.empty((blk.shape[0], 2 * B), dtype=torch.float32, device=blocks.device)
        sub[:, 0::2] = lut[(blk & 0x0F).long()]
        sub[:, 1::2] = lut[(blk >> 4).long()]
        out[r0:r0 + rows_per_chunk] = torch.ldexp(sub, flat_s[r0:r0 + rows_per_chunk]).to(dtype)
    return out.view(*prefix, G * 2 * B)


def quantize_mxfp4(w: torch.Tensor):
    """Inverse of :func:`dequant_mxfp4` (round to nearest): ``w [..., rows, K]`` with K % 32 == 0 ->
    (``blocks`` uint8 ``[..., rows, K/32, 16]``, ``scales`` uint8 ``[..., rows, K/32]``)."""
    *prefix, K = w.shape
    assert K % 32 == 0
    g = w.float().reshape(-1, K // 32, 32)
    amax = g.abs().amax(dim=-1).clamp_min(2.0 ** -126)
    # the largest e2m1 magnitude is 6 = 1.5 * 2^2: pick the scale that maps the group maximum below 8
    exp = torch.ceil(torch.log2(amax / 6.0)).clamp(-127, 127)
    scaled = g / torch.exp2(exp)[..., None]
    mags = torch.tensor(_FP4_VALUES[:8], dtype=torch.float32, device=w.device)
    idx = (scaled.abs()[..., None] - mags).abs().argmin(dim=-1)
    idx = idx + 8 * (scaled < 0)
    idx = idx.to(torch.uint8)
    blocks = (idx[..., 0::2] | (idx[..., 1::2] << 4)).reshape(*prefix, K // 32, 16)
    scales = (exp + 127).to(torch.uint8).reshape(*prefix, K // 32)
    return blocks.contiguous(), scales.contiguous()


# ------------------------------------------------------------------------- affine group quantisation
# Checkpoints converted for MLX store a quantised linear layer as three tensors: ``<name>.weight`` (uint32,
# ``32 / bits`` values per word, the first value in the lowest bits), ``<name>.scales`` and ``<name>.biases``
# (one pair per group of ``group_size`` inputs): ``w = q * scale + bias``. ``config.json`` carries
# ``"quantization": {"group_size": g, "bits": b, "<module path>": {"group_size": ..., "bits": ...} | false}``
# with per-module overrides. The reference rebuilds quantised MLX modules from these
# (``src/parallax/server/shard_loader.py:495-537,610-643``); this engine serves bf16 / fp8 on B200, so the
# layers are expanded to floating point when the shard is loaded.
def quantize_affine(w: torch.Tensor, bits: int = 4, group_size: int = 64):
    """``w [out, in]`` -> ``(packed uint32 as int32 [out, in * bits / 32], scales, biases [out, in / group])``."""
    if 32 % bits:
        raise ValueError("bits must divide 32 (2, 4 or 8)")
    out_f, in_f = w.shape
    g = w.float().view(out_f, in_f // group_size, group_size)
    lo, hi = g.amin(-1, keepdim=True), g.amax(-1, keepdim=True)
    levels = (1 << bits) - 1
    scale = ((hi - lo) / levels).clamp_min(1e-8)
    q = ((g - lo) / scale).round().clamp_(0, levels).to(torch.int64).view(out_f, in_f)
    per = 32 // bits
    shifts = (torch.arange(per, dtype=torch.int64) * bits)
    words = (q.view(out_f, in_f // per, per) << shifts).sum(-1)
    words = torch.where(words >= 2 ** 31, words - 2 ** 32, words).to(torch.int32)     # torch has no uint32 math
    return words, scale.squeeze(-1).to(torch.float16), lo.squeeze(-1).to(torch.float16)


def dequant_affine(words: torch.Tensor, scales: torch.Tensor, biases: torch.Tensor, bits: int, group_size: int,
                   dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """Expand an affine group-quantised weight (see above) to ``[out, in]`` in ``dtype``."""
    if 32 % bits:
        raise ValueError(f"{bits}-bit affine quantisation is packed across word boundaries; supported: 2, 4, 8")
    per = 32 // bits
    w64 = words.to(torch.int64) & 0xFFFFFFFF
    shifts = (torch.arange(per, dtype=torch.int64, device=words.device) * bits)
    q = ((w64.unsqueeze(-1) >> shifts) & ((1 << bits) - 1)).reshape(words.shape[0], -1).float()
    out_f, in_f = q.shape
    if scales.shape != (out_f, in_f // group_size):
        raise ValueError(f"scales {tuple(scales.shape)} do not fit a [{out_f}, {in_f}] weight in groups of {group_size}")
    g = q.view(out_f, in_f // group_size, group_size)
    return (g * scales.float().unsqueeze(-1) + biases.float().unsqueeze(-1)).view(out_f, in_f).to(dtype)


def expand_affine_quantized(tensors: dict, quantization: Optional[dict], dtype: torch.dtype = torch.bfloat16) -> int:
    """In place: every ``<module>.weight`` that comes with ``.scales`` / ``.biases`` is replaced by its floating
    expansion and the two side tensors are dropped. Per-module entries of ``quantization`` override the global
    ``bits`` / ``group_size`` (a module path may be given with or without the ``model.`` / ``language_model.``
    prefixes a converter added); ``false`` marks a module that was left unquantised. Returns the number of
    layers expanded."""
    if not quantization or "bits" not in quantization:
        return 0
    n = 0
    for key in [k for k in tensors if k.endswith(".scales")]:
        mod = key[: -len(".scales")]
        wkey, bkey = mod + ".weight", mod + ".biases"
        if wkey not in tensors or bkey not in tensors:
            continue
        spec = None
        for cand in (mod, "model." + mod, "language_model." + mod, mod.removeprefix("model."),
                     mod.removeprefix("language_model.")):
            if cand in quantization:
                spec = quantization[cand]
                break
        if spec is False:
            continue
        spec = spec if isinstance(spec, dict) else {}
        bits = int(spec.get("bits", quantization["bits"]))
        group = int(spec.get("group_size", quantization["group_size"]))
        tensors[wkey] = dequant_affine(tensors[wkey], tensors.pop(key), tensors.pop(bkey), bits, group, dtype)
        n += 1
    return n
