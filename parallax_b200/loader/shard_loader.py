"""Checkpoint loading for one pipeline stage.

The checkpoint format is plain HuggingFace: ``config.json``, ``model.safetensors`` or sharded
``model-0000X-of-0000Y.safetensors`` with ``model.safetensors.index.json``. A stage opens only
the files that hold tensors of its layer range and reads only the matching keys, as the
reference's loader does (``src/parallax/server/shard_loader.py:359-471``). Also here: fusing
LoRA adapters into the base weights at load time (``:114-226``) and reloading weights from a
refit directory (``:557-653``).
"""

from __future__ import annotations

import json
import logging
import re
from pathlib import Path
from typing import Iterable, Optional

import torch

from parallax_b200.loader.filter import (filter_weight_files, normalize_weight_key,
                                         should_include_weight_key)
from parallax_b200.models.config import ModelConfig, config_from_hf
from parallax_b200.models.registry import family_of, supported_architectures

logger = logging.getLogger(__name__)

_INT_DTYPES = {torch.int8, torch.uint8, torch.int32, torch.int64, torch.float8_e4m3fn, torch.float8_e5m2}


class ShardLoader:
    def __init__(self, model_path: str, start_layer: Optional[int] = None, end_layer: Optional[int] = None,
                 use_hfcache: bool = False):
        from parallax_b200.utils.model_download import selective_model_download

        self.model_path = Path(selective_model_download(model_path, start_layer, end_layer, use_hfcache))
        self.hf_config = json.loads((self.model_path / "config.json").read_text())
        self.config: ModelConfig = config_from_hf(self.hf_config)
        family_of(self.config.architecture)  # raises for unsupported architectures
        n = self.config.num_hidden_layers
        self.start_layer = 0 if start_layer is None else start_layer
        self.end_layer = n if end_layer is None else end_layer
        if not (0 <= self.start_layer < self.end_layer <= n):
            raise ValueError(f"invalid layer range [{self.start_layer}, {self.end_layer}) for {n} layers")

    @property
    def is_first(self) -> bool:
        return self.start_layer == 0

    @property
    def is_last(self) -> bool:
        return self.end_layer == self.config.num_hidden_layers

    def weight_files(self) -> list[str]:
        files = sorted(str(p) for p in self.model_path.glob("*.safetensors")
                       if not p.name.startswith("adapter_"))
        if not files:
            raise FileNotFoundError(f"no safetensors files under {self.model_path}")
        return filter_weight_files(self.model_path, files, self.start_layer, self.end_layer,
                                   self.is_first, self.is_last, self.hf_config)

    def wanted(self, key: str) -> bool:
        return should_include_weight_key(normalize_weight_key(key), self.start_layer, self.end_layer,
                                         self.is_first, self.is_last, self.config.tie_word_embeddings)

    def load_weights(self, device="cpu", dtype: Optional[torch.dtype] = None) -> dict[str, torch.Tensor]:
        """HF-named tensors of this stage. Floating tensors are cast to ``dtype``; packed
        quantised payloads (int / fp8) and their scales keep their storage type."""
        from safetensors import safe_open

        out: dict[str, torch.Tensor] = {}
        for f in self.weight_files():
            with safe_open(f, framework="pt", device=str(device)) as sf:
                for key in sf.keys():
                    if not self.wanted(key):
                        continue
                    t = sf.get_tensor(key)
                    if dtype is not None and t.dtype not in _INT_DTYPES and t.is_floating_point() \
                            and not key.endswith("_scale_inv"):
                        t = t.to(dtype)
                    out[normalize_weight_key(key)] = t
        q = (self.hf_config or {}).get("quantization")
        if isinstance(q, dict) and "bits" in q:
            from parallax_b200.loader.quant import expand_affine_quantized

            n = expand_affine_quantized(out, q, dtype or torch.bfloat16)
            logger.info("expanded %d affine group-quantised layers (per-module overrides honoured)", n)
        logger.info("stage [%d, %d): loaded %d tensors from %s", self.start_layer, self.end_layer,
                    len(out), self.model_path)
        return out

    def build_worker(self, device, dtype=None, lora_paths: Optional[Iterable[str]] = None, **worker_kw):
        """Load this stage's weights and build the :class:`StageWorker` that serves them."""
        from parallax_b200.engine.worker import StageWorker

        dev = torch.device(device)
        dt = dtype or (torch.bfloat16 if dev.type == "cuda" else torch.float32)
        weights = self.load_weights("cpu", None)
        for lp in lora_paths or []:
            apply_lora_adapter(weights, lp)
        return StageWorker(self.config, self.start_layer, self.end_layer, dev, dt, weights=weights, **worker_kw)


# --------------------------------------------------------------------------- LoRA
_LORA_RE = re.compile(r"^(?:base_model\.model\.)?(.*)\.lora_([AB])(?:\.default)?\.weight$")


def apply_lora_adapter(weights: dict[str, torch.Tensor], adapter_path: str, scale: Optional[float] = None) -> int:
    """Fuse a PEFT LoRA adapter into ``weights`` in place: ``W += (alpha / r) * B @ A``.
    DoRA magnitude vectors (``lora_magnitude_vector``) rescale the fused rows. Returns the
    number of matrices updated; tensors of other stages are ignored."""
    from safetensors.torch import load_file

    p = Path(adapter_path)
    cfg = json.loads((p / "adapter_config.json").read_text()) if (p / "adapter_config.json").exists() else {}
    r = cfg.get("r") or cfg.get("lora_rank") or 8
    alpha = cfg.get("lora_alpha", r)
    s = scale if scale is not None else alpha / r
    f = p / "adapter_model.safetensors" if p.is_dir() else p
    tensors = load_file(str(f))
    pairs: dict[str, dict[str, torch.Tensor]] = {}
    mags: dict[str, torch.Tensor] = {}
    for k, v in tensors.items():
        m = _LORA_RE.match(k)
        if m:
            pairs.setdefault(normalize_weight_key(m.group(1)), {})[m.group(2)] = v
        elif "lora_magnitude_vector" in k:
            base = k.split(".lora_magnitude_vector")[0].replace("base_model.model.", "")
            mags[normalize_weight_key(base)] = v
    n = 0
    for base, ab in pairs.items():
        key = base + ".weight"
        if key not in weights or "A" not in ab or "B" not in ab:
            continue
        w = weights[key].float()
        w = w + s * (ab["B"].float() @ ab["A"].float())
        if base in mags:
            w = w * (mags[base].float().flatten() / w.norm(dim=1).clamp_min(1e-12))[:, None]
        weights[key] = w.to(weights[key].dtype)
        n += 1
    return n


def supported() -> list[str]:
    return supported_architectures()
