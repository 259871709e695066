"""Which checkpoint tensors (and files) a pipeline stage needs.

A stage that owns decoder layers ``[start, end)`` needs: the embedding table if it is the
first stage; the final norm and lm_head if it is the last stage (plus the embedding table
when embeddings are tied); and every ``layers.N.*`` tensor with ``start <= N < end``. VLM
checkpoints nest the text tower under ``language_model.``; those keys are mapped to the
text-only layout first. Same selection rule as
``src/parallax/utils/weight_filter_utils.py:11-118``.
"""

from __future__ import annotations

import json
import re
from pathlib import Path
from typing import Iterable, Optional

_LM_PREFIXES = ("model.language_model.", "language_model.")
_LAYER_RE = re.compile(r"(?:^|\.)layers\.(\d+)\.")


def normalize_weight_key(key: str) -> str:
    for prefix in _LM_PREFIXES:
        if key.startswith(prefix):
            rest = key[len(prefix):]
            if rest.startswith("model.lm_head."):
                return rest[len("model."):]
            if rest.startswith("model.") or rest.startswith("lm_head."):
                return rest
            return "model." + rest
    return key


def layer_index_of(key: str) -> Optional[int]:
    m = _LAYER_RE.search(key)
    return int(m.group(1)) if m else None


def should_include_weight_key(key: str, start_layer: int, end_layer: int, is_first_shard: bool,
                              is_last_shard: bool, tie_word_embeddings: bool = False) -> bool:
    if key.startswith("model.") and "embed_tokens" in key:
        if is_first_shard:
            return True
        if is_last_shard and tie_word_embeddings and key.startswith("model.embed_tokens"):
            return True
        return False
    if is_last_shard and ("model.norm" in key or "lm_head" in key):
        return True
    idx = layer_index_of(key)
    if idx is not None:
        return start_layer <= idx < end_layer
    return False


def filter_weights_for_range(tensors: dict, start_layer: int, end_layer: int, num_layers: int,
                             tie_word_embeddings: bool = False) -> dict:
    first, last = start_layer == 0, end_layer == num_layers
    out = {}
    for k, v in tensors.items():
        nk = normalize_weight_key(k)
        if should_include_weight_key(nk, start_layer, end_layer, first, last, tie_word_embeddings):
            out[nk] = v
    return out


def filter_weight_files(model_path, weight_files: Iterable[str], start_layer: int, end_layer: int,
                        is_first_shard: bool, is_last_shard: bool, config: Optional[dict] = None) -> list[str]:
    """Keep only the safetensors files that hold a tensor this stage needs (by the index)."""
    model_path = Path(model_path)
    weight_files = list(weight_files)
    index_file = model_path / "model.safetensors.index.json"
    if not index_file.exists():
        return weight_files
    weight_map = json.loads(index_file.read_text()).get("weight_map") or {}
    if not weight_map:
        return weight_files
    if config is None:
        cfg_file = model_path / "config.json"
        config = json.loads(cfg_file.read_text()) if cfg_file.exists() else {}
    tie = bool(config.get("tie_word_embeddings", False))
    needed = {
        fname for key, fname in weight_map.items()
        if should_include_weight_key(normalize_weight_key(key), start_layer, end_layer,
                                     is_first_shard, is_last_shard, tie)
    }
    if not needed:
        return weight_files
    return [wf for wf in weight_files if Path(wf).name in needed]
