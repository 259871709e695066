"""Resolve a model name to local files, downloading only what a stage needs.

``selective_model_download`` fetches metadata first (config, tokenizer, safetensors index) and
then only the weight shards that contain tensors of ``[start_layer, end_layer)`` - the
behaviour of ``src/parallax/utils/model_download.py:79-228``. ``USE_MODELSCOPE=1`` switches the
hub. A path that exists on disk is used as is (this is the only mode that works offline).
"""

from __future__ import annotations

import json
import logging
import os
from pathlib import Path
from typing import Optional

from parallax_b200.loader.filter import normalize_weight_key, should_include_weight_key

logger = logging.getLogger(__name__)

METADATA_PATTERNS = ["*.json", "*.txt", "*.model", "*.jinja", "tokenizer*", "*.tiktoken"]


def use_modelscope() -> bool:
    return os.environ.get("USE_MODELSCOPE", "").lower() in ("1", "true", "yes")


def load_config_only(model: str, local_files_only: bool = False) -> dict:
    """config.json of a local directory or of a hub repo (normalised for VLM text towers)."""
    from parallax_b200.models.config import normalize_hf_config

    p = Path(model)
    if p.is_dir():
        return normalize_hf_config(json.loads((p / "config.json").read_text()))
    from huggingface_hub import hf_hub_download

    f = hf_hub_download(repo_id=model, filename="config.json", local_files_only=local_files_only)
    return normalize_hf_config(json.loads(Path(f).read_text()))


def needed_weight_files(index: dict, start_layer: int, end_layer: int, num_layers: int,
                        tie_word_embeddings: bool) -> list[str]:
    first, last = start_layer == 0, end_layer == num_layers
    files = []
    for key, fname in (index.get("weight_map") or {}).items():
        if fname in files:
            continue
        if should_include_weight_key(normalize_weight_key(key), start_layer, end_layer, first, last,
                                     tie_word_embeddings):
            files.append(fname)
    return files


def _snapshot(repo: str, patterns: list[str], local_files_only: bool) -> Path:
    if use_modelscope():
        from modelscope import snapshot_download as ms_download

        return Path(ms_download(repo, allow_patterns=patterns, local_files_only=local_files_only))
    from huggingface_hub import snapshot_download

    return Path(snapshot_download(repo_id=repo, allow_patterns=patterns, local_files_only=local_files_only))


def selective_model_download(model: str, start_layer: Optional[int] = None, end_layer: Optional[int] = None,
                             local_files_only: bool = False) -> Path:
    p = Path(model)
    if p.is_dir():
        return p
    root = _snapshot(model, METADATA_PATTERNS, local_files_only)
    cfg = json.loads((root / "config.json").read_text())
    n = int((cfg.get("text_config") or cfg).get("num_hidden_layers", 0))
    index_file = root / "model.safetensors.index.json"
    if start_layer is None or end_layer is None or not index_file.exists():
        return _snapshot(model, METADATA_PATTERNS + ["*.safetensors"], local_files_only)
    files = needed_weight_files(json.loads(index_file.read_text()), start_layer, end_layer, n,
                                bool(cfg.get("tie_word_embeddings", False)))
    logger.info("stage [%s, %s): downloading %d weight file(s)", start_layer, end_layer, len(files))
    return _snapshot(model, METADATA_PATTERNS + files, local_files_only)
