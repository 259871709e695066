"""Online weight refit (RL): content-addressed weight blocks -> tensors of one stage.

A refit request names content ids (CIDv1, raw codec, sha2-256, base32) and maps weight names
to them; a node fetches only the blocks of its layer range, verifies each against its CID,
joins tensors that were split into ``<name>.weight_partN`` pieces, and hands the result to the
executor either in memory or as ``adapter_model.safetensors`` on disk. Same data contract as
``src/parallax/utils/weight_refit_utils.py:20-206``.
"""

from __future__ import annotations

import base64
import hashlib
import json
import logging
import os
import re
import struct
from collections import defaultdict
from typing import Optional

import torch

from parallax_b200.loader.filter import should_include_weight_key

logger = logging.getLogger(__name__)

_PART_RE = re.compile(r"^(.*)\.weight_part(\d+)$")
_ST_DTYPES = {"F16": torch.float16, "BF16": torch.bfloat16, "F32": torch.float32, "F64": torch.float64,
              "I8": torch.int8, "I16": torch.int16, "I32": torch.int32, "I64": torch.int64,
              "U8": torch.uint8, "BOOL": torch.bool, "F8_E4M3": torch.float8_e4m3fn,
              "F8_E5M2": torch.float8_e5m2}


def calculate_cid(data: bytes) -> str:
    """CIDv1 / raw / sha2-256 in lower-case base32 with the multibase prefix ``b``."""
    digest = hashlib.sha256(data).digest()
    cid = bytes([0x01, 0x55, 0x12, 0x20]) + digest
    return "b" + base64.b32encode(cid).decode("ascii").lower().rstrip("=")


calculate_cid_manual = calculate_cid


def verify_block(data: bytes, cid: str) -> bool:
    return calculate_cid(data) == cid


def concat_weight_partition(tensors: dict[str, torch.Tensor], save_directory: Optional[str] = None) -> dict:
    """Join ``x.weight_part0..N`` along dim 0 into ``x.weight``; other tensors pass through.
    With ``save_directory`` the result is written to ``adapter_model.safetensors`` there and an
    empty dict is returned."""
    out: dict[str, torch.Tensor] = {}
    parts: dict[str, dict[int, torch.Tensor]] = defaultdict(dict)
    for k, v in tensors.items():
        m = _PART_RE.match(k)
        if m:
            parts[m.group(1)][int(m.group(2))] = v
        else:
            out[k] = v
    for base, d in parts.items():
        idx = sorted(d)
        if idx != list(range(len(idx))):
            raise ValueError(f"missing partitions for {base}: have {idx}")
        out[base + ".weight"] = torch.cat([d[i] for i in idx], dim=0)
    if save_directory is None:
        return out
    from safetensors.torch import save_file

    os.makedirs(save_directory, exist_ok=True)
    save_file({k: v.contiguous() for k, v in out.items()}, os.path.join(save_directory, "adapter_model.safetensors"))
    return {}


def filter_weight_cid_list(start_layer: int, end_layer: int, hidden_layers: int, index_map: dict[str, str]) -> list[str]:
    """CIDs of the blocks that hold a tensor of layers [start, end) (+ embed / norm / head)."""
    first, last = start_layer == 0, end_layer == hidden_layers
    need = {cid for key, cid in index_map.items()
            if should_include_weight_key(key, start_layer, end_layer, first, last, tie_word_embeddings=True)}
    return sorted(need)


def parse_safetensors_from_memory(raw: bytes) -> dict[str, torch.Tensor]:
    """Decode a safetensors blob without touching the filesystem."""
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n].decode("utf-8"))
    header.pop("__metadata__", None)
    body = memoryview(raw)[8 + n:]
    out = {}
    for name, info in header.items():
        dt = _ST_DTYPES[info["dtype"]]
        b, e = info["data_offsets"]
        if e == b:
            out[name] = torch.empty(info["shape"], dtype=dt)
            continue
        storage = torch.frombuffer(bytearray(body[b:e]), dtype=torch.uint8)
        out[name] = storage.view(dt).reshape(info["shape"])
    return out


class RefitVersionStore:
    """Keeps the newest ``keep`` refit versions on disk and drops older ones."""

    def __init__(self, root: str = "/tmp", keep: int = 3):
        self.root, self.keep = root, keep
        self.versions: list[str] = []

    def path_for(self, time_stamp) -> str:
        return os.path.join(self.root, str(time_stamp))

    def add(self, time_stamp) -> list[str]:
        import shutil

        p = self.path_for(time_stamp)
        if p not in self.versions:
            self.versions.append(p)
        dropped = []
        while len(self.versions) > self.keep:
            old = self.versions.pop(0)
            shutil.rmtree(old, ignore_errors=True)
            dropped.append(old)
        return dropped


def apply_refit_to_stage(worker, cfg, refit: dict) -> int:
    """Apply a weight-refit request whose blocks are readable files (``paths``: cid -> file) to one stage worker:
    pick the blocks that hold this stage's layers, check every block against its content id, join partitioned
    tensors and hand them to the stage's own loader. Returns the number of tensors used. Every rank of a
    tensor-parallel node runs this on the same request."""
    need = filter_weight_cid_list(worker.start_layer, worker.end_layer, cfg.num_hidden_layers, refit.get("index_map") or {})
    paths = refit.get("paths") or {}
    tensors = {}
    for cid in need:
        p = paths.get(cid)
        if p is None:
            logger.warning("refit block %s has no source; skipped", cid)
            continue
        with open(p, "rb") as f:
            blob = f.read()
        if not verify_block(blob, cid):
            raise ValueError(f"refit block {cid} failed its content-id check")
        tensors.update(parse_safetensors_from_memory(blob))
    return worker.model.update_weights(concat_weight_partition(tensors))
