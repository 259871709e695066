"""Hardware description reported by a node when it joins a cluster.

Peak fp16/bf16 TFLOP/s and memory bandwidth come from a table keyed by the CUDA device name
(the reference's table, ``src/parallax/server/server_info.py:122-144``, stops at Ampere/Ada and
falls back to 50 TFLOP/s / 600 GB/s for anything else; entries for Hopper and Blackwell are
added here, and on a B200 box the measured peaks file is preferred when present).
"""

from __future__ import annotations

import json
import os
from dataclasses import asdict, dataclass
from typing import Optional

try:
    import torch
except Exception:  # pragma: no cover
    torch = None

# substring of the lower-cased device name -> (dense fp16/bf16 TFLOP/s, memory GB/s)
GPU_DB: dict[str, tuple[float, float]] = {
    "b200": (2250.0, 7700.0),
    "gb200": (2500.0, 8000.0),
    "b100": (1800.0, 8000.0),
    "h200": (989.0, 4800.0),
    "h100": (989.0, 3350.0),
    "h20": (148.0, 4000.0),
    "a100-80g": (312.0, 2039.0),
    "a100 80": (312.0, 2039.0),
    "a100-40g": (312.0, 1935.0),
    "a100 40": (312.0, 1935.0),
    "l40s": (362.0, 864.0),
    "rtx 5090": (104.8, 1792.0),
    "rtx 4090": (82.6, 1008.0),
}
FALLBACK = (50.0, 600.0)


def match_gpu_specs(name: str, vram_gb: float) -> tuple[float, float]:
    key = name.lower()
    if "a100" in key:
        return GPU_DB["a100-80g"] if ("80" in key or vram_gb >= 60) else GPU_DB["a100-40g"]
    for sub, spec in GPU_DB.items():
        if sub in key:
            return spec
    return FALLBACK


@dataclass
class HardwareInfo:
    num_gpus: int
    gpu_name: str
    tflops_fp16: float
    memory_gb: float
    memory_bandwidth_gbps: float
    device: str = "cuda"

    def dumps(self) -> dict:
        return asdict(self)

    @classmethod
    def detect(cls, measured_peaks_path: Optional[str] = None) -> "HardwareInfo":
        if torch is None or not torch.cuda.is_available():
            import psutil

            return cls(num_gpus=0, gpu_name="cpu", tflops_fp16=1.0,
                       memory_gb=round(psutil.virtual_memory().total / 2 ** 30, 1),
                       memory_bandwidth_gbps=50.0, device="cpu")
        props = torch.cuda.get_device_properties(0)
        vram = props.total_memory / 2 ** 30
        tf, bw = match_gpu_specs(props.name, vram)
        if measured_peaks_path and os.path.exists(measured_peaks_path):
            try:
                m = json.load(open(measured_peaks_path))
                tf, bw = float(m.get("bf16_tflops", tf)), float(m.get("hbm_gbs", bw))
            except (OSError, ValueError):
                pass
        return cls(num_gpus=torch.cuda.device_count(), gpu_name=props.name, tflops_fp16=tf,
                   memory_gb=round(vram, 1), memory_bandwidth_gbps=bw, device="cuda")
