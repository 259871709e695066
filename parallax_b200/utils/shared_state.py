"""State shared between the launcher, the control-channel process and the executors of a node.

Holds the current layer allocation, the node status and the metrics that the heartbeat
reports (in-flight requests, EWMA of the per-layer latency). Backed by a
``multiprocessing.Manager().dict()`` when processes share it, or by a plain dict inside one
process. Same keys as ``src/parallax/utils/shared_state.py:14-162``.
"""

from __future__ import annotations

import multiprocessing
import time
from typing import Any, Optional

_DEFAULTS = {
    "block_start_index": None, "block_end_index": None, "model_name": None, "tp_size": None,
    "enable_weight_refit": None, "weight_refit_mode": None, "_layer_allocation_changed": False,
    "status": None,
}


class SharedState:
    def __init__(self, backing=None):
        if backing is None:
            backing = dict(_DEFAULTS)
            backing["metrics"] = {"current_requests": 0, "layer_latency_ms": None, "_last_update_ts": 0.0}
        elif isinstance(backing, SharedState):
            backing = backing._dict
        self._dict = backing

    @classmethod
    def create(cls, in_process: bool = False) -> "SharedState":
        """New state with defaults; ``in_process=True`` avoids the manager process."""
        if in_process:
            return cls()
        mgr = multiprocessing.Manager()
        d = mgr.dict()
        for k, v in _DEFAULTS.items():
            d[k] = v
        m = mgr.dict()
        m["current_requests"] = 0
        m["layer_latency_ms"] = None
        m["_last_update_ts"] = 0.0
        d["metrics"] = m
        st = cls(d)
        st._manager = mgr  # keep the manager process alive as long as the state
        return st

    # dict-like access
    def get(self, key: str, default: Any = None) -> Any:
        return self._dict.get(key, default)

    def set(self, key: str, value: Any) -> None:
        self._dict[key] = value

    def update(self, **kw) -> None:
        for k, v in kw.items():
            self._dict[k] = v

    def __getitem__(self, key: str) -> Any:
        return self._dict[key]

    def __setitem__(self, key: str, value: Any) -> None:
        self._dict[key] = value

    def __contains__(self, key: str) -> bool:
        return key in self._dict

    @property
    def dict(self):
        return self._dict

    # metrics
    def get_metrics(self) -> dict:
        m = self._dict.get("metrics")
        return {k: m[k] for k in m.keys()} if m else {}

    def update_metrics(self, *, current_requests: Optional[int] = None,
                       layer_latency_ms_sample: Optional[float] = None, ewma_alpha: float = 0.2) -> None:
        m = self._dict.get("metrics")
        if m is None:
            raise RuntimeError("metrics not initialized in shared_state")
        if current_requests is not None:
            m["current_requests"] = int(current_requests)
        if layer_latency_ms_sample is not None:
            prev = m.get("layer_latency_ms")
            x = float(layer_latency_ms_sample)
            m["layer_latency_ms"] = x if prev is None else (1.0 - ewma_alpha) * float(prev) + ewma_alpha * x
        m["_last_update_ts"] = time.time()
        if not hasattr(m, "_callmethod"):  # plain dict: write back is implicit; manager dict: already shared
            self._dict["metrics"] = m

    # allocation / status
    def get_model_info(self) -> dict:
        keys = ("model_name", "block_start_index", "block_end_index", "tp_size", "enable_weight_refit",
                "weight_refit_mode")
        d = {k: self._dict.get(k) for k in keys}
        d["_layer_allocation_changed"] = self._dict.get("_layer_allocation_changed", False)
        return d

    def set_layer_allocation(self, model_name, start_layer, end_layer, tp_size=1, changed=True) -> None:
        self.update(model_name=model_name, block_start_index=start_layer, block_end_index=end_layer,
                    tp_size=tp_size, _layer_allocation_changed=changed)

    def get_layer_allocation_changed(self) -> bool:
        return bool(self._dict.get("_layer_allocation_changed", False))

    def get_status(self) -> Optional[str]:
        return self._dict.get("status")

    def set_status(self, status: str) -> None:
        self._dict["status"] = status
