"""Step tracer: host phases and device time of every engine step as a Chrome trace
(``chrome://tracing`` / Perfetto JSON).

The reference has no tracing or profiling hooks (only an EWMA of per-layer latency,
``src/parallax/server/executor/base_executor.py:711-732``). Enabled with ``Engine(..., trace=...)``
or the ``PXL_TRACE=<file>`` environment variable; costs two CUDA events per step.

``PXL_NVTX=1`` additionally wraps every stage forward and engine step in an NVTX range (:func:`nvtx_range`),
so that a timeline tool shows the steps by name; off, the helper is a no-op without any call into CUDA.
"""

from __future__ import annotations

import json
import os
import time
from typing import Optional


_NVTX: Optional[bool] = None


class _NoRange:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


_NO_RANGE = _NoRange()


class _NvtxRange:
    def __init__(self, name: str):
        self.name = name

    def __enter__(self):
        import torch

        torch.cuda.nvtx.range_push(self.name)
        return self

    def __exit__(self, *a):
        import torch

        torch.cuda.nvtx.range_pop()
        return False


def nvtx_enabled() -> bool:
    global _NVTX
    if _NVTX is None:
        on = os.environ.get("PXL_NVTX", "") not in ("", "0")
        if on:
            import torch

            on = torch.cuda.is_available()
        _NVTX = on
    return _NVTX


def nvtx_range(name: str):
    """``with nvtx_range("stage 0 [0,18) T=512"): ...``"""
    return _NvtxRange(name) if nvtx_enabled() else _NO_RANGE


class StepTracer:
    def __init__(self, path: str, pid: int = 0):
        self.path, self.pid = path, pid
        self.events: list[dict] = []
        self._t0 = time.perf_counter()
        self._pending: list = []          # (step, start_event, end_event, host_ts)

    @classmethod
    def from_env(cls, pid: int = 0) -> Optional["StepTracer"]:
        p = os.environ.get("PXL_TRACE")
        return cls(p, pid) if p else None

    def _us(self, t: float) -> float:
        return (t - self._t0) * 1e6

    def span(self, name: str, t_begin: float, t_end: float, tid: str = "host", **args) -> None:
        self.events.append({"name": name, "ph": "X", "pid": self.pid, "tid": tid, "ts": self._us(t_begin),
                            "dur": max((t_end - t_begin) * 1e6, 0.01), "args": args})

    def device_span(self, step: int, start_event, end_event, host_ts: float, **args) -> None:
        """CUDA events of one step; resolved lazily so that tracing never adds a synchronisation."""
        self._pending.append((step, start_event, end_event, host_ts, args))
        self._drain(block=False)

    def _drain(self, block: bool) -> None:
        keep = []
        for step, s, e, ts, args in self._pending:
            if block:
                e.synchronize()
            if e.query():
                self.events.append({"name": f"step {step}", "ph": "X", "pid": self.pid, "tid": "device", "ts": self._us(ts),
                                    "dur": s.elapsed_time(e) * 1e3, "args": args})
            else:
                keep.append((step, s, e, ts, args))
        self._pending = keep

    def save(self) -> None:
        self._drain(block=True)
        with open(self.path, "w") as f:
            json.dump({"traceEvents": self.events, "displayTimeUnit": "ms"}, f)
