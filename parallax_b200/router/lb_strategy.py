"""Load-balancing strategies of the multi-cluster router.

* ``round_robin`` - least normalised load (inflight / max_running_request), ties broken by a
  rotating cursor over the endpoints ordered by URL;
* ``performance`` - lowest score = inflight penalty + EMA TTFT + weight * EMA TPOT + error-rate
  penalty + recent-error penalty; optional top-k randomisation and exploration;
* ``random``.

Scores and defaults follow ``src/router/lb_strategy.py:25-171`` of the reference (cold-start
TTFT 3000 ms, TPOT 50 ms).
"""

from __future__ import annotations

import random
import time
from dataclasses import dataclass
from typing import Literal, Sequence

StrategyName = Literal["round_robin", "performance", "random"]
SUPPORTED_STRATEGIES: tuple[str, ...] = ("round_robin", "performance", "random")


@dataclass
class PerformanceConfig:
    ema_alpha: float = 0.1
    default_ttft_ms: float = 3000.0
    default_tpot_ms: float = 50.0
    inflight_penalty_ms: float = 1000.0
    err_rate_penalty_ms: float = 5000.0
    recent_error_window_sec: float = 30.0
    recent_error_penalty_ms: float = 2000.0
    tpot_weight: float = 1.0
    top_k: int = 1
    explore_ratio: float = 0.0


# (type, predicate, message) per runtime-patchable key
PERFORMANCE_RULES = {
    "ema_alpha": (float, lambda x: 0.0 < x <= 1.0, "ema_alpha must be in (0, 1]"),
    "default_ttft_ms": (float, lambda x: x > 0, "default_ttft_ms must be > 0"),
    "default_tpot_ms": (float, lambda x: x >= 0, "default_tpot_ms must be >= 0"),
    "inflight_penalty_ms": (float, lambda x: x >= 0, "inflight_penalty_ms must be >= 0"),
    "err_rate_penalty_ms": (float, lambda x: x >= 0, "err_rate_penalty_ms must be >= 0"),
    "recent_error_window_sec": (float, lambda x: x >= 0, "recent_error_window_sec must be >= 0"),
    "recent_error_penalty_ms": (float, lambda x: x >= 0, "recent_error_penalty_ms must be >= 0"),
    "tpot_weight": (float, lambda x: x >= 0, "tpot_weight must be >= 0"),
    "top_k": (int, lambda x: x >= 1, "top_k must be >= 1"),
    "explore_ratio": (float, lambda x: 0.0 <= x < 1.0, "explore_ratio must be in [0, 1)"),
}


class PerformanceStrategy:
    name = "performance"

    def __init__(self, cfg: PerformanceConfig):
        self.cfg = cfg

    def score(self, cand) -> float:
        m, c = cand.metrics, self.cfg
        ttft = c.default_ttft_ms if m.ema_ttft_ms is None else float(m.ema_ttft_ms)
        tpot = c.default_tpot_ms if m.ema_tpot_ms is None else float(m.ema_tpot_ms)
        err = (float(m.total_errors) / max(float(m.total_requests), 1.0)) * c.err_rate_penalty_ms
        recent = 0.0
        if m.last_error_ts is not None and time.time() - float(m.last_error_ts) < c.recent_error_window_sec:
            recent = c.recent_error_penalty_ms
        return float(m.inflight) * c.inflight_penalty_ms + ttft + c.tpot_weight * tpot + err + recent

    def select(self, candidates: Sequence):
        if not candidates:
            raise ValueError("No candidates")
        if self.cfg.explore_ratio > 0.0 and random.random() < self.cfg.explore_ratio:
            return random.choice(list(candidates))
        ranked = sorted(candidates, key=self.score)
        k = min(max(int(self.cfg.top_k), 1), len(ranked))
        return ranked[0] if k == 1 else random.choice(ranked[:k])


class RandomStrategy:
    name = "random"

    def select(self, candidates: Sequence):
        if not candidates:
            raise ValueError("No candidates")
        return random.choice(list(candidates))


class RoundRobinStrategy:
    name = "round_robin"

    def __init__(self):
        self._cursor = 0

    def select(self, candidates: Sequence):
        if not candidates:
            raise ValueError("No candidates")
        ordered = sorted(candidates, key=lambda x: getattr(x, "base_url", str(x)))
        n = len(ordered)
        start = self._cursor % n
        best, best_load = start, float("inf")
        for step in range(n):
            i = (start + step) % n
            m = getattr(ordered[i], "metrics", None)
            inflight = int(getattr(m, "inflight", 0)) if m is not None else 0
            cap = getattr(m, "max_running_request", None) if m is not None else None
            load = inflight / (cap if isinstance(cap, int) and cap > 0 else 1)
            if load < best_load:
                best, best_load = i, load
        self._cursor = best + 1
        return ordered[best]


def make_strategy(name: str, *, performance_cfg: PerformanceConfig):
    if name == "performance":
        return PerformanceStrategy(performance_cfg)
    if name == "random":
        return RandomStrategy()
    if name == "round_robin":
        return RoundRobinStrategy()
    raise ValueError(f"Unknown strategy: {name}")
