"""Endpoint registry of the multi-cluster router: membership, health, metrics, selection.

Tracks per endpoint: in-flight count, totals, EMA TTFT / TPOT, last error, the readiness
probe result (``GET <endpoint>/cluster/status_json`` with a TTL cache), one hour of
per-second output throughput, and recent request samples. Behavioural counterpart of
``EndpointRegistry`` in ``src/router/main.py:103-615``.
"""

from __future__ import annotations

import asyncio
import time
import uuid
from collections import deque
from dataclasses import asdict, dataclass, field
from typing import Any, Optional

from parallax_b200.router.lb_strategy import (PERFORMANCE_RULES, SUPPORTED_STRATEGIES, PerformanceConfig,
                                              make_strategy)

THROUGHPUT_HISTORY_SEC = 3600
THROUGHPUT_DISPLAY_LAG_SEC = 1
MAX_REQUEST_SAMPLES = 200


class RouterError(Exception):
    def __init__(self, status_code: int, detail: str):
        super().__init__(detail)
        self.status_code, self.detail = status_code, detail


@dataclass
class RouterConfig:
    strategy: str = "round_robin"
    performance: PerformanceConfig = field(default_factory=PerformanceConfig)
    status_check_path: str = "/cluster/status_json"
    status_check_ttl_sec: float = 3.0
    status_check_timeout_sec: float = 3.0


@dataclass
class EndpointMetrics:
    inflight: int = 0
    total_requests: int = 0
    total_errors: int = 0
    last_error_ts: Optional[float] = None
    ema_ttft_ms: Optional[float] = None
    ema_tpot_ms: Optional[float] = None
    last_ttft_ms: Optional[float] = None
    last_tpot_ms: Optional[float] = None
    last_status_ok: Optional[bool] = None
    last_status: Optional[str] = None
    last_status_ts: Optional[float] = None
    last_status_error: Optional[str] = None
    max_running_request: Optional[int] = None
    request_samples: deque = field(default_factory=lambda: deque(maxlen=MAX_REQUEST_SAMPLES))


@dataclass
class Endpoint:
    endpoint_id: str
    base_url: str
    enabled: bool = True
    created_ts: float = field(default_factory=time.time)
    metrics: EndpointMetrics = field(default_factory=EndpointMetrics)


def join_url(base_url: str, path: str) -> str:
    return base_url.rstrip("/") + path


_PROBE_RULES = {
    "status_check_path": (str, lambda v: bool(v.strip()), "status_check_path must be a non-empty string"),
    "status_check_ttl_sec": (float, lambda v: v >= 0, "status_check_ttl_sec must be >= 0"),
    "status_check_timeout_sec": (float, lambda v: v > 0, "status_check_timeout_sec must be > 0"),
}


def _coerce(value: Any, kind, name: str):
    if kind is str:
        if not isinstance(value, str):
            raise ValueError(f"{name} must be a string")
        return value
    if isinstance(value, bool):
        raise ValueError(f"{name} must be a number" if kind is float else f"{name} must be an integer")
    if kind is int:
        if isinstance(value, int) or (isinstance(value, float) and value.is_integer()):
            return int(value)
        raise ValueError(f"{name} must be an integer")
    if isinstance(value, (int, float)):
        return float(value)
    raise ValueError(f"{name} must be a number")


class EndpointRegistry:
    def __init__(self, *, config: Optional[RouterConfig] = None, http_client_factory=None):
        self._lock = asyncio.Lock()
        self._endpoints: dict[str, Endpoint] = {}
        self._config = config or RouterConfig()
        self._strategy = make_strategy(self._config.strategy, performance_cfg=self._config.performance)
        self._buckets: dict[str, deque] = {}
        self._client = None
        self._client_factory = http_client_factory

    # ---- http client
    async def get_client(self):
        if self._client is None:
            if self._client_factory is not None:
                self._client = self._client_factory()
            else:
                import httpx

                self._client = httpx.AsyncClient(timeout=httpx.Timeout(20 * 60))
        return self._client

    async def aclose(self) -> None:
        if self._client is not None:
            await self._client.aclose()
            self._client = None

    # ---- config
    def _config_view(self) -> dict:
        c = self._config
        return {"strategy": c.strategy,
                "prob": {k: getattr(c, k) for k in _PROBE_RULES},
                "config": asdict(c.performance) if c.strategy == "performance" else {}}

    async def get_balancer_config(self) -> dict:
        async with self._lock:
            return {**self._config_view(), "available_strategies": list(SUPPORTED_STRATEGIES)}

    async def set_balancer_config(self, patch: dict) -> dict:
        """Runtime patch: ``strategy``, probe settings (under ``prob``/``common`` or top level)
        and performance-strategy settings (under ``config`` or top level). Validated atomically."""
        async with self._lock:
            c = self._config
            probe = dict(patch.get("prob") or patch.get("common") or {})
            perf = dict(patch.get("config") or {})
            for k in _PROBE_RULES:
                if k in patch:
                    probe[k] = patch[k]
            for k in PERFORMANCE_RULES:
                if k in patch:
                    perf[k] = patch[k]
            strategy = patch.get("strategy", c.strategy)
            if not isinstance(strategy, str):
                raise ValueError("strategy must be a string")
            if strategy not in SUPPORTED_STRATEGIES:
                raise ValueError(f"strategy must be one of: {', '.join(SUPPORTED_STRATEGIES)}")
            new_probe, new_perf = {}, {}
            for k, v in probe.items():
                if k not in _PROBE_RULES:
                    raise ValueError(f"Unknown prob key: {k}")
                kind, ok, msg = _PROBE_RULES[k]
                x = _coerce(v, kind, k)
                if not ok(x):
                    raise ValueError(msg)
                new_probe[k] = x.strip() if kind is str else x
            if perf and strategy != "performance":
                raise ValueError("config is only supported for performance strategy")
            for k, v in perf.items():
                if k not in PERFORMANCE_RULES:
                    raise ValueError(f"Unknown performance config key: {k}")
                kind, ok, msg = PERFORMANCE_RULES[k]
                x = _coerce(v, kind, k)
                if not ok(x):
                    raise ValueError(msg)
                new_perf[k] = x
            c.strategy = strategy
            for k, v in new_probe.items():
                setattr(c, k, v)
            for k, v in new_perf.items():
                setattr(c.performance, k, v)
            self._strategy = make_strategy(c.strategy, performance_cfg=c.performance)
            return {"updated": list(patch.keys()), **self._config_view()}

    # ---- membership
    async def register(self, base_url: str, *, status_ok=None, status_val=None, max_running_request=None,
                       status_error=None, status_ts=None) -> Endpoint:
        base_url = base_url.strip().rstrip("/")
        if not base_url.startswith(("http://", "https://")):
            raise ValueError("base_url must start with http:// or https://")
        async with self._lock:
            ep = self._endpoints.get(base_url)
            if ep is None:
                ep = Endpoint(endpoint_id=str(uuid.uuid4()), base_url=base_url)
                self._endpoints[base_url] = ep
                self._buckets.setdefault(base_url, deque())
                if status_ok is not None:
                    ep.metrics.max_running_request = max_running_request
            ep.enabled = True
            if status_ok is not None:
                m = ep.metrics
                m.last_status_ok, m.last_status, m.last_status_error = status_ok, status_val, status_error
                m.last_status_ts = time.time() if status_ts is None else status_ts
            return ep

    async def unregister(self, *, base_url: str) -> int:
        base_url = base_url.strip().rstrip("/")
        async with self._lock:
            self._buckets.pop(base_url, None)
            return 1 if self._endpoints.pop(base_url, None) is not None else 0

    async def set_endpoint_enabled(self, *, base_url: str, enabled: bool) -> Endpoint:
        base_url = base_url.strip().rstrip("/")
        async with self._lock:
            ep = self._endpoints.get(base_url)
            if ep is None:
                raise KeyError("Endpoint not found")
            ep.enabled = bool(enabled)
            return ep

    async def snapshot(self) -> list[Endpoint]:
        async with self._lock:
            return list(self._endpoints.values())

    # ---- health
    async def probe_endpoint_status(self, base_url: str):
        """(ok, status, max_running_request, error) from the endpoint's status document."""
        c = self._config
        try:
            client = await self.get_client()
            resp = await client.get(join_url(base_url, c.status_check_path), timeout=c.status_check_timeout_sec)
            if resp.status_code != 200:
                return False, None, 0, f"Non-200 status: {resp.status_code}"
            data = resp.json()
            inner = data.get("data", {}) if isinstance(data, dict) else {}
            status = inner.get("status")
            if status != "available":
                return False, status, 0, f"Not available: {status}"
            return True, status, inner.get("max_running_request"), None
        except Exception as e:
            return False, None, 0, str(e)

    async def _refresh_one(self, ep: Endpoint, now: float) -> None:
        last = ep.metrics.last_status_ts
        if last is not None and now - last < self._config.status_check_ttl_sec:
            return
        ok, status, maxr, err = await self.probe_endpoint_status(ep.base_url)
        async with self._lock:
            cur = self._endpoints.get(ep.base_url)
            if cur is None:
                return
            m = cur.metrics
            m.last_status_ok, m.last_status, m.max_running_request = bool(ok), status, maxr
            m.last_status_ts, m.last_status_error = now, err

    async def refresh_statuses_if_needed(self, endpoints: list[Endpoint]) -> None:
        now = time.time()
        await asyncio.gather(*[self._refresh_one(ep, now) for ep in endpoints])

    async def choose_best(self) -> Endpoint:
        eps = await self.snapshot()
        if not eps:
            raise RouterError(503, "No downstream endpoints registered")
        eps = [e for e in eps if e.enabled]
        if not eps:
            raise RouterError(503, "No enabled downstream endpoints")
        await self.refresh_statuses_if_needed(eps)
        healthy = [e for e in eps if e.metrics.last_status_ok is True]
        unknown = [e for e in eps if e.metrics.last_status_ok is None]
        pool = healthy or unknown
        if not pool:
            raise RouterError(503, "No healthy downstream endpoints")
        try:
            return self._strategy.select(pool)
        except ValueError as e:
            raise RouterError(503, str(e)) from e

    # ---- metrics
    def _ema(self, prev: Optional[float], value: float) -> float:
        a = self._config.performance.ema_alpha
        return value if prev is None else prev * (1 - a) + value * a

    def _record_buckets(self, base_url: str, buckets: dict[int, int]) -> None:
        q = self._buckets.setdefault(base_url, deque())
        for sec in sorted(buckets):
            cnt = int(buckets[sec])
            if cnt <= 0:
                continue
            if q and q[-1][0] == int(sec):
                q[-1] = (int(sec), q[-1][1] + cnt)
            else:
                q.append((int(sec), cnt))
        cutoff = int(time.time() - THROUGHPUT_HISTORY_SEC)
        while q and q[0][0] < cutoff:
            q.popleft()

    def throughput_series_1h(self, base_url: str, *, end_sec: int) -> tuple[int, list[int]]:
        start = int(end_sec) - (THROUGHPUT_HISTORY_SEC - 1)
        series = [0] * THROUGHPUT_HISTORY_SEC
        for s, cnt in self._buckets.get(base_url, ()):
            if start <= s <= end_sec:
                series[s - start] += cnt
        return start, series

    async def mark_start(self, base_url: str) -> None:
        async with self._lock:
            ep = self._endpoints.get(base_url)
            if ep is not None:
                ep.metrics.inflight += 1
                ep.metrics.total_requests += 1

    async def mark_error(self, base_url: str) -> None:
        async with self._lock:
            ep = self._endpoints.get(base_url)
            if ep is not None:
                ep.metrics.total_errors += 1
                ep.metrics.last_error_ts = time.time()

    async def mark_ttft(self, base_url: str, *, ttft_ms: float) -> None:
        async with self._lock:
            ep = self._endpoints.get(base_url)
            if ep is not None:
                ep.metrics.last_ttft_ms = float(ttft_ms)
                ep.metrics.ema_ttft_ms = self._ema(ep.metrics.ema_ttft_ms, float(ttft_ms))

    async def mark_throughput_bucket(self, base_url: str, *, sec: int, count: int) -> None:
        if count <= 0:
            return
        async with self._lock:
            if base_url in self._endpoints:
                self._record_buckets(base_url, {int(sec): int(count)})

    async def mark_finish(self, base_url: str, *, ttft_ms, tpot_ms, output_units, output_buckets,
                          sample_ttft_ms=None, ttft_already_counted: bool = False) -> None:
        async with self._lock:
            ep = self._endpoints.get(base_url)
            if ep is None:
                return
            m = ep.metrics
            m.inflight = max(m.inflight - 1, 0)
            if ttft_ms is not None and not ttft_already_counted:
                m.last_ttft_ms = ttft_ms
                m.ema_ttft_ms = self._ema(m.ema_ttft_ms, ttft_ms)
            if tpot_ms is not None:
                m.last_tpot_ms = tpot_ms
                m.ema_tpot_ms = self._ema(m.ema_tpot_ms, tpot_ms)
            if isinstance(output_units, int) and output_units > 0 and isinstance(output_buckets, dict):
                self._record_buckets(base_url, output_buckets)
            m.request_samples.append({"ts": time.time(), "tpot_ms": tpot_ms, "output_units": output_units,
                                      "ttft_ms": sample_ttft_ms if sample_ttft_ms is not None else ttft_ms})

    async def list_endpoints(self) -> list[dict]:
        eps = await self.snapshot()
        await self.refresh_statuses_if_needed(eps)
        end = int(time.time()) - THROUGHPUT_DISPLAY_LAG_SEC
        out = []
        for ep in eps:
            start, series = self.throughput_series_1h(ep.base_url, end_sec=end)
            metrics = {k: v for k, v in asdict(ep.metrics).items() if k != "request_samples"}
            metrics.update(request_samples=list(ep.metrics.request_samples), throughput_tok_s=float(series[-1]),
                           throughput_series_1h={"start_sec": start, "tok_s": series})
            item: dict[str, Any] = {"endpoint_id": ep.endpoint_id, "base_url": ep.base_url,
                                    "created_ts": ep.created_ts, "enabled": ep.enabled, "metrics": metrics}
            if self._config.strategy == "performance":
                item["score"] = float(self._strategy.score(ep))
            out.append(item)
        return out

    async def broadcast_raw(self, *, path: str, headers: dict, body: bytes) -> list[dict]:
        eps = await self.snapshot()
        if not eps:
            raise RouterError(503, "No downstream endpoints registered")
        client = await self.get_client()

        async def one(ep: Endpoint) -> dict:
            try:
                resp = await client.post(join_url(ep.base_url, path), headers=headers, content=body)
                is_json = "application/json" in resp.headers.get("content-type", "").lower()
                return {"endpoint_id": ep.endpoint_id, "base_url": ep.base_url, "ok": 200 <= resp.status_code < 300,
                        "status_code": resp.status_code, "response": resp.json() if is_json else resp.text}
            except Exception as e:
                return {"endpoint_id": ep.endpoint_id, "base_url": ep.base_url, "ok": False,
                        "status_code": None, "error": str(e)}

        return list(await asyncio.gather(*[one(ep) for ep in eps]))
