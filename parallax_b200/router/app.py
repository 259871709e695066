"""HTTP load-balancing router in front of several clusters.

``/register /unregister /endpoints /endpoint/enabled /balancer/config /v1/chat/completions
/weight/refit /health`` and a small HTML dashboard at ``/`` - the API of
``src/router/main.py:781-1044``. Chat completions are proxied to the endpoint the active
strategy picks; streamed responses are passed through byte for byte while their SSE ``data:``
lines are counted to measure TTFT, TPOT and per-second throughput.

    python -m parallax_b200.router.app --port 8081
"""

from __future__ import annotations

import argparse
import time
from contextlib import asynccontextmanager
from typing import Any, AsyncIterator, Optional

from fastapi import FastAPI, HTTPException
from fastapi import Request as HttpRequest
from fastapi.middleware.cors import CORSMiddleware
from fastapi.responses import HTMLResponse, JSONResponse, StreamingResponse

from parallax_b200.router.registry import Endpoint, EndpointRegistry, RouterConfig, RouterError, join_url

_FORWARDED = {"authorization", "content-type", "accept", "user-agent", "x-request-id"}
APIS = ["/health", "/balancer/config", "/endpoint/enabled", "/register", "/unregister", "/endpoints",
        "/v1/chat/completions", "/weight/refit"]


def filter_forward_headers(raw: dict) -> dict:
    out = {k: v for k, v in raw.items() if k.lower() in _FORWARDED}
    if not any(k.lower() == "accept" for k in out):
        out["Accept"] = "application/json"
    return out


class SSEMeter:
    """Counts contentful ``data:`` lines of an SSE byte stream as it passes through."""

    def __init__(self):
        self.start = time.time()
        self.first: Optional[float] = None
        self.events = 0
        self.buckets: dict[int, int] = {}
        self._buf = bytearray()

    def feed(self, chunk: bytes) -> list[float]:
        """Returns the arrival time of every new contentful event in this chunk."""
        self._buf.extend(chunk)
        stamps = []
        while (i := self._buf.find(b"\n")) >= 0:
            line = bytes(self._buf[:i]).rstrip(b"\r")
            del self._buf[:i + 1]
            if line.startswith(b"data:") and line[5:].strip() != b"[DONE]":
                now = time.time()
                if self.first is None:
                    self.first = now
                self.events += 1
                self.buckets[int(now)] = self.buckets.get(int(now), 0) + 1
                stamps.append(now)
        return stamps

    def summary(self) -> dict:
        total_ms = (time.time() - self.start) * 1e3
        ttft = None if self.first is None else (self.first - self.start) * 1e3
        tpot = None if (ttft is None or self.events <= 0) else max(total_ms - ttft, 0.0) / self.events
        return {"ttft_ms": ttft, "tpot_ms": tpot, "output_units": self.events or None,
                "output_buckets": dict(self.buckets)}


def create_app(registry: Optional[EndpointRegistry] = None) -> FastAPI:
    reg = registry or EndpointRegistry(config=RouterConfig())

    @asynccontextmanager
    async def lifespan(_: FastAPI):
        try:
            yield
        finally:
            await reg.aclose()

    app = FastAPI(lifespan=lifespan, title="parallax_b200 router")
    app.add_middleware(CORSMiddleware, allow_origins=["*"], allow_credentials=True, allow_methods=["*"],
                       allow_headers=["*"])
    app.state.registry = reg

    async def _json_object(req: HttpRequest) -> dict:
        payload = await req.json()
        if not isinstance(payload, dict):
            raise HTTPException(status_code=400, detail="Payload must be a JSON object")
        return payload

    def _http(e: RouterError) -> HTTPException:
        return HTTPException(status_code=e.status_code, detail=e.detail)

    @app.get("/health")
    async def health():
        return {"status": "ok", "apis": APIS}

    @app.get("/balancer/config")
    async def get_config():
        return {"config": await reg.get_balancer_config()}

    @app.post("/balancer/config")
    async def set_config(req: HttpRequest):
        try:
            return await reg.set_balancer_config(await _json_object(req))
        except ValueError as e:
            raise HTTPException(status_code=400, detail=str(e)) from e

    @app.post("/endpoint/enabled")
    async def set_enabled(req: HttpRequest):
        p = await _json_object(req)
        url = p.get("base_url") or p.get("endpoint")
        if not url:
            raise HTTPException(status_code=400, detail="Missing base_url")
        if not isinstance(p.get("enabled"), bool):
            raise HTTPException(status_code=400, detail="enabled must be a boolean")
        try:
            ep = await reg.set_endpoint_enabled(base_url=str(url), enabled=p["enabled"])
        except KeyError as e:
            raise HTTPException(status_code=404, detail=str(e)) from e
        return {"base_url": ep.base_url, "enabled": ep.enabled}

    @app.post("/register")
    async def register(req: HttpRequest):
        p = await _json_object(req)
        url = p.get("endpoint") or p.get("base_url")
        if not url:
            raise HTTPException(status_code=400, detail="Missing endpoint/base_url")
        url = str(url).strip().rstrip("/")
        ok, status, maxr, err = await reg.probe_endpoint_status(url)
        if status is None:
            raise HTTPException(status_code=400, detail=f"Endpoint not ready: {err or 'no status'}")
        try:
            ep = await reg.register(url, status_ok=ok, status_val=status, max_running_request=maxr, status_error=err)
        except ValueError as e:
            raise HTTPException(status_code=400, detail=str(e)) from e
        return {"endpoint_id": ep.endpoint_id, "base_url": ep.base_url}

    @app.post("/unregister")
    async def unregister(req: HttpRequest):
        p = await _json_object(req)
        url = p.get("endpoint") or p.get("base_url")
        if not url:
            raise HTTPException(status_code=400, detail="Missing endpoint/base_url")
        return {"removed": await reg.unregister(base_url=str(url))}

    @app.get("/endpoints")
    async def endpoints():
        return {"endpoints": await reg.list_endpoints()}

    @app.post("/weight/refit")
    async def weight_refit(req: HttpRequest):
        """Broadcast a weight-refit request to every registered cluster."""
        try:
            results = await reg.broadcast_raw(path="/weight/refit", headers=filter_forward_headers(dict(req.headers)),
                                              body=await req.body())
        except RouterError as e:
            raise _http(e) from e
        ok = all(r.get("ok") is True for r in results)
        return JSONResponse(status_code=200 if ok else 207,
                            content={"ok": ok, "broadcast_count": len(results), "results": results})

    async def _finish_failed(ep: Endpoint) -> None:
        await reg.mark_error(ep.base_url)
        await reg.mark_finish(ep.base_url, ttft_ms=None, tpot_ms=None, output_units=None, output_buckets=None)

    @app.post("/v1/chat/completions")
    async def chat(req: HttpRequest):
        body: dict[str, Any] = await req.json()
        try:
            ep = await reg.choose_best()
        except RouterError as e:
            raise _http(e) from e
        await reg.mark_start(ep.base_url)
        url = join_url(ep.base_url, "/v1/chat/completions")
        headers = filter_forward_headers(dict(req.headers))
        client = await reg.get_client()
        if not body.get("stream", False):
            t0 = time.time()
            try:
                resp = await client.post(url, headers=headers, json=body)
                await reg.mark_finish(ep.base_url, ttft_ms=(time.time() - t0) * 1e3, tpot_ms=None,
                                      output_units=None, output_buckets=None)
                return JSONResponse(status_code=resp.status_code, content=resp.json())
            except Exception as e:
                await _finish_failed(ep)
                raise HTTPException(status_code=502, detail=f"Upstream error: {e}") from e

        meter = SSEMeter()

        async def relay() -> AsyncIterator[bytes]:
            failed = False
            try:
                async with client.stream("POST", url, headers=headers, json=body) as upstream:
                    async for chunk in upstream.aiter_bytes():
                        if chunk:
                            first_before = meter.first
                            meter.feed(chunk)
                            if first_before is None and meter.first is not None:
                                await reg.mark_ttft(ep.base_url, ttft_ms=(meter.first - meter.start) * 1e3)
                        yield chunk
            except Exception:
                failed = True
                await reg.mark_error(ep.base_url)
                raise
            finally:
                m = meter.summary()
                await reg.mark_finish(ep.base_url, ttft_ms=m["ttft_ms"], tpot_ms=None if failed else m["tpot_ms"],
                                      output_units=m["output_units"], output_buckets=m["output_buckets"],
                                      sample_ttft_ms=m["ttft_ms"], ttft_already_counted=True)

        return StreamingResponse(relay(), media_type="text/event-stream",
                                 headers={"Cache-Control": "no-cache", "X-Content-Type-Options": "nosniff"})

    @app.get("/")
    async def ui():
        from pathlib import Path

        page = Path(__file__).resolve().parent / "ui" / "endpoints.html"
        return HTMLResponse(page.read_text(encoding="utf-8") if page.exists() else "<h1>parallax router</h1>")

    return app


def main(argv=None) -> None:
    import uvicorn

    ap = argparse.ArgumentParser(description="parallax_b200 HTTP router")
    ap.add_argument("--host", type=str, default="0.0.0.0", help="Listen host")
    ap.add_argument("--port", type=int, default=8081, help="Listen port")
    ap.add_argument("--strategy", type=str, default="round_robin", choices=["round_robin", "performance", "random"])
    a = ap.parse_args(argv)
    uvicorn.run(create_app(EndpointRegistry(config=RouterConfig(strategy=a.strategy))), host=a.host, port=a.port,
                log_level="info")


if __name__ == "__main__":
    main()
