"""Forwards ``/v1/chat/completions`` from the cluster backend to the first node of a route.

Resolve a routing table (retrying while every pipeline is busy), stamp it into the request's
``vllm_xargs`` together with the scheduler request id, POST the request to the first hop and
relay the answer (SSE pass-through for streams). Error mapping and retry budget follow
``src/backend/server/request_handler.py:33-245``: 503 not ready, 429 all pipelines busy, 502
when the downstream keeps failing.
"""

from __future__ import annotations

import asyncio
import json
import logging
import os
import time
from typing import Optional

from fastapi.responses import Response, StreamingResponse

from parallax_b200.backend.scheduler_manage import NODE_STATUS_AVAILABLE
from parallax_b200.frontend.engine_core_protocol import (PARALLAX_ROUTING_TABLE_EXTRA_ARG,
                                                         PARALLAX_SCHEDULER_REQUEST_ID_EXTRA_ARG)
from parallax_b200.frontend.openai_compat import openai_error_response
from parallax_b200.utils.request_metrics import get_request_metrics

logger = logging.getLogger(__name__)


class RequestHandler:
    MAX_FORWARD_RETRY = 10
    MAX_ROUTING_RETRY = 20
    # seconds between attempts (the reference's 10 and 5); the environment can shorten them for small clusters
    FORWARD_DELAY_SEC = float(os.environ.get("PARALLAX_FORWARD_RETRY_DELAY_S", "10"))
    RETRY_DELAY_SEC = float(os.environ.get("PARALLAX_ROUTING_RETRY_DELAY_S", "5"))

    def __init__(self, http_client_factory=None):
        self.scheduler_manage = None
        self._client = None
        self._client_factory = http_client_factory

    def set_scheduler_manage(self, scheduler_manage) -> None:
        self.scheduler_manage = scheduler_manage

    async def _http(self):
        if self._client is None:
            if self._client_factory is not None:
                self._client = self._client_factory()
            else:
                import httpx

                self._client = httpx.AsyncClient(timeout=httpx.Timeout(10 * 60), trust_env=False)
        return self._client

    def _prepare_backend_request(self, data: dict, request_id: str, routing_table: list[str]) -> dict:
        out = dict(data)
        out.pop("rid", None)
        out.pop("routing_table", None)
        if not out.get("request_id"):
            out["request_id"] = str(request_id)
        out["model"] = self.scheduler_manage.get_model_name()
        xargs = out.get("vllm_xargs")
        xargs = dict(xargs) if isinstance(xargs, dict) else {}
        xargs[PARALLAX_ROUTING_TABLE_EXTRA_ARG] = list(routing_table)
        xargs[PARALLAX_SCHEDULER_REQUEST_ID_EXTRA_ARG] = str(request_id)
        out["vllm_xargs"] = xargs
        return out

    async def _resolve_route(self, request_id, received_ts):
        """Returns (routing_table, error_response)."""
        for attempt in range(self.MAX_ROUTING_RETRY):
            try:
                table = await asyncio.to_thread(self.scheduler_manage.get_routing_table, request_id, received_ts)
            except Exception as e:
                logger.exception("routing failed: %s", e)
                return None, openai_error_response("Get routing table error", status_code=500,
                                                   err_type="server_error", code="routing_table_error")
            if table is None:
                return None, openai_error_response("Routing pipelines not ready", status_code=503,
                                                   err_type="server_unavailable", code="routing_not_ready")
            if table:
                return table, None
            if attempt + 1 < self.MAX_ROUTING_RETRY:
                await asyncio.sleep(self.RETRY_DELAY_SEC)
        return None, openai_error_response("All pipelines are busy or not ready. Please retry later.",
                                           status_code=429, err_type="rate_limit_error", code="rate_limit_exceeded")

    async def v1_chat_completions(self, data: dict, request_id, received_ts: float):
        sm = self.scheduler_manage
        if sm is None or sm.get_schedule_status() != NODE_STATUS_AVAILABLE:
            return openai_error_response("Server is not ready", status_code=503, err_type="server_unavailable",
                                         code="server_not_ready")
        start = time.time()
        for attempt in range(self.MAX_FORWARD_RETRY):
            table, err = await self._resolve_route(request_id, received_ts)
            if err is not None:
                return err
            url = sm.get_call_url_by_node_id(table[0])
            body = self._prepare_backend_request(data, str(request_id), table)
            try:
                if url is None:
                    raise RuntimeError(f"no call URL known for node {table[0]}")
                client = await self._http()
                target = url + "/v1/chat/completions"
                if data.get("stream", False):
                    return StreamingResponse(self._relay_stream(client, target, body, table, request_id, start),
                                             media_type="text/event-stream",
                                             headers={"X-Content-Type-Options": "nosniff", "Cache-Control": "no-cache"})
                resp = await client.post(target, json=body)
                sm.release_request(table)
                return Response(content=resp.content, status_code=resp.status_code,
                                headers={"content-type": resp.headers.get("content-type", "application/json")})
            except Exception as e:
                logger.warning("forward attempt %d for %s failed: %s", attempt + 1, request_id, e)
                sm.release_request(table)
                if attempt + 1 < self.MAX_FORWARD_RETRY:
                    await asyncio.sleep(self.FORWARD_DELAY_SEC)
        return openai_error_response("Downstream request failed", status_code=502, err_type="upstream_error",
                                     code="upstream_error")

    async def _relay_stream(self, client, url: str, body: dict, table: list[str], request_id, start: float):
        first = last = None
        last_chunk: Optional[bytes] = None
        try:
            async with client.stream("POST", url, json=body) as upstream:
                async for chunk in upstream.aiter_bytes():
                    if not chunk:
                        continue
                    last = time.time()
                    first = first or last
                    if not chunk.startswith(b"data: [DONE]"):
                        last_chunk = chunk
                    yield chunk
        except Exception as e:
            logger.warning("stream of %s broke: %s", request_id, e)
            yield ("data: " + json.dumps({"error": {"message": "upstream stream failed", "type": "upstream_error"}})
                   + "\n\n").encode()
        finally:
            self.scheduler_manage.release_request(table)
            if last_chunk is not None:
                tps, ttft, n_in, n_out = get_request_metrics(last_chunk, start, first, last)
                if tps is not None:
                    logger.info("request %s | TPS %.2f | TTFT %s ms | in %s | out %s", request_id, tps, ttft, n_in, n_out)
