"""Cluster control plane ("backend"): REST surface over the cluster scheduler.

Endpoints (``src/backend/main.py:42-236`` of the reference): ``POST /weight/refit``,
``GET /weight/refit/timestamp``, ``GET /model/list``, ``GET /v1/models``,
``POST /scheduler/init``, ``GET /node/join/command``, ``GET /cluster/status`` (ndjson stream),
``GET /cluster/status_json``, ``POST /v1/chat/completions``; plus the node-facing control
calls ``POST /node/join``, ``/node/update``, ``/node/leave`` that replace the reference's
libp2p RPCs, and a static status page.

    python -m parallax_b200.backend.app --port 3001 --model-name Qwen/Qwen3-8B --init-nodes-num 1
"""

from __future__ import annotations

import argparse
import asyncio
import json
import time
import uuid
from typing import Optional

from fastapi import FastAPI
from fastapi import Request as HttpRequest
from fastapi.middleware.cors import CORSMiddleware
from fastapi.responses import HTMLResponse, JSONResponse, StreamingResponse

from parallax_b200.backend.request_handler import RequestHandler
from parallax_b200.backend.scheduler_manage import SchedulerManage
from parallax_b200.backend.static_config import get_model_list, get_node_join_command, init_model_info_dict_cache
from parallax_b200.frontend.openai_compat import openai_error_response, openai_models_payload

def _ui_page(name: str) -> str:
    from pathlib import Path

    return (Path(__file__).resolve().parent.parent / "frontend" / "ui" / name).read_text()



def create_app(scheduler_manage: SchedulerManage, request_handler: Optional[RequestHandler] = None) -> FastAPI:
    sm = scheduler_manage
    rh = request_handler or RequestHandler()
    rh.set_scheduler_manage(sm)
    app = FastAPI(title="parallax_b200 backend")
    app.add_middleware(CORSMiddleware, allow_origins=["*"], allow_credentials=True, allow_methods=["*"],
                       allow_headers=["*"])
    app.state.scheduler_manage = sm

    @app.get("/chat")
    async def chat_ui():
        return HTMLResponse(_ui_page("index.html"))

    @app.post("/weight/refit")
    async def weight_refit(req: HttpRequest):
        ok = sm.weight_refit(await req.json())
        return JSONResponse({"type": "weight_refit", "data": None if ok else "Sever not ready"},
                            status_code=200 if ok else 500)

    @app.get("/weight/refit/timestamp")
    async def weight_refit_timestamp():
        return {"latest_timestamp": sm.get_last_refit_time()}

    @app.get("/model/list")
    async def model_list():
        return {"type": "model_list", "data": get_model_list()}

    @app.get("/v1/models")
    async def v1_models():
        return openai_models_payload(sm.get_model_name())

    @app.post("/scheduler/init")
    async def scheduler_init(req: HttpRequest):
        body = await req.json()
        name, n = body.get("model_name"), body.get("init_nodes_num")
        if name is None:
            return JSONResponse({"type": "scheduler_init", "error": "model_name is required"}, status_code=400)
        if n is None:
            return JSONResponse({"type": "scheduler_init", "error": "init_nodes_num is required"}, status_code=400)
        try:
            if sm.is_running():
                sm.stop()
            sm.run(name, int(n), bool(body.get("is_local_network", True)))
        except Exception as e:
            return JSONResponse({"type": "scheduler_init", "error": str(e)}, status_code=500)
        return {"type": "scheduler_init", "data": {"model_name": name, "init_nodes_num": n,
                                                   "is_local_network": body.get("is_local_network")}}

    @app.get("/node/join/command")
    async def node_join_command():
        return {"type": "node_join_command", "data": get_node_join_command(sm.get_peer_id(), sm.get_is_local_network())}

    @app.get("/cluster/status")
    async def cluster_status():
        async def gen():
            while True:
                yield json.dumps(sm.get_cluster_status(), ensure_ascii=False) + "\n"
                await asyncio.sleep(1)

        return StreamingResponse(gen(), media_type="application/x-ndjson",
                                 headers={"Cache-Control": "no-cache", "Connection": "keep-alive"})

    @app.get("/cluster/status_json")
    async def cluster_status_json():
        return sm.get_cluster_status()

    # ---- node-facing control calls
    def _handler_or_503():
        if sm.connection_handler is None:
            return None, JSONResponse({"error": "Scheduler is not initialized"}, status_code=503)
        return sm.connection_handler, None

    @app.post("/node/join")
    async def node_join(req: HttpRequest):
        h, err = _handler_or_503()
        if err:
            return err
        msg = await req.json()
        return await asyncio.to_thread(h.node_join, msg, float(msg.get("wait_seconds", 300)))

    @app.post("/node/update")
    async def node_update(req: HttpRequest):
        h, err = _handler_or_503()
        if err:
            return err
        alloc, refit = await asyncio.to_thread(h.node_update, await req.json())
        return {"layer_allocation": alloc, "refit_request": refit}

    @app.post("/node/leave")
    async def node_leave(req: HttpRequest):
        h, err = _handler_or_503()
        if err:
            return err
        return h.node_leave(await req.json())

    @app.post("/node/addresses")
    async def node_addresses():
        return dict(sm.call_urls)

    @app.post("/v1/chat/completions")
    async def chat(req: HttpRequest):
        try:
            data = await req.json()
        except Exception:
            return openai_error_response("Invalid request body", status_code=400, err_type="invalid_request_error")
        if not isinstance(data, dict):
            return openai_error_response("Request body must be a JSON object", status_code=400,
                                         err_type="invalid_request_error")
        return await rh.v1_chat_completions(data, uuid.uuid4(), time.time())

    @app.get("/")
    async def index():
        # the cluster web app: set up -> join -> chat (one static file, hash routes)
        return HTMLResponse(_ui_page("app.html"), headers={"Cache-Control": "no-store"})

    return app


def parse_args(argv=None) -> argparse.Namespace:
    p = argparse.ArgumentParser(formatter_class=argparse.ArgumentDefaultsHelpFormatter)
    p.add_argument("--initial-peers", nargs="+", default=[])
    p.add_argument("--relay-servers", nargs="+", default=[])
    p.add_argument("--announce-maddrs", nargs="+", default=[])
    p.add_argument("--tcp-port", type=int, default=0)
    p.add_argument("--udp-port", type=int, default=0)
    p.add_argument("--dht-prefix", type=str, default="gradient")
    p.add_argument("--host", type=str, default="localhost", help="Host to listen on")
    p.add_argument("--port", type=int, default=3001, help="Port to listen on")
    p.add_argument("--log-level", type=str, default="INFO", choices=["DEBUG", "INFO", "WARNING", "ERROR"])
    p.add_argument("--model-name", type=str, default=None, help="Model name")
    p.add_argument("--init-nodes-num", type=int, default=None, help="Number of initial nodes")
    p.add_argument("--is-local-network", type=lambda s: str(s).lower() not in ("0", "false", "no"), default=True)
    p.add_argument("--use-hfcache", action="store_true", default=False)
    p.add_argument("--enable-weight-refit", type=lambda s: str(s).lower() in ("1", "true", "yes"), default=False)
    p.add_argument("--weight-refit-mode", type=str, default="disk")
    return p.parse_args(argv)


def main(argv=None) -> None:
    import uvicorn

    from parallax_b200.utils.logging_config import set_log_level

    a = parse_args(argv)
    set_log_level(a.log_level)
    if a.model_name is None:
        init_model_info_dict_cache(a.use_hfcache)
    adv = (a.announce_maddrs[0] if a.announce_maddrs else f"{'127.0.0.1' if a.host in ('localhost', '0.0.0.0') else a.host}:{a.port}")
    sm = SchedulerManage(http_port=a.port, use_hfcache=a.use_hfcache, enable_weight_refit=a.enable_weight_refit,
                         weight_refit_mode=a.weight_refit_mode, advertise_addr=adv)
    if a.model_name is not None and a.init_nodes_num is not None:
        sm.run(a.model_name, a.init_nodes_num, a.is_local_network)
    from parallax_b200.utils.banner import display_parallax_run
    from parallax_b200.utils.version_check import check_latest_release

    display_parallax_run()
    check_latest_release()
    uvicorn.run(create_app(sm), host=a.host, port=a.port, log_level="info")


if __name__ == "__main__":
    main()
