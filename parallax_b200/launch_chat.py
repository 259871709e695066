"""``parallax chat``: a local HTTP endpoint (default port 3002) that forwards chat completions
and cluster-status queries to a cluster backend and serves a minimal chat page. Counterpart of
``src/parallax/launch_chat.py`` + ``src/parallax/server/node_chat_http_server.py:75-325``."""

from __future__ import annotations

import argparse

from fastapi import FastAPI
from fastapi import Request as HttpRequest
from fastapi.responses import HTMLResponse, Response, StreamingResponse

_PAGE = """<!doctype html><meta charset="utf-8"><title>parallax chat</title>
<style>body{font-family:system-ui;max-width:48rem;margin:2rem auto}#log{white-space:pre-wrap;border:1px solid #ccc;padding:1rem;min-height:12rem}
textarea{width:100%;height:4rem}</style><h1>parallax chat</h1><div id="log"></div>
<textarea id="msg" placeholder="Say something"></textarea><button onclick="send()">Send</button>
<script>const hist=[];async function send(){const t=document.getElementById('msg');hist.push({role:'user',content:t.value});
const log=document.getElementById('log');log.textContent+='\\n> '+t.value+'\\n';t.value='';
const r=await fetch('/v1/chat/completions',{method:'POST',headers:{'content-type':'application/json'},body:JSON.stringify({messages:hist,stream:true,max_tokens:512})});
const rd=r.body.getReader(),dec=new TextDecoder();let acc='',buf='';for(;;){const {value,done}=await rd.read();if(done)break;buf+=dec.decode(value);
let i;while((i=buf.indexOf('\\n'))>=0){const line=buf.slice(0,i).trim();buf=buf.slice(i+1);if(!line.startsWith('data:')||line.includes('[DONE]'))continue;
try{const d=JSON.parse(line.slice(5));const c=(d.choices[0]||{}).delta;if(c&&c.content){acc+=c.content;log.textContent+=c.content;}}catch(e){}}}
hist.push({role:'assistant',content:acc});}</script>"""


def create_chat_app(scheduler_addr: str, http_client_factory=None) -> FastAPI:
    base = scheduler_addr if scheduler_addr.startswith("http") else f"http://{scheduler_addr}"
    base = base.rstrip("/")
    app = FastAPI(title="parallax_b200 chat")
    holder = {}

    async def client():
        if "c" not in holder:
            if http_client_factory is not None:
                holder["c"] = http_client_factory()
            else:
                import httpx

                holder["c"] = httpx.AsyncClient(timeout=httpx.Timeout(20 * 60), trust_env=False)
        return holder["c"]

    @app.get("/")
    async def page():
        return HTMLResponse(_PAGE)

    @app.get("/cluster/status_json")
    async def status():
        c = await client()
        r = await c.get(base + "/cluster/status_json")
        return Response(content=r.content, status_code=r.status_code, media_type="application/json")

    @app.get("/v1/models")
    async def models():
        c = await client()
        r = await c.get(base + "/v1/models")
        return Response(content=r.content, status_code=r.status_code, media_type="application/json")

    @app.post("/v1/chat/completions")
    async def chat(req: HttpRequest):
        body = await req.json()
        c = await client()
        if body.get("stream", False):
            async def relay():
                async with c.stream("POST", base + "/v1/chat/completions", json=body) as up:
                    async for chunk in up.aiter_bytes():
                        if chunk:
                            yield chunk

            return StreamingResponse(relay(), media_type="text/event-stream", headers={"Cache-Control": "no-cache"})
        r = await c.post(base + "/v1/chat/completions", json=body)
        return Response(content=r.content, status_code=r.status_code,
                        media_type=r.headers.get("content-type", "application/json"))

    return app


def main(argv=None) -> None:
    import uvicorn

    p = argparse.ArgumentParser()
    p.add_argument("--scheduler-addr", type=str, default="127.0.0.1:3001")
    p.add_argument("--host", type=str, default="localhost")
    p.add_argument("--node-chat-port", type=int, default=3002)
    a, _ = p.parse_known_args(argv)
    uvicorn.run(create_chat_app(a.scheduler_addr), host=a.host, port=a.node_chat_port, log_level="info")


if __name__ == "__main__":
    main()
