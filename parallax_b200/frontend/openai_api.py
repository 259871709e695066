"""OpenAI-compatible HTTP frontend of a serving node.

Endpoints: ``POST /v1/chat/completions``, ``POST /v1/completions`` (streaming via SSE and
non-streaming), ``GET /v1/models``, ``GET /health``, ``POST /abort``. The frontend tokenises
(chat template), submits a :class:`Request` to the engine loop, detokenises incrementally,
applies stop strings and reports usage. The reference delegates this part to an external Rust
binary (``src/parallax/server/vllm_rust_frontend.py``); request options it carried in
``vllm_xargs`` (routing table, scheduler request id) are accepted here as well.
"""

from __future__ import annotations

import asyncio
import json
import time
import uuid
from typing import Any, AsyncIterator, Optional

from fastapi import FastAPI
from fastapi import Request as HttpRequest
from fastapi.responses import JSONResponse, StreamingResponse

from parallax_b200.engine.request import Request, RequestStatus, SamplingParams
from parallax_b200.engine.service import EngineLoop, TokenEvent
from parallax_b200.frontend.openai_compat import openai_error_response, openai_models_payload
from parallax_b200.frontend.tokenizer import IncrementalDetokenizer, TokenizerWrapper

_FINISH = {RequestStatus.FINISHED_EOS: "stop", RequestStatus.FINISHED_MAX_LENGTH: "length",
           RequestStatus.FINISHED_ABORT: "abort", RequestStatus.CANCELLED: "abort", RequestStatus.ERROR: "error"}


def _num(body: dict, key: str, default):
    v = body.get(key)
    return default if v is None else v


def sampling_params_from_body(body: dict, default_max_tokens: int = 512) -> SamplingParams:
    stop = body.get("stop")
    if isinstance(stop, str):
        stop = [stop]
    max_tokens = body.get("max_completion_tokens") or body.get("max_tokens") or default_max_tokens
    top_k = int(_num(body, "top_k", -1))
    return SamplingParams(
        max_new_tokens=int(max_tokens), min_new_tokens=int(_num(body, "min_tokens", 0)),
        temperature=float(_num(body, "temperature", 1.0)), top_p=float(_num(body, "top_p", 1.0)),
        min_p=float(_num(body, "min_p", 0.0)), top_k=top_k if top_k > 0 else -1,
        stop_token_ids=body.get("stop_token_ids"), ignore_eos=bool(body.get("ignore_eos", False)),
        stop_strs=stop, repetition_penalty=float(_num(body, "repetition_penalty", 1.0)),
        presence_penalty=float(_num(body, "presence_penalty", 0.0)),
        frequency_penalty=float(_num(body, "frequency_penalty", 0.0)), seed=body.get("seed"),
        json_schema=_json_schema_of(body))


def _json_schema_of(body: dict):
    """``response_format`` of the OpenAI API (``{"type": "json_schema", "json_schema": {"schema": ...}}`` or
    ``{"type": "json_object"}``) or a bare ``json_schema`` field, as JSON text; None when the reply is free text."""
    import json

    rf = body.get("response_format")
    schema = body.get("json_schema")
    if isinstance(rf, dict):
        if rf.get("type") == "json_object":
            schema = {"type": "object"}
        elif rf.get("type") == "json_schema":
            js = rf.get("json_schema") or {}
            schema = js.get("schema", js) if isinstance(js, dict) else js
    if schema is None:
        return None
    return schema if isinstance(schema, str) else json.dumps(schema)


async def _events(q, poll_s: float = 0.002) -> AsyncIterator[TokenEvent]:
    """Bridge a thread-side queue into the asyncio world without blocking the loop."""
    import queue as _q

    while True:
        try:
            ev = q.get_nowait()
        except _q.Empty:
            await asyncio.sleep(poll_s)
            continue
        yield ev
        if ev.finished:
            return


def create_app(loop: EngineLoop, tokenizer: TokenizerWrapper, model_name: str, max_model_len: int = 32768):
    app = FastAPI(title="parallax_b200 node")
    app.state.loop, app.state.tokenizer, app.state.model_name = loop, tokenizer, model_name
    eng = getattr(loop, "engine", None)
    if eng is not None and getattr(eng, "tokenizer", 0) is None:
        eng.tokenizer = tokenizer      # constrained decoding (response_format) checks tokens by their text

    @app.get("/")
    @app.get("/ui")
    async def ui():
        from pathlib import Path

        from fastapi.responses import HTMLResponse

        return HTMLResponse((Path(__file__).resolve().parent / "ui" / "index.html").read_text())

    @app.get("/health")
    async def health():
        return {"status": "ok", "inflight": loop.num_inflight, "steps": loop.steps}

    @app.get("/v1/models")
    async def models():
        return openai_models_payload(model_name)

    @app.post("/abort")
    async def abort(req: HttpRequest):
        body = await req.json()
        for rid in body.get("request_ids", [body.get("request_id")]):
            if rid:
                loop.abort(str(rid))
        return {"ok": True}

    def _build(body: dict, chat: bool):
        if chat:
            msgs = body.get("messages")
            if not isinstance(msgs, list) or not msgs:
                raise ValueError("'messages' must be a non-empty list")
            ids = tokenizer.apply_chat_template(msgs, add_generation_prompt=True,
                                                **(body.get("chat_template_kwargs") or {}))
        else:
            prompt = body.get("prompt")
            if isinstance(prompt, list) and prompt and isinstance(prompt[0], int):
                ids = [int(x) for x in prompt]
            elif isinstance(prompt, str):
                ids = tokenizer.encode(prompt)
            else:
                raise ValueError("'prompt' must be a string or a list of token ids")
        if not ids:
            raise ValueError("empty prompt")
        sp = sampling_params_from_body(body)
        sp.verify()
        if not sp.ignore_eos and tokenizer.eos_token_ids:
            sp.stop_token_ids = (sp.stop_token_ids or set()) | tokenizer.eos_token_ids
        if len(ids) >= max_model_len:
            raise ValueError(f"prompt has {len(ids)} tokens; the limit is {max_model_len - 1}")
        xargs = body.get("vllm_xargs") or {}
        r = Request(request_id=body.get("request_id") or f"{'chatcmpl' if chat else 'cmpl'}-{uuid.uuid4().hex}",
                    input_ids=ids, sampling_params=sp, routing_table=xargs.get("parallax_routing_table") or [],
                    max_total_length=min(max_model_len, len(ids) + sp.max_new_tokens),
                    return_probs=bool(body.get("return_probs", False)),
                    lora_path=body.get("lora_path") or xargs.get("lora_path") or None)
        r.scheduler_request_id = xargs.get("parallax_scheduler_request_id")
        return r

    def _chunk(rid: str, chat: bool, created: int, delta: Optional[str], finish: Optional[str], first: bool,
               usage: Optional[dict] = None) -> str:
        if chat:
            d: dict[str, Any] = {}
            if first:
                d["role"] = "assistant"
            if delta is not None:
                d["content"] = delta      # may be "" while a multi-byte character is still incomplete
            choice = {"index": 0, "delta": d, "finish_reason": finish}
            obj = "chat.completion.chunk"
        else:
            choice = {"index": 0, "text": delta or "", "finish_reason": finish}
            obj = "text_completion"
        payload = {"id": rid, "object": obj, "created": created, "model": model_name, "choices": [choice]}
        if usage is not None:
            payload["usage"] = usage
        return f"data: {json.dumps(payload, ensure_ascii=False)}\n\n"

    async def _serve(http_req: HttpRequest, chat: bool):
        try:
            body = await http_req.json()
            req = _build(body, chat)
        except ValueError as e:
            return openai_error_response(str(e), status_code=400, err_type="invalid_request_error")
        except Exception as e:
            return openai_error_response(f"bad request: {e}", status_code=400, err_type="invalid_request_error")
        created = int(time.time())
        q = loop.submit(req)
        detok = IncrementalDetokenizer(tokenizer, req.sampling_params.stop_strs)
        stream = bool(body.get("stream", False))
        include_usage = bool((body.get("stream_options") or {}).get("include_usage", True))

        def usage() -> dict:
            return {"prompt_tokens": req.prompt_len, "completion_tokens": req.output_length,
                    "total_tokens": req.prompt_len + req.output_length,
                    "prompt_tokens_details": {"cached_tokens": req.num_cached_tokens}}

        async def gen_stream():
            first, finish = True, None
            try:
                async for ev in _events(q):
                    if await http_req.is_disconnected():
                        loop.abort(req.request_id)
                    text = ""
                    if ev.token_id is not None and not (ev.finished and ev.status == RequestStatus.FINISHED_EOS
                                                        and ev.token_id in (req.sampling_params.stop_token_ids or ())):
                        text = detok.add(ev.token_id)
                    if detok.stopped and not ev.finished:
                        loop.abort(req.request_id)
                        finish = "stop"
                    if ev.finished:
                        text += detok.flush()
                        finish = finish or ("error" if (ev.error or ev.status == RequestStatus.ERROR)
                                            else _FINISH.get(ev.status, "stop"))
                    if text or first:
                        yield _chunk(req.request_id, chat, created, text, None, first)
                        first = False
                    if ev.finished:
                        yield _chunk(req.request_id, chat, created, None, finish, False,
                                     usage() if include_usage else None)
                yield "data: [DONE]\n\n"
            except asyncio.CancelledError:
                loop.abort(req.request_id)
                raise

        if stream:
            return StreamingResponse(gen_stream(), media_type="text/event-stream")

        pieces, finish, err = [], None, None
        async for ev in _events(q):
            if ev.token_id is not None and not (ev.finished and ev.status == RequestStatus.FINISHED_EOS
                                                and ev.token_id in (req.sampling_params.stop_token_ids or ())):
                pieces.append(detok.add(ev.token_id))
            if detok.stopped and not ev.finished:
                loop.abort(req.request_id)
                finish = "stop"
            if ev.finished:
                pieces.append(detok.flush())
                err = ev.error
                if err is None and ev.status == RequestStatus.ERROR:
                    err = "the request failed on the serving node (a pipeline peer did not answer, or a step failed)"
                finish = finish or _FINISH.get(ev.status, "stop")
        if err:
            return openai_error_response(err, status_code=500)
        text = "".join(pieces)
        if chat:
            choice = {"index": 0, "message": {"role": "assistant", "content": text}, "finish_reason": finish}
            obj = "chat.completion"
        else:
            choice = {"index": 0, "text": text, "finish_reason": finish}
            obj = "text_completion"
        out = {"id": req.request_id, "object": obj, "created": created, "model": model_name,
               "choices": [choice], "usage": usage()}
        if req.return_probs:
            out["choices"][0]["token_probs"] = req.output_probs
        if getattr(req, "routed_experts", None) is not None:
            # engines started with --enable-return-routed-experts: [token][MoE layer][top-k] expert ids of
            # every token that was fed to the model (prompt and all generated tokens but the last)
            out["choices"][0]["routed_experts"] = req.routed_experts
        return JSONResponse(out)

    @app.post("/weight/refit")
    async def weight_refit(req: HttpRequest):
        """Online refit of a stand-alone server (cluster nodes get theirs from the scheduler): the scheduler's
        request format, ``{"index_map": {weight: content id}, "paths": {content id: file}}``. Applied on the engine
        thread between two steps."""
        eng = getattr(loop, "engine", None)
        if eng is None or not hasattr(eng, "apply_refit") or not hasattr(loop, "call"):
            return openai_error_response("this server takes weight refits from its scheduler", status_code=404)
        try:
            body = await req.json()
            used = await asyncio.wrap_future(loop.call(lambda: eng.apply_refit(body)))
        except Exception as e:
            return openai_error_response(f"weight refit failed: {e}", status_code=400, err_type="invalid_request_error")
        return JSONResponse({"type": "weight_refit", "data": {"tensors": int(used)}})

    @app.post("/v1/chat/completions")
    async def chat_completions(req: HttpRequest):
        return await _serve(req, chat=True)

    @app.post("/v1/completions")
    async def completions(req: HttpRequest):
        return await _serve(req, chat=False)

    return app
