"""OpenAI-style payload helpers shared by the node frontend, the cluster backend and the router
(error bodies, ``/v1/models`` body, and the envelope that carries a non-streaming HTTP
response through an RPC hop; cf. ``src/backend/server/openai_compat.py:10-95``)."""

from __future__ import annotations

import base64
import json
from typing import Any, Optional

ENVELOPE_KEY = "__parallax_http_response__"


def openai_error_payload(message: str, *, err_type: str = "server_error", param: Optional[str] = None,
                         code: Optional[str] = None) -> dict:
    return {"error": {"message": message, "type": err_type, "param": param, "code": code or err_type}}


def openai_error_response(message: str, *, status_code: int, err_type: str = "server_error",
                          param: Optional[str] = None, code: Optional[str] = None):
    from fastapi.responses import JSONResponse

    return JSONResponse(content=openai_error_payload(message, err_type=err_type, param=param, code=code),
                        status_code=status_code)


def openai_models_payload(model_name: Optional[str]) -> dict:
    data = [{"id": model_name, "object": "model", "created": 0, "owned_by": "parallax"}] if model_name else []
    return {"object": "list", "data": data}


def encode_http_response_envelope(*, status_code: int, content_type: Optional[str], body: bytes) -> bytes:
    env = {ENVELOPE_KEY: True, "status_code": int(status_code), "content_type": content_type or "application/json",
           "body_base64": base64.b64encode(body).decode("ascii")}
    return json.dumps(env, separators=(",", ":")).encode("utf-8")


def decode_http_response_envelope(content: bytes) -> Optional[tuple[int, str, bytes]]:
    try:
        env: Any = json.loads(content.decode("utf-8"))
    except (UnicodeDecodeError, json.JSONDecodeError):
        return None
    if not isinstance(env, dict) or env.get(ENVELOPE_KEY) is not True or not isinstance(env.get("body_base64"), str):
        return None
    try:
        body = base64.b64decode(env["body_base64"])
    except ValueError:
        return None
    return int(env.get("status_code", 200)), str(env.get("content_type") or "application/json"), body
