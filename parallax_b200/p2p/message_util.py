"""Wire format of stage-to-stage packets that leave the box (node-to-node pipeline hops).

Inside one NVSwitch box activations move GPU-to-GPU over NCCL and never touch this module.
Between boxes (or between processes in the CPU tests) a batch of ``IntermediateRequest``s is
serialised as one ``ForwardRequest`` message with the same fields as the reference's protobuf
schema (``src/parallax/p2p/proto/forward.proto:6-57``, helpers
``src/parallax/p2p/message_util.py:18-219``): forward mode, and per request: rid,
output_length, routing_table, input_ids, sampling_params, next_token_id, hidden_states,
lora_path, token_prob, return_probs (+ chunked-prefill markers). Tensors travel as raw
little-endian bytes with dtype and shape; encoding is msgpack.
"""

from __future__ import annotations

from typing import Any, Optional

import msgpack
import numpy as np
import torch

from parallax_b200.engine.request import IntermediateRequest, RequestStatus, SamplingParams

FORWARD_MODE_EXTEND = 0
FORWARD_MODE_DECODE = 1
FORWARD_MODE_MIXED = 2

_DTYPES = {
    "float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16,
    "int32": torch.int32, "int64": torch.int64, "uint8": torch.uint8, "int8": torch.int8,
    "float8_e4m3fn": torch.float8_e4m3fn,
}
_DTYPE_NAMES = {v: k for k, v in _DTYPES.items()}


def tensor_to_bytes(t: torch.Tensor) -> dict:
    """Device tensors are copied to the host; bf16/fp8 are shipped as their raw bit patterns."""
    t = t.detach().contiguous().cpu()
    name = _DTYPE_NAMES.get(t.dtype)
    if name is None:
        raise TypeError(f"unsupported tensor dtype {t.dtype}")
    raw = t.view(torch.uint8) if t.dtype != torch.uint8 else t
    return {"dtype": name, "shape": list(t.shape), "data": raw.numpy().tobytes()}


def bytes_to_tensor(d: dict, device=None) -> torch.Tensor:
    dtype = _DTYPES[d["dtype"]]
    buf = np.frombuffer(d["data"], dtype=np.uint8).copy()
    t = torch.from_numpy(buf).view(dtype).reshape(d["shape"])
    return t.to(device) if device is not None else t


def _req_to_dict(r: IntermediateRequest) -> dict:
    d: dict[str, Any] = {
        "rid": r.request_id,
        "output_length": int(r.output_length),
        "current_position": int(r.current_position),
        "status": r.status.value,
        "routing_table": list(r.routing_table or []),
        "input_ids": [int(x) for x in (r.input_ids or [])],
        "sampling_params": r.sampling_params.to_dict() if r.sampling_params is not None else None,
        "next_token_id": -1 if r.next_token_id is None else int(r.next_token_id),
        "hidden_states": tensor_to_bytes(r.hidden_states) if r.hidden_states is not None else None,
        "lora_path": r.lora_path or "",
        "token_prob": -1.0 if r.token_prob is None else float(r.token_prob),
        "return_probs": bool(r.return_probs),
        "is_chunked": bool(r.is_chunked),
        "is_last_chunk": bool(r.is_last_chunk),
        "chunk_start": int(r.chunk_start),
        "abort": bool(r.abort),
    }
    return d


def _dict_to_req(d: dict, device=None) -> IntermediateRequest:
    sp = SamplingParams.from_dict(d["sampling_params"]) if d.get("sampling_params") else SamplingParams()
    r = IntermediateRequest(
        request_id=d["rid"], current_position=d["current_position"], status=RequestStatus(d["status"]),
        input_ids=list(d["input_ids"]) or None,
        hidden_states=bytes_to_tensor(d["hidden_states"], device) if d.get("hidden_states") else None,
        next_token_id=None if d["next_token_id"] < 0 else d["next_token_id"],
        routing_table=list(d["routing_table"]), sampling_params=sp, lora_path=d.get("lora_path") or None,
        token_prob=None if d["token_prob"] < 0 else d["token_prob"], return_probs=d["return_probs"],
        is_chunked=d.get("is_chunked", False), is_last_chunk=d.get("is_last_chunk", True),
        chunk_start=d.get("chunk_start", 0), output_length=d["output_length"])
    r.abort = d.get("abort", False)
    return r


def request_to_proto(reqs: list[IntermediateRequest], forward_mode: Optional[int] = None) -> bytes:
    """Serialise a batch of stage packets into one ForwardRequest message."""
    if forward_mode is None:
        kinds = {r.is_prefill for r in reqs}
        forward_mode = FORWARD_MODE_MIXED if len(kinds) > 1 else (
            FORWARD_MODE_EXTEND if kinds == {True} else FORWARD_MODE_DECODE)
    return msgpack.packb({"forward_mode": forward_mode, "reqs": [_req_to_dict(r) for r in reqs]},
                         use_bin_type=True)


def proto_to_request(payload: bytes, device=None) -> list[IntermediateRequest]:
    msg = msgpack.unpackb(payload, raw=False)
    return [_dict_to_req(d, device) for d in msg["reqs"]]


def forward_mode_of(payload: bytes) -> int:
    return msgpack.unpackb(payload, raw=False)["forward_mode"]


def abort_request_to_proto(request_ids: list[str]) -> bytes:
    return msgpack.packb({"abort": [str(r) for r in request_ids]}, use_bin_type=True)


def proto_to_abort_request(payload: bytes) -> list[str]:
    return list(msgpack.unpackb(payload, raw=False)["abort"])
