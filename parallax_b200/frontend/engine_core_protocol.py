"""Engine-core wire protocol (msgpack over ZMQ) between an HTTP frontend and the engine.

The frame layout is an external contract (vLLM's engine-core protocol, which the reference
speaks to its Rust frontend, ``src/parallax/server/engine_core_protocol.py:27-396``):

* request frames ``[type, payload]`` with type ``0x00`` ADD, ``0x01`` ABORT, ``0x02``
  START_DP_WAVE, ``0x03`` UTILITY (the last two are rejected);
* an ADD payload is a 20-field positional array (or a map with the same names);
* the engine answers with an 8-field ``outputs`` array holding 13-field ``output`` arrays.

Features the engine does not implement (log-probs, logit bias, structured outputs,
multi-modal inputs, LoRA per request, prompt embeddings) are rejected explicitly rather
than ignored.
"""

from __future__ import annotations

import time
from enum import IntEnum
from typing import Any, Iterable, Mapping, Optional

import msgpack

from parallax_b200.engine.request import Request, SamplingParams

ENGINE_IDENTITY = (0).to_bytes(2, "little")

REQUEST_TYPE_ADD = b"\x00"
REQUEST_TYPE_ABORT = b"\x01"
REQUEST_TYPE_START_DP_WAVE = b"\x02"
REQUEST_TYPE_UTILITY = b"\x03"


class EngineCoreFinishReason(IntEnum):
    STOP = 0
    LENGTH = 1
    ABORT = 2
    ERROR = 3
    REPETITION = 4


class UnsupportedEngineCoreField(ValueError):
    pass


# (name, default) in wire order
_REQUEST_SCHEMA: list[tuple[str, Any]] = [
    ("request_id", None), ("prompt_token_ids", None), ("mm_features", None), ("sampling_params", None),
    ("pooling_params", None), ("arrival_time", None), ("lora_request", None), ("cache_salt", None),
    ("data_parallel_rank", None), ("prompt_embeds", None), ("prompt_is_token_ids", None),
    ("client_index", 0), ("current_wave", 0), ("priority", 0), ("trace_headers", None),
    ("resumable", False), ("external_req_id", None), ("reasoning_ended", None),
    ("reasoning_parser_kwargs", None), ("abort_immediately", False),
]
ENGINE_CORE_REQUEST_FIELDS = [n for n, _ in _REQUEST_SCHEMA]
ENGINE_CORE_OUTPUT_FIELD_COUNT = 13
ENGINE_CORE_OUTPUTS_FIELD_COUNT = 8
PARALLAX_ROUTING_TABLE_EXTRA_ARG = "parallax_routing_table"
PARALLAX_SCHEDULER_REQUEST_ID_EXTRA_ARG = "parallax_scheduler_request_id"
PARALLAX_ENGINE_CORE_VERSION = "parallax"

_UNSUPPORTED_SAMPLING = ("logprobs", "prompt_logprobs", "logit_bias", "allowed_token_ids",
                         "_bad_words_token_ids", "bad_words_token_ids", "structured_outputs",
                         "logprob_token_ids", "skip_reading_prefix_cache")
_UNSUPPORTED_REQUEST = ("mm_features", "pooling_params", "lora_request", "prompt_embeds",
                        "reasoning_parser_kwargs")


def _unpack(payload: bytes) -> Any:
    return msgpack.unpackb(payload, raw=False, strict_map_key=False)


def _pack(value: Any) -> bytes:
    return msgpack.packb(value, use_bin_type=True)


def _str_keys(m: Mapping) -> dict:
    return {(k.decode("utf-8") if isinstance(k, bytes) else str(k)): v for k, v in m.items()}


def decode_engine_core_request(payload) -> dict:
    value = _unpack(payload) if isinstance(payload, (bytes, bytearray)) else payload
    if isinstance(value, Mapping):
        out = _str_keys(value)
    elif isinstance(value, (list, tuple)):
        if len(value) > len(_REQUEST_SCHEMA):
            raise ValueError(f"Expected at most {len(_REQUEST_SCHEMA)} fields, got {len(value)}")
        out = {name: value[i] for i, (name, _) in enumerate(_REQUEST_SCHEMA[:len(value)])}
    else:
        raise TypeError(f"Expected MessagePack array or map, got {type(value)!r}")
    for name, default in _REQUEST_SCHEMA:
        out.setdefault(name, default)
    return out


def decode_engine_core_abort(payload) -> list[str]:
    value = _unpack(payload) if isinstance(payload, (bytes, bytearray)) else payload
    if not isinstance(value, (list, tuple)):
        raise TypeError(f"Expected abort request id list, got {type(value)!r}")
    return [str(r) for r in value]


def decode_engine_core_frame(request_type: bytes, payload: bytes) -> tuple[str, Any]:
    if request_type == REQUEST_TYPE_ADD:
        return "add", decode_engine_core_request(payload)
    if request_type == REQUEST_TYPE_ABORT:
        return "abort", decode_engine_core_abort(payload)
    if request_type == REQUEST_TYPE_UTILITY:
        raise UnsupportedEngineCoreField("EngineCoreRequest Utility calls are not supported")
    if request_type == REQUEST_TYPE_START_DP_WAVE:
        raise UnsupportedEngineCoreField("EngineCoreRequest StartDpWave is not supported")
    raise ValueError(f"Unknown engine-core request type frame: {request_type!r}")


def encode_engine_core_request(request) -> bytes:
    return _pack(request)


def encode_engine_core_abort(request_ids: Iterable[str]) -> bytes:
    return _pack(list(request_ids))


def engine_core_ready_payload(*, max_model_len: int, dtype: Optional[str], block_size: int = 16,
                              num_gpu_blocks: int = 0, dp_stats_address: Optional[str] = None,
                              world_size: int = 1, data_parallel_size: int = 1) -> bytes:
    """Registration message the engine sends once it can accept requests."""
    return _pack({
        "max_model_len": int(max_model_len), "num_gpu_blocks": int(num_gpu_blocks),
        "block_size": int(block_size), "dp_stats_address": dp_stats_address, "dtype": dtype,
        "vllm_version": PARALLAX_ENGINE_CORE_VERSION, "world_size": int(world_size),
        "data_parallel_size": int(data_parallel_size),
    })


def _extra_args(params: Mapping) -> dict:
    extra = params.get("extra_args")
    if extra is None:
        return {}
    if not isinstance(extra, Mapping):
        raise UnsupportedEngineCoreField("EngineCoreSamplingParams.extra_args must be a map")
    return _str_keys(extra)


def routing_table_from_engine_core_sampling_params(params: Optional[Mapping]) -> list[str]:
    if params is None:
        return []
    table = _extra_args(_str_keys(params)).get(PARALLAX_ROUTING_TABLE_EXTRA_ARG)
    if table is None:
        return []
    where = f"EngineCoreSamplingParams.extra_args.{PARALLAX_ROUTING_TABLE_EXTRA_ARG}"
    if not isinstance(table, (list, tuple)):
        raise UnsupportedEngineCoreField(f"{where} must be a list")
    out = []
    for nid in table:
        if isinstance(nid, bytes):
            nid = nid.decode("utf-8")
        if not isinstance(nid, str) or not nid:
            raise UnsupportedEngineCoreField(f"{where} must contain non-empty strings")
        out.append(nid)
    return out


def scheduler_request_id_from_sampling_params(params: Optional[Mapping]) -> Optional[str]:
    if params is None:
        return None
    v = _extra_args(_str_keys(params)).get(PARALLAX_SCHEDULER_REQUEST_ID_EXTRA_ARG)
    return None if v is None else str(v)


def sampling_params_from_engine_core(params: Optional[Mapping]) -> SamplingParams:
    if params is None:
        return SamplingParams()
    p = _str_keys(params)
    for name in _UNSUPPORTED_SAMPLING:
        if p.get(name) is not None:
            raise UnsupportedEngineCoreField(f"EngineCoreSamplingParams.{name} is not supported")
    unknown = sorted(set(_extra_args(p)) - {PARALLAX_ROUTING_TABLE_EXTRA_ARG,
                                            PARALLAX_SCHEDULER_REQUEST_ID_EXTRA_ARG})
    if unknown:
        raise UnsupportedEngineCoreField(
            "EngineCoreSamplingParams.extra_args contains unsupported fields: " + ", ".join(unknown))
    top_k = int(p.get("top_k", 0) or 0)
    return SamplingParams(
        max_new_tokens=int(p.get("max_tokens", 128) or 128), min_new_tokens=int(p.get("min_tokens", 0) or 0),
        temperature=float(p.get("temperature", 1.0)), top_p=float(p.get("top_p", 1.0)),
        min_p=float(p.get("min_p", 0.0)), top_k=top_k if top_k > 0 else -1,
        stop_token_ids=[int(t) for t in (p.get("stop_token_ids") or [])],
        ignore_eos=p.get("_eos_token_id") is None,
        repetition_penalty=float(p.get("repetition_penalty", 1.0)),
        presence_penalty=float(p.get("presence_penalty", 0.0)),
        frequency_penalty=float(p.get("frequency_penalty", 0.0)),
    )


def engine_core_request_to_initial_request(request, *, max_sequence_length: Optional[int] = None) -> Request:
    d = decode_engine_core_request(request)
    for name in _UNSUPPORTED_REQUEST:
        if d.get(name) is not None:
            raise UnsupportedEngineCoreField(f"EngineCoreRequest.{name} is not supported")
    mask = d.get("prompt_is_token_ids")
    if mask is not None and not all(bool(x) for x in mask):
        raise UnsupportedEngineCoreField("EngineCoreRequest.prompt_embeds is not supported")
    if d.get("data_parallel_rank") not in (None, 0):
        raise UnsupportedEngineCoreField("EngineCoreRequest.data_parallel_rank is not supported")
    if d.get("abort_immediately"):
        raise UnsupportedEngineCoreField("EngineCoreRequest.abort_immediately is not supported")
    if d.get("prompt_token_ids") is None:
        raise UnsupportedEngineCoreField("EngineCoreRequest.prompt_token_ids is required")
    ids = [int(t) for t in d["prompt_token_ids"]]
    raw = d.get("sampling_params")
    sp = sampling_params_from_engine_core(raw)
    sp.max_new_tokens = max(1, int(sp.max_new_tokens))
    total = len(ids) + sp.max_new_tokens
    if max_sequence_length is not None:
        total = min(total, int(max_sequence_length))
    req = Request(request_id=str(d["request_id"]), input_ids=ids, sampling_params=sp,
                  routing_table=routing_table_from_engine_core_sampling_params(raw),
                  max_total_length=total, return_probs=False,
                  arrival_time=d.get("arrival_time"))
    req.scheduler_request_id = scheduler_request_id_from_sampling_params(raw)
    return req


def make_engine_core_output(*, request_id: str, new_token_ids: Optional[list[int]] = None,
                            finish_reason=None, stop_reason=None) -> list:
    out: list[Any] = [None] * ENGINE_CORE_OUTPUT_FIELD_COUNT
    out[0] = request_id
    out[1] = [int(t) for t in (new_token_ids or [])]
    out[5] = None if finish_reason is None else int(finish_reason)
    out[6] = stop_reason
    out[12] = 0
    return out


def make_engine_core_outputs(outputs: list[list], *, engine_index: int = 0,
                             finished_requests: Optional[Iterable[str]] = None,
                             timestamp: Optional[float] = None) -> list:
    out: list[Any] = [None] * ENGINE_CORE_OUTPUTS_FIELD_COUNT
    out[0] = int(engine_index)
    out[1] = outputs
    out[3] = time.monotonic() if timestamp is None else float(timestamp)
    out[5] = list(finished_requests) if finished_requests is not None else None
    return out


def encode_engine_core_outputs(outputs: list[list], **kw) -> bytes:
    return _pack(make_engine_core_outputs(outputs, **kw))


def finish_reason_of(req: Request) -> Optional[EngineCoreFinishReason]:
    from parallax_b200.engine.request import RequestStatus as S

    return {S.FINISHED_EOS: EngineCoreFinishReason.STOP, S.FINISHED_MAX_LENGTH: EngineCoreFinishReason.LENGTH,
            S.FINISHED_ABORT: EngineCoreFinishReason.ABORT, S.CANCELLED: EngineCoreFinishReason.ABORT,
            S.ERROR: EngineCoreFinishReason.ERROR}.get(req.status)
