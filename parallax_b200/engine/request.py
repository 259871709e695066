"""Request state and sampling parameters.

``Request`` is the first-stage view of a generation request (prompt, outputs, status,
chunked-prefill progress); ``IntermediateRequest`` is the packet that travels between
pipeline stages and between nodes (request id, position, hidden states or the sampled
token, routing table, sampling parameters). Field set and status vocabulary follow
``src/parallax/server/request.py:71-393`` and
``src/parallax/server/sampling/sampling_params.py:8-65``.
"""

from __future__ import annotations

import time
import uuid
from enum import Enum
from typing import Any, Optional


class SamplingParams:
    def __init__(
        self,
        max_new_tokens: int = 128,
        min_new_tokens: int = 0,
        temperature: float = 1.0,
        top_p: float = 1.0,
        min_p: float = 0.0,
        top_k: int = -1,
        stop_token_ids: Optional[list[int]] = None,
        ignore_eos: bool = False,
        stop_strs=None,
        repetition_penalty: float = 1.0,
        presence_penalty: float = 0.0,
        frequency_penalty: float = 0.0,
        json_schema: Optional[str] = None,
        seed: Optional[int] = None,
    ):
        self.max_new_tokens = max_new_tokens
        self.min_new_tokens = min_new_tokens
        self.temperature = temperature
        self.top_p = top_p
        self.min_p = min_p
        self.top_k = top_k
        self.stop_token_ids = set(stop_token_ids) if stop_token_ids else None
        self.ignore_eos = ignore_eos
        self.stop_strs = stop_strs
        self.repetition_penalty = repetition_penalty
        self.presence_penalty = presence_penalty
        self.frequency_penalty = frequency_penalty
        self.json_schema = json_schema
        self.seed = seed
        if self.temperature == 0.0:  # greedy
            self.temperature = 1.0
            self.top_k = 1

    @property
    def is_greedy(self) -> bool:
        return self.top_k == 1

    @property
    def has_penalties(self) -> bool:
        return self.repetition_penalty != 1.0 or self.presence_penalty != 0.0 or self.frequency_penalty != 0.0

    def verify(self) -> None:
        if self.temperature < 0.0:
            raise ValueError(f"temperature must be non-negative, got {self.temperature}.")
        if not 0.0 < self.top_p <= 1.0:
            raise ValueError(f"top_p must be in (0, 1], got {self.top_p}.")
        if not 0.0 <= self.min_p <= 1.0:
            raise ValueError(f"min_p must be in [0, 1], got {self.min_p}.")
        if not -2.0 <= self.frequency_penalty <= 2.0:
            raise ValueError(f"frequency_penalty must be in [-2, 2], got {self.frequency_penalty}.")
        if not -2.0 <= self.presence_penalty <= 2.0:
            raise ValueError(f"presence_penalty must be in [-2, 2], got {self.presence_penalty}.")
        if not 0.0 <= self.repetition_penalty <= 2.0:
            raise ValueError(f"repetition_penalty must be in [0, 2], got {self.repetition_penalty}.")
        if self.top_k < -1 or self.top_k == 0:
            raise ValueError(f"top_k must be -1 (disabled) or >= 1, got {self.top_k}.")
        if self.max_new_tokens < 0 or self.min_new_tokens < 0:
            raise ValueError("max_new_tokens / min_new_tokens must be non-negative.")

    def to_dict(self) -> dict:
        d = dict(self.__dict__)
        if d["stop_token_ids"] is not None:
            d["stop_token_ids"] = sorted(d["stop_token_ids"])
        return d

    @classmethod
    def from_dict(cls, d: dict) -> "SamplingParams":
        sp = cls()
        for k, v in d.items():
            if k == "stop_token_ids" and v is not None:
                v = set(v)
            setattr(sp, k, v)
        return sp


class RequestStatus(Enum):
    PREFILLING = "PREFILLING"
    DECODING = "DECODING"
    FINISHED_EOS = "FINISHED_EOS"
    FINISHED_MAX_LENGTH = "FINISHED_MAX_LENGTH"
    FINISHED_ABORT = "FINISHED_ABORT"
    ERROR = "ERROR"
    CANCELLED = "CANCELLED"


_FINISHED = {
    RequestStatus.FINISHED_EOS,
    RequestStatus.FINISHED_MAX_LENGTH,
    RequestStatus.FINISHED_ABORT,
    RequestStatus.ERROR,
    RequestStatus.CANCELLED,
}


# Stands in ``output_ids`` for a token that has been sampled on the device but not read back yet (the
# engine launches the next step before it reads the previous step's tokens).
PENDING_TOKEN = -1


class Request:
    """Generation request as tracked by the first pipeline stage."""

    def __init__(
        self,
        request_id: Optional[str] = None,
        input_ids: Optional[list[int]] = None,
        sampling_params: Optional[SamplingParams] = None,
        routing_table: Optional[list[str]] = None,
        max_total_length: int = 32768,
        lora_path: Optional[str] = None,
        return_probs: bool = False,
        arrival_time: Optional[float] = None,
    ):
        self.request_id = request_id or str(uuid.uuid4())
        self.rid = self.request_id
        self.input_ids: list[int] = list(input_ids or [])
        self.origin_input_ids = list(self.input_ids)
        self.prompt_len = len(self.input_ids)
        self.output_ids: list[int] = []
        self.output_probs: list[float] = []
        self.sampling_params = sampling_params or SamplingParams()
        self.routing_table = routing_table or []
        self.max_total_length = max_total_length
        self.lora_path = lora_path
        self.return_probs = return_probs
        self.status = RequestStatus.PREFILLING
        self.abort = False
        self.ready_for_next_step = True
        self.arrival_time = arrival_time if arrival_time is not None else time.time()
        self.last_updated_time: Optional[float] = None
        self.first_token_time: Optional[float] = None
        self.finish_time: Optional[float] = None
        # chunked prefill progress: prompt tokens whose KV is computed (or reused from cache)
        self.num_computed_tokens = 0
        self.num_cached_tokens = 0
        self.is_chunked = False
        self.scheduler_request_id: Optional[str] = None

    # ---- derived ----------------------------------------------------------
    @property
    def max_new_tokens(self) -> int:
        return self.sampling_params.max_new_tokens

    @property
    def output_length(self) -> int:
        return len(self.output_ids)

    @property
    def total_length(self) -> int:
        return self.prompt_len + len(self.output_ids)

    @property
    def is_finished(self) -> bool:
        return self.status in _FINISHED

    @property
    def is_prefill(self) -> bool:
        return self.status == RequestStatus.PREFILLING

    @property
    def is_decoding(self) -> bool:
        return self.status == RequestStatus.DECODING

    @property
    def remaining_prefill(self) -> int:
        return self.prompt_len - self.num_computed_tokens

    def update_status(self, status: RequestStatus) -> None:
        self.status = status
        if status in _FINISHED and self.finish_time is None:
            self.finish_time = time.time()

    def commit_new_token(self, token_id: int, prob: Optional[float] = None, now: Optional[float] = None) -> None:
        """Append a sampled token; the first one moves the request to DECODING. ``now``: the caller's
        clock reading when it commits many requests at once."""
        if self.status in _FINISHED:
            return
        self.output_ids.append(int(token_id))
        if prob is not None:
            self.output_probs.append(float(prob))
        if now is None:
            now = time.time()
        if self.first_token_time is None:
            self.first_token_time = now
        if self.status == RequestStatus.PREFILLING:
            self.status = RequestStatus.DECODING
        self.last_updated_time = now

    def penalty_entries(self) -> tuple[list[int], list[int]]:
        """Distinct tokens this request has seen and how often each was GENERATED (0 = prompt only): the
        per-row input of the penalty kernel. Tokens still on the device are not counted."""
        counts: dict[int, int] = {}
        for t in self.output_ids:
            if t != PENDING_TOKEN:
                counts[t] = counts.get(t, 0) + 1
        prompt_only = set(self.input_ids).difference(counts)
        toks = list(counts) + list(prompt_only)
        return toks, list(counts.values()) + [0] * len(prompt_only)

    def reserve_token(self) -> int:
        """Append a placeholder for the token that the step just launched will produce; returns its
        index in ``output_ids``. The request counts as DECODING from here on."""
        self.output_ids.append(PENDING_TOKEN)
        if self.status == RequestStatus.PREFILLING:
            self.status = RequestStatus.DECODING
        return len(self.output_ids) - 1

    def fill_token(self, index: int, token_id: int, prob: Optional[float] = None, now: Optional[float] = None) -> None:
        """The value of a reserved token arrived."""
        self.output_ids[index] = int(token_id)
        if prob is not None:
            self.output_probs.append(float(prob))
        if now is None:
            now = time.time()
        if self.first_token_time is None:
            self.first_token_time = now
        self.last_updated_time = now

    @property
    def all_token_ids(self) -> list[int]:
        return self.input_ids + self.output_ids

    def __repr__(self) -> str:
        return (f"Request({self.request_id}, {self.status.value}, prompt={self.prompt_len}, "
                f"computed={self.num_computed_tokens}, out={len(self.output_ids)})")


InitialRequest = Request


class IntermediateRequest:
    """Stage-to-stage packet. Carries hidden states forward and the sampled token back."""

    def __init__(
        self,
        request_id: str,
        current_position: int,
        status: RequestStatus = RequestStatus.PREFILLING,
        input_ids: Optional[list[int]] = None,
        hidden_states: Any = None,
        next_token_id: Optional[int] = None,
        routing_table: Optional[list[str]] = None,
        sampling_params: Optional[SamplingParams] = None,
        lora_path: Optional[str] = None,
        token_prob: Optional[float] = None,
        return_probs: bool = False,
        is_chunked: bool = False,
        is_last_chunk: bool = True,
        chunk_start: int = 0,
        output_length: int = 0,
    ):
        self.request_id = request_id
        self.rid = request_id
        self.current_position = current_position
        self.status = status
        self.input_ids = input_ids
        self.hidden_states = hidden_states
        self.next_token_id = next_token_id
        self.routing_table = routing_table or []
        self.sampling_params = sampling_params or SamplingParams()
        self.lora_path = lora_path
        self.token_prob = token_prob
        self.return_probs = return_probs
        self.is_chunked = is_chunked
        self.is_last_chunk = is_last_chunk
        self.chunk_start = chunk_start
        self.output_length = output_length
        self.abort = False

    @property
    def is_prefill(self) -> bool:
        return self.status == RequestStatus.PREFILLING

    @property
    def is_decoding(self) -> bool:
        return self.status == RequestStatus.DECODING

    @property
    def is_finished(self) -> bool:
        return self.status in _FINISHED

    @classmethod
    def from_request(cls, req: Request, hidden_states: Any = None, chunk_start: int = 0,
                     num_tokens: Optional[int] = None) -> "IntermediateRequest":
        if req.is_prefill:
            end = chunk_start + (num_tokens if num_tokens is not None else req.prompt_len - chunk_start)
            return cls(req.request_id, end, req.status, input_ids=req.input_ids[:end],
                       hidden_states=hidden_states, routing_table=req.routing_table,
                       sampling_params=req.sampling_params, lora_path=req.lora_path,
                       return_probs=req.return_probs, is_chunked=req.is_chunked,
                       is_last_chunk=end >= req.prompt_len, chunk_start=chunk_start,
                       output_length=req.output_length)
        return cls(req.request_id, req.total_length, req.status, hidden_states=hidden_states,
                   next_token_id=req.output_ids[-1] if req.output_ids else None,
                   routing_table=req.routing_table, sampling_params=req.sampling_params,
                   lora_path=req.lora_path, return_probs=req.return_probs,
                   output_length=req.output_length)
