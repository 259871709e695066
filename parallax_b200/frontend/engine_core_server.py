"""The engine's end of the engine-core wire protocol, and a small client for the frontend's end.

An external HTTP frontend (the reference launches vLLM's Rust one, ``src/parallax/server/vllm_rust_frontend.py``)
owns two ZMQ sockets: a ROUTER on which it sends ``[identity, type, payload]`` request frames and a PULL on which
it reads output frames. The engine connects a DEALER with identity ``00 00`` to the first and a PUSH to the
second, announces itself with a ready message, then turns ADD / ABORT frames into engine requests and streams
every new token back as an ``outputs`` frame (``src/parallax/server/executor/base_executor.py:273-310,456``).

:class:`EngineCoreServer` is that engine side on top of :class:`parallax_b200.engine.service.EngineLoop`;
:class:`EngineCoreClient` is the frontend side, used by the tests and by anyone who wants to drive the engine
from another process without HTTP.
"""

from __future__ import annotations

import logging
import threading
from typing import Optional

import zmq

from parallax_b200.engine.service import EngineLoop, TokenEvent
from parallax_b200.frontend import engine_core_protocol as proto

logger = logging.getLogger(__name__)


class EngineCoreServer:
    def __init__(self, loop: EngineLoop, input_endpoint: str, output_endpoint: str, *, max_model_len: int,
                 dtype: str = "bfloat16", block_size: int = 16, num_gpu_blocks: int = 0):
        self.loop = loop
        self.max_model_len = max_model_len
        self.ctx = zmq.Context.instance()
        self.inp = self.ctx.socket(zmq.DEALER)
        self.inp.setsockopt(zmq.IDENTITY, proto.ENGINE_IDENTITY)
        self.inp.setsockopt(zmq.SNDHWM, 0)
        self.inp.setsockopt(zmq.RCVHWM, 0)
        self.inp.connect(input_endpoint)
        self.out = self.ctx.socket(zmq.PUSH)
        self.out.setsockopt(zmq.SNDHWM, 0)
        self.out.connect(output_endpoint)
        self._out_lock = threading.Lock()
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._ready = proto.engine_core_ready_payload(max_model_len=max_model_len, dtype=dtype, block_size=block_size,
                                                      num_gpu_blocks=num_gpu_blocks)
        prev = loop.on_event

        def on_event(ev: TokenEvent) -> None:
            if prev is not None:
                prev(ev)
            self._send_event(ev)

        loop.on_event = on_event

    # ---- engine -> frontend
    def _send_event(self, ev: TokenEvent) -> None:
        reason = None
        if ev.finished:
            reason = {"FINISHED_EOS": proto.EngineCoreFinishReason.STOP,
                      "FINISHED_MAX_LENGTH": proto.EngineCoreFinishReason.LENGTH,
                      "FINISHED_ABORT": proto.EngineCoreFinishReason.ABORT,
                      "CANCELLED": proto.EngineCoreFinishReason.ABORT}.get(ev.status.value,
                                                                           proto.EngineCoreFinishReason.ERROR)
        out = proto.make_engine_core_output(request_id=ev.request_id,
                                            new_token_ids=[] if ev.token_id is None else [ev.token_id],
                                            finish_reason=reason)
        frame = proto.encode_engine_core_outputs([out], finished_requests=[ev.request_id] if ev.finished else None)
        with self._out_lock:
            self.out.send(frame)

    # ---- frontend -> engine
    def _serve(self) -> None:
        self.inp.send(self._ready)
        poller = zmq.Poller()
        poller.register(self.inp, zmq.POLLIN)
        while not self._stop.is_set():
            if not poller.poll(100):
                continue
            frames = self.inp.recv_multipart()
            if len(frames) < 2:
                continue
            try:
                kind, body = proto.decode_engine_core_frame(frames[0], frames[1])
                if kind == "add":
                    req = proto.engine_core_request_to_initial_request(body, max_sequence_length=self.max_model_len)
                    self.loop.submit(req)
                else:
                    for rid in body:
                        self.loop.abort(rid)
            except Exception as exc:      # a bad frame must not take the engine down
                logger.warning("engine-core frame rejected: %s", exc)
                rid = None
                try:
                    rid = proto.decode_engine_core_request(frames[1]).get("request_id")
                except Exception:
                    pass
                if rid is not None:
                    out = proto.make_engine_core_output(request_id=str(rid), finish_reason=proto.EngineCoreFinishReason.ERROR,
                                                        stop_reason=str(exc))
                    with self._out_lock:
                        self.out.send(proto.encode_engine_core_outputs([out], finished_requests=[str(rid)]))

    def start(self) -> None:
        self._thread = threading.Thread(target=self._serve, name="EngineCoreServer", daemon=True)
        self._thread.start()

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(2.0)
        self.inp.close(0)
        self.out.close(0)


class EngineCoreClient:
    """Frontend side: binds the two endpoints, waits for the engine's ready message, sends requests and reads
    output frames."""

    def __init__(self, input_endpoint: str, output_endpoint: str):
        self.ctx = zmq.Context.instance()
        self.router = self.ctx.socket(zmq.ROUTER)
        self.router.bind(input_endpoint)
        self.pull = self.ctx.socket(zmq.PULL)
        self.pull.bind(output_endpoint)
        self.engine_info: Optional[dict] = None

    def wait_ready(self, timeout_s: float = 30.0) -> dict:
        if not self.router.poll(int(timeout_s * 1000)):
            raise TimeoutError("no engine registered")
        ident, payload = self.router.recv_multipart()
        assert ident == proto.ENGINE_IDENTITY
        self.engine_info = proto._unpack(payload)
        return self.engine_info

    def add(self, request_id: str, prompt_token_ids, sampling_params: dict) -> None:
        fields = {"request_id": request_id, "prompt_token_ids": list(prompt_token_ids), "sampling_params": sampling_params}
        self.router.send_multipart([proto.ENGINE_IDENTITY, proto.REQUEST_TYPE_ADD, proto.encode_engine_core_request(fields)])

    def abort(self, request_ids) -> None:
        self.router.send_multipart([proto.ENGINE_IDENTITY, proto.REQUEST_TYPE_ABORT, proto.encode_engine_core_abort(request_ids)])

    def read(self, timeout_s: float = 30.0) -> Optional[list]:
        """One ``outputs`` frame as a decoded list, or None on timeout."""
        if not self.pull.poll(int(timeout_s * 1000)):
            return None
        return proto._unpack(self.pull.recv())

    def close(self) -> None:
        self.router.close(0)
        self.pull.close(0)
