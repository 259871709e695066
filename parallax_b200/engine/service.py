"""Engine run loop in a background thread with per-request event streams.

This is the serving-side wrapper around :class:`Engine.step`: it accepts requests and aborts
from any thread, keeps stepping while there is work, pushes ``(token, finished)`` events to
each request's queue, and feeds the node metrics (in-flight requests, EWMA per-layer
latency) that the cluster heartbeat reports. It plays the role of the reference's executor
``run_loop`` (``src/parallax/server/executor/base_executor.py:634-769``): receive, admit,
time out, batch, forward, emit outputs, release.
"""

from __future__ import annotations

import logging
import queue
import threading
import time
from dataclasses import dataclass
from typing import Callable, Optional

from parallax_b200.engine.request import Request, RequestStatus

logger = logging.getLogger(__name__)


@dataclass
class TokenEvent:
    request_id: str
    token_id: Optional[int]
    finished: bool
    status: RequestStatus
    prob: Optional[float] = None
    error: Optional[str] = None


class EngineLoop:
    def __init__(self, engine, shared_state=None, idle_sleep_s: float = 0.002,
                 on_event: Optional[Callable[[TokenEvent], None]] = None):
        self.engine = engine
        self.shared_state = shared_state
        self.idle_sleep_s = idle_sleep_s
        self.on_event = on_event
        self._inbox: "queue.Queue[tuple[str, object]]" = queue.Queue()
        self._streams: dict[str, "queue.Queue[TokenEvent]"] = {}
        self._lock = threading.Lock()
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self.steps = 0
        self.errors = 0
        self._reported = -1          # 0 once the idle load has been written to the shared metrics

    # ---- client side (any thread)
    def submit(self, req: Request) -> "queue.Queue[TokenEvent]":
        q: "queue.Queue[TokenEvent]" = queue.Queue()
        if self._stop.is_set():
            q.put(TokenEvent(req.request_id, None, True, RequestStatus.ERROR, error="the engine stopped serving"))
            return q
        with self._lock:
            self._streams[req.request_id] = q
        self._inbox.put(("add", req))
        return q

    def abort(self, request_id: str) -> None:
        self._inbox.put(("abort", request_id))

    def call(self, fn):
        """Run ``fn()`` on the engine thread between two steps (weight refit, cache maintenance). Returns a
        ``concurrent.futures.Future`` with its result."""
        import concurrent.futures

        fut: "concurrent.futures.Future" = concurrent.futures.Future()
        self._inbox.put(("call", (fn, fut)))
        return fut

    def start(self) -> None:
        if self._thread is None:
            self._stop.clear()
            self._thread = threading.Thread(target=self._run, name="EngineLoop", daemon=True)
            self._thread.start()

    def stop(self, timeout: float = 5.0) -> None:
        """Stop stepping and end every open stream with an error event, so that nobody waits for tokens that will
        never come; requests submitted afterwards are refused the same way."""
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout)
            self._thread = None
        with self._lock:
            open_streams, self._streams = self._streams, {}
        for rid, q in open_streams.items():
            q.put(TokenEvent(rid, None, True, RequestStatus.ERROR, error="the engine stopped serving"))

    @property
    def num_inflight(self) -> int:
        with self._lock:
            return len(self._streams)

    # ---- engine thread
    def _emit(self, ev: TokenEvent) -> None:
        with self._lock:
            q = self._streams.get(ev.request_id)
            if ev.finished:
                self._streams.pop(ev.request_id, None)
        if q is not None:
            q.put(ev)
        if self.on_event is not None:
            self.on_event(ev)

    def _drain_inbox(self) -> None:
        while True:
            try:
                kind, payload = self._inbox.get_nowait()
            except queue.Empty:
                return
            if kind == "add":
                req: Request = payload  # type: ignore[assignment]
                try:
                    self.engine.add_request(req)
                except Exception as exc:  # invalid sampling params etc.
                    req.update_status(RequestStatus.ERROR)
                    self._emit(TokenEvent(req.request_id, None, True, req.status, error=str(exc)))
            elif kind == "call":
                fn, fut = payload
                try:
                    fut.set_result(fn())
                except BaseException as exc:
                    fut.set_exception(exc)
            else:
                gone = self.engine.abort_request(str(payload))
                if gone is not None:     # cancelled before it ever ran: close its stream here
                    self._emit(TokenEvent(gone.request_id, None, True, gone.status))

    def _fail_batch(self, exc: Exception) -> None:
        """A failed forward pass releases every running request with an ERROR event."""
        self.errors += 1
        logger.exception("engine step failed: %s", exc)
        sched = self.engine.scheduler
        for req in list(sched.running_requests()):
            req.update_status(RequestStatus.ERROR)
            sched.evict_request(req.request_id)
            self.engine.cache.free_request(req.request_id)
            self._emit(TokenEvent(req.request_id, None, True, req.status, error=str(exc)))

    def _run(self) -> None:
        eng = self.engine
        num_layers = sum(s.end_layer - s.start_layer for s in eng.stages) or 1
        while not self._stop.is_set():
            self._drain_inbox()
            if not eng.has_work():
                if self.shared_state is not None and self._reported != 0:
                    try:        # the reported load follows the engine to idle (see the peer loop)
                        self.shared_state.update_metrics(current_requests=0)
                        self._reported = 0
                    except Exception:
                        pass
                time.sleep(self.idle_sleep_s)
                continue
            self._reported = -1
            t0 = time.perf_counter()
            try:
                results = eng.step()
            except Exception as exc:
                self._fail_batch(exc)
                continue
            dt_ms = (time.perf_counter() - t0) * 1e3
            self.steps += 1
            for req, tok in results:
                prob = req.output_probs[-1] if (tok is not None and req.output_probs) else None
                self._emit(TokenEvent(req.request_id, tok, req.is_finished, req.status, prob=prob))
            if self.shared_state is not None and results:
                try:
                    self.shared_state.update_metrics(current_requests=eng.scheduler.num_running_requests,
                                                     layer_latency_ms_sample=dt_ms / num_layers)
                except Exception:
                    pass
