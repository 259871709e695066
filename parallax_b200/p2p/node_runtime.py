"""Runtime of a cluster worker node: peer executor + packet endpoints + (first peer) frontend.

One ``NodeRuntime`` serves one layer allocation. It owns a :class:`PeerExecutor`, a run thread
and an HTTP app with

* ``POST /pp_forward``  - ForwardRequest message from the previous peer (hidden states) or, on
                          the first peer, from the last peer (sampled tokens);
* ``POST /pp_abort``    - request ids to release;
* the OpenAI endpoints when this node hosts layer 0.

The run thread is the counterpart of the reference's executor loop for non-standalone nodes
(``src/parallax/server/executor/base_executor.py:634-769``) and of its P2P sender
(``src/parallax/p2p/server.py:628-749``).
"""

from __future__ import annotations

import logging
import queue
import threading
import time
from typing import Optional

from fastapi import FastAPI
from fastapi import Request as HttpRequest

from parallax_b200.engine.request import Request, RequestStatus
from parallax_b200.engine.service import TokenEvent

logger = logging.getLogger(__name__)


class PeerLoop:
    """Drives a PeerExecutor; exposes the EngineLoop interface (submit / abort) on the first peer."""

    def __init__(self, peer, transport, shared_state=None, idle_sleep_s: float = 0.002):
        self.peer, self.transport, self.state = peer, transport, shared_state
        self.idle_sleep_s = idle_sleep_s
        self._inbox: "queue.Queue[tuple[str, object]]" = queue.Queue()
        self._streams: dict[str, "queue.Queue[TokenEvent]"] = {}
        self._lock = threading.Lock()
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self.steps = 0
        self.default_route = None       # callable -> routing table for requests that arrive without one
        self._reported = -1             # request count last written to the shared metrics

    # ---- frontend side
    def submit(self, req: Request):
        q: "queue.Queue[TokenEvent]" = queue.Queue()
        if self._stop.is_set():
            q.put(TokenEvent(req.request_id, None, True, RequestStatus.ERROR,
                             error="the node stopped serving (shutdown or reload)"))
            return q
        with self._lock:
            self._streams[req.request_id] = q
        if not req.routing_table and self.default_route is not None:
            table = self.default_route()       # no scheduler: peers chained by their layer ranges
            if table is None:
                raise RuntimeError("no chain of peers covers every layer yet; start the missing nodes")
            req.routing_table = list(table)
        if not req.routing_table:
            req.routing_table = [self.peer.node_id]
        self._inbox.put(("add", req))
        return q

    def abort(self, request_id: str) -> None:
        self._inbox.put(("abort", request_id))

    @property
    def num_inflight(self) -> int:
        with self._lock:
            return len(self._streams)

    # ---- network side
    def on_packets(self, packets) -> None:
        self._inbox.put(("packets", packets))

    def on_abort(self, request_ids) -> None:
        self._inbox.put(("release", list(request_ids)))

    def start(self) -> None:
        self._thread = threading.Thread(target=self._run, name="PeerLoop", daemon=True)
        self._thread.start()

    def stop(self) -> None:
        """Stop stepping and end every open stream with an error event: a client whose request was in flight (or
        arrived while the node was going down, e.g. for a new layer allocation) gets an answer instead of waiting
        for one that will never come. Requests submitted after this are refused the same way."""
        self._stop.set()
        if self._thread is not None:
            self._thread.join(5.0)
        with self._lock:
            open_streams, self._streams = self._streams, {}
        for rid, q in open_streams.items():
            q.put(TokenEvent(rid, None, True, RequestStatus.ERROR, error="the node stopped serving (shutdown or reload)"))

    # ---- loop
    def _emit(self, req: Request, tok) -> None:
        ev = TokenEvent(req.request_id, tok, req.is_finished, req.status,
                        prob=req.output_probs[-1] if (tok is not None and req.output_probs) else None)
        with self._lock:
            q = self._streams.get(req.request_id)
            if ev.finished:
                self._streams.pop(req.request_id, None)
        if q is not None:
            q.put(ev)

    def _broadcast_release(self, releases, tables: dict) -> None:
        for rid in releases:
            table = tables.pop(rid, None)
            if table and len(table) > 1:
                self.transport.send_abort([rid], table, self.peer.node_id)

    def _forward(self, packets, tables: dict) -> None:
        """Hand packets to their next hops. What cannot be delivered (the peer died or is unknown) ends its request
        here: the first peer fails it towards the client and releases it everywhere; a later peer frees its share
        and tells the first peer, which does the rest."""
        lost = self.transport.send_forward(packets, self.peer.node_id)
        if not lost:
            return
        peer = self.peer
        if peer.is_first:
            releases = []
            for pk in lost:
                req = peer.scheduler.get_running_request(pk.request_id)
                if req is None or req.is_finished:
                    continue
                req.update_status(RequestStatus.ERROR)
                peer.scheduler.evict_request(req.request_id)
                peer.cache.free_request(req.request_id)
                self._emit(req, None)
                releases.append(req.request_id)
            self._broadcast_release(releases, tables)
            return
        from parallax_b200.engine.request import IntermediateRequest

        for pk in lost:
            peer.release([pk.request_id])
            table = pk.routing_table or []
            if table and table[0] != peer.node_id:
                bad = IntermediateRequest(pk.request_id, pk.current_position, RequestStatus.FINISHED_ABORT, routing_table=table)
                bad.abort = True
                self.transport.send_to(table[0], [bad])

    def _run(self) -> None:
        peer = self.peer
        tables: dict[str, list[str]] = {}
        n_layers = peer.worker.end_layer - peer.worker.start_layer
        while not self._stop.is_set():
            busy = False
            while True:
                try:
                    kind, payload = self._inbox.get_nowait()
                except queue.Empty:
                    break
                busy = True
                try:
                    if kind == "add":
                        req: Request = payload  # type: ignore[assignment]
                        tables[req.request_id] = list(req.routing_table)
                        try:
                            peer.add_request(req)
                        except Exception as exc:
                            req.update_status(RequestStatus.ERROR)
                            self._emit(req, None)
                            logger.warning("rejected request %s: %s", req.request_id, exc)
                    elif kind == "abort":
                        try:
                            gone = peer.scheduler.cancel_request(str(payload))
                            if gone is not None:       # cancelled before it ever ran: close its stream here
                                self._emit(gone, None)
                        except ValueError:
                            pass
                    elif kind == "release":
                        peer.release(payload)
                    elif kind == "packets":
                        if peer.is_first:
                            events, releases = peer.receive_tokens(payload)
                            for req, tok in events:
                                self._emit(req, tok)
                            self._broadcast_release(releases, tables)
                        else:
                            t0 = time.perf_counter()
                            out = peer.process_packets(payload)
                            self.steps += 1
                            if out:
                                self._forward(out, tables)
                            if self.state is not None:
                                self.state.update_metrics(current_requests=len(peer.mirror),
                                                          layer_latency_ms_sample=(time.perf_counter() - t0) * 1e3 / n_layers)
                except Exception as exc:
                    logger.exception("peer loop error: %s", exc)
            if peer.is_first and peer.has_work():
                busy = True
                t0 = time.perf_counter()
                try:
                    packets, events, releases = peer.step_first()
                except Exception as exc:
                    logger.exception("first-peer step failed: %s", exc)
                    for req in list(peer.scheduler.running_requests()):
                        req.update_status(RequestStatus.ERROR)
                        peer.scheduler.evict_request(req.request_id)
                        peer.cache.free_request(req.request_id)
                        self._emit(req, None)
                    continue
                self.steps += 1
                for req, tok in events:
                    self._emit(req, tok)
                self._broadcast_release(releases, tables)
                if packets:
                    self._forward(packets, tables)
                if self.state is not None and (packets or events):
                    self.state.update_metrics(current_requests=peer.scheduler.num_running_requests,
                                              layer_latency_ms_sample=(time.perf_counter() - t0) * 1e3 / n_layers)
            # the load this node reports with its heartbeats must follow the requests it holds, also when the last
            # ones end without another step (a count left over from a busy moment made the scheduler answer 429)
            holding = peer.scheduler.num_running_requests + peer.scheduler.num_queued_requests if peer.is_first \
                else len(peer.mirror)
            if self.state is not None and holding != self._reported:
                try:
                    self.state.update_metrics(current_requests=holding)
                    self._reported = holding
                except Exception:
                    pass
            if not busy:
                time.sleep(self.idle_sleep_s)


def create_peer_app(loop: PeerLoop, tokenizer=None, model_name: str = "", max_model_len: int = 32768):
    from parallax_b200.p2p.message_util import proto_to_abort_request, proto_to_request

    if loop.peer.is_first and tokenizer is not None:
        from parallax_b200.frontend.openai_api import create_app

        app = create_app(loop, tokenizer, model_name, max_model_len)
    else:
        app = FastAPI(title="parallax_b200 peer")

        @app.get("/health")
        async def health():
            return {"status": "ok", "steps": loop.steps}

    @app.get("/peer/stats")
    async def peer_stats():
        """What this peer currently holds: requests in its scheduler, shadow requests of later peers, requests with
        KV memory, open client streams, steps run."""
        p = loop.peer
        return {"node_id": p.node_id, "layers": [p.worker.start_layer, p.worker.end_layer], "steps": loop.steps,
                "running": p.scheduler.num_running_requests + p.scheduler.num_queued_requests, "mirror": len(p.mirror),
                "kv_requests": len(p.cache.reqs), "free_blocks": p.cache.num_free_blocks(), "streams": loop.num_inflight}

    @app.post("/pp_forward")
    async def pp_forward(req: HttpRequest):
        loop.on_packets(proto_to_request(await req.body()))
        return {"ok": True}

    @app.post("/pp_abort")
    async def pp_abort(req: HttpRequest):
        loop.on_abort(proto_to_abort_request(await req.body()))
        return {"ok": True}

    return app


class NodeRuntime:
    def __init__(self, args, agent, state, model_name: str, start_layer: int, end_layer: int):
        import torch

        from parallax_b200.engine.peer import PeerExecutor
        from parallax_b200.frontend.tokenizer import TokenizerWrapper
        from parallax_b200.launch import _lora_spec, resolve_model, serve_http
        from parallax_b200.p2p.server import PeerTransport

        self.args, self.agent, self.state = args, agent, state
        args.model_path = args.model_path or model_name
        args.start_layer, args.end_layer = start_layer, end_layer
        cfg, loader, name, path = resolve_model(args)
        device = "cuda:0" if torch.cuda.is_available() else "cpu"
        self.group, self._followers = None, []
        tp = int(getattr(args, "tp_size", 1) or 1)
        if tp > 1:
            # the node's GPUs run this peer's layers tensor-parallel: this process is rank 0, the others follow
            from parallax_b200.parallel.peer_group import launch_followers

            spec = dict(model_path=path, model_name=name.split("/")[-1], start_layer=start_layer, end_layer=end_layer,
                        device_type="cuda" if device != "cpu" else "cpu",
                        dtype=args.dtype if args.dtype in ("bfloat16", "float16") else "bfloat16",
                        page_size=args.kv_block_size, kv_fraction=args.kv_cache_memory_fraction,
                        kv_cache_dtype=getattr(args, "kv_cache_dtype", None), max_batch_size=args.max_batch_size,
                        max_num_tokens_per_batch=args.max_num_tokens_per_batch, max_total_length=args.max_sequence_length,
                        num_blocks=None if device != "cpu" else 1024, log_level=args.log_level, lora=_lora_spec(args))
            self.group, self._followers = launch_followers(spec, tp)
        weights = loader.load_weights("cpu", None) if (loader is not None and self.group is None) else None
        self.peer = PeerExecutor(cfg, start_layer, end_layer, device=device, node_id=agent.node_id,
                                 stage_group=self.group,
                                 page_size=args.kv_block_size, kv_fraction=args.kv_cache_memory_fraction,
                                 kv_cache_dtype=getattr(args, "kv_cache_dtype", None),
                                 max_batch_size=args.max_batch_size,
                                 max_num_tokens_per_batch=args.max_num_tokens_per_batch,
                                 micro_batch_ratio=args.micro_batch_ratio,
                                 chunked_prefill_size=args.chunked_prefill_size,
                                 enable_prefix_cache=args.enable_prefix_cache,
                                 max_total_length=args.max_sequence_length,
                                 request_timeout_s=args.request_timeout_s, weights=weights, shared_state=state,
                                 num_blocks=(self.group.num_blocks if self.group is not None
                                             else (None if device != "cpu" else 1024)),
                                 lora=_lora_spec(args))
        self.peer_urls: dict[str, str] = {}

        def resolve(node_id: str):
            if node_id not in self.peer_urls:
                try:
                    self.peer_urls.update(agent.scheduler.node_addresses())
                except Exception as e:
                    logger.warning("could not fetch peer addresses: %s", e)
            return self.peer_urls.get(node_id)

        self.loop = PeerLoop(self.peer, PeerTransport(resolve, notify_url=args.notify_url), state)
        tok = TokenizerWrapper.from_pretrained(path, vocab_size=cfg.vocab_size) if self.peer.is_first else None
        from parallax_b200.frontend.tokenizer import LazyTokenizer

        # constrained decoding turns token ids into text where tokens are sampled (the last peer) and where the
        # document's end is noticed (the first peer)
        self.peer.tokenizer = tok if tok is not None else LazyTokenizer(path, cfg.vocab_size)
        self.app = create_peer_app(self.loop, tok, name, args.max_sequence_length)

        @self.app.post("/peers")
        async def set_peers(req: HttpRequest):
            self.peer_urls.update(await req.json())
            return {"ok": True}

        static = getattr(agent, "peers", None)
        if static is not None:
            # no scheduler: this node tells others who it is, and the first node routes by layer range
            @self.app.get("/peer/info")
            async def peer_info():
                return static.describe()

            if self.peer.is_first:
                self.loop.default_route = lambda: static.route(cfg.num_hidden_layers)

        self.loop.start()
        self.server, self.thread = serve_http(self.app, args.host, args.port, args.log_level)

    def apply_refit(self, refit: dict) -> int:
        """Apply a weight-refit request whose blocks are readable files (``paths``: cid -> file); on a
        tensor-parallel node every rank applies it to its own slices."""
        from parallax_b200.utils.weight_refit import apply_refit_to_stage

        try:
            if self.group is not None:
                return self.group.command("refit", refit,
                                          local=lambda: apply_refit_to_stage(self.peer.worker, self.peer.cfg, refit))
            return apply_refit_to_stage(self.peer.worker, self.peer.cfg, refit)
        finally:
            # K/V pages cached for prefix reuse were computed with the old weights
            self.peer.cache.invalidate_prefix_cache()

    def serve_until_allocation_changes(self, poll_s: float = 0.5) -> None:
        while not self.state.get_layer_allocation_changed() and self.thread.is_alive():
            time.sleep(poll_s)

    def shutdown(self) -> None:
        self.server.should_exit = True
        self.loop.stop()
        self.thread.join(5.0)
        if self.group is not None:
            from parallax_b200.parallel.peer_group import stop_followers

            stop_followers(self.group, self._followers)
            self.group = None
