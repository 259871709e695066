"""Executor of ONE pipeline peer that talks to its neighbours through stage packets.

This is the cross-node path (``parallax join``): a peer owns layers ``[start, end)``; the
first peer owns the request state and the batch scheduler, later peers are driven by the
packets they receive, the last peer samples and sends only the token id back to the first
peer - the protocol of the reference's executor
(``src/parallax/server/executor/base_executor.py:566-769,845-863``,
``src/parallax/server/request.py:268-393``). Packets are :class:`IntermediateRequest`s and
are serialised by :mod:`parallax_b200.p2p.message_util` when they leave the process.

Every peer keeps its own paged KV cache and prefix cache; the prompt token ids travel with
prefill packets so that each peer can publish and match prefixes itself. The first peer
decides how many cached tokens are skipped (``chunk_start``); a later peer that cannot serve
that prefix from its own cache answers with an abort for the request.

Chunked prefill: the first peer re-queues a request for its next chunk as soon as its own
layers are done with the current one, so chunks stream through the stages back to back; the
last peer drops the logits of non-final chunks.
"""

from __future__ import annotations

import logging
from typing import Optional

import torch

from parallax_b200 import ops
from parallax_b200.engine.batch import BatchBuilder
from parallax_b200.engine.engine import Planner
from parallax_b200.engine.request import IntermediateRequest, Request, RequestStatus
from parallax_b200.engine.scheduler import ScheduledSeq
from parallax_b200.engine.worker import StageWorker
from parallax_b200.models.config import ModelConfig

logger = logging.getLogger(__name__)


class PeerExecutor:
    def __init__(self, cfg: ModelConfig, start_layer: int, end_layer: int, device="cpu", dtype=None,
                 node_id: str = "node", page_size: int = 16, num_blocks: Optional[int] = None,
                 kv_fraction: float = 0.8, max_batch_size: int = 8, max_num_tokens_per_batch: int = 16384,
                 micro_batch_ratio: int = 1, chunked_prefill_size: Optional[int] = 1024,
                 enable_prefix_cache: bool = True, max_total_length: int = 32768,
                 request_timeout_s: Optional[float] = 600, eos_token_id=None, seed: int = 0,
                 weights: Optional[dict] = None, shared_state=None, kv_cache_dtype: Optional[str] = None,
                 stage_group=None, lora: Optional[dict] = None):
        """``stage_group`` (:class:`parallax_b200.parallel.peer_group.TPStageGroup`): the node's GPUs run this
        peer's layers tensor-parallel; this process is rank 0 of that group and the group owns the stage worker.
        ``lora``: per-request adapters ``{"max_loaded", "max_rank", "paths": {name: dir}}``; every peer keeps the
        slots of its own layers and loads an adapter when the first packet that names it arrives (the adapter's
        name travels with the packets, as in ``src/parallax/server/request.py:268-393``)."""
        self.cfg, self.node_id = cfg, node_id
        self.device = torch.device(device)
        self.group = stage_group
        # the rotary table covers every position a request may reach, whatever length the checkpoint's
        # config advertises (positions beyond that length are the caller's choice, as with the reference's
        # on-the-fly rotary embedding); a table cut at the advertised length was read out of bounds
        max_positions = max_total_length + 8
        max_requests = max(max_batch_size * 2, 16)
        if cfg.has_linear_layers:
            # recurrent layers keep one state slot per request (the cache manager's row of the request). Prefix
            # reuse would need state snapshots that every peer of a pipeline holds for the same prefixes; peers
            # cache independently, so hybrid models run without the prefix cache here
            enable_prefix_cache = False
        if stage_group is not None:
            self.worker = stage_group.worker
        else:
            self.worker = StageWorker(cfg, start_layer, end_layer, self.device, dtype, page_size, num_blocks=num_blocks,
                                      kv_fraction=kv_fraction, seed=seed, weights=weights, max_positions=max_positions,
                                      kv_cache_dtype=kv_cache_dtype,
                                      num_linear_slots=max_requests if cfg.has_linear_layers else 0)
        self.is_first, self.is_last = self.worker.is_first, self.worker.is_last
        self.planner = Planner(cfg, self.worker.num_blocks, page_size, max_batch_size, max_num_tokens_per_batch,
                               micro_batch_ratio, chunked_prefill_size, enable_prefix_cache, max_total_length,
                               request_timeout_s, eos_token_id, shared_state)
        self.scheduler, self.cache = self.planner.scheduler, self.planner.cache
        self.builder = BatchBuilder(self.device, max_num_tokens_per_batch + max_batch_size, max_batch_size,
                                    self.cache.max_blocks_per_seq)
        self.mirror: dict[str, Request] = {}   # later peers: per-request shadow state
        # JSON-schema constrained requests: the peer that samples (the last one) keeps a matcher per request and
        # picks among the step's candidates; the first peer keeps a twin to know when the document is complete
        self.tokenizer = None                  # anything with token_text(id) and eos_token_ids; set by the node runtime
        self._grammars: dict = {}
        import random as _random

        self._py_rng = _random.Random(seed + 777)
        self.lora = None
        if lora:
            from parallax_b200.loader.lora import LoRAManager, LoRAStack

            if not hasattr(self.worker.model, "lora"):
                raise ValueError("per-request LoRA on a pipeline peer needs a GQA decoder family")
            n_slots = int(lora.get("max_loaded") or 4)
            if stage_group is not None:
                # a tensor-parallel node: the group built a sliced stack on every rank; loads go out as commands
                from parallax_b200.loader.lora import LoRAAdapter

                def load_everywhere(slot, name, path):
                    stage_group.command("lora_load", (int(slot), name, path),
                                        local=lambda: self.worker.model.lora.load(int(slot), LoRAAdapter.load(path, name)))

                self.lora = LoRAManager([], n_slots, lora.get("paths"), on_load=load_everywhere)
            else:
                self.worker.model.lora = LoRAStack(self.worker.model, n_slots, int(lora.get("max_rank") or 64))
                self.lora = LoRAManager([self.worker.model.lora], n_slots, lora.get("paths"))
        self._gen = torch.Generator(device=self.device)
        self._gen.manual_seed(seed + 777)

    # ------------------------------------------------------------------ shared forward
    def _run(self, seqs: list[ScheduledSeq], hidden_of: Optional[dict]):
        """Plan and run one batch. ``hidden_of`` (later peers) maps ``id(seq)`` to that sequence's
        incoming activations: the batch's hidden states are assembled AFTER planning, from the
        sequences that planning kept, so a decode request dropped for lack of KV memory takes its row
        with it instead of shifting every row behind it."""
        on_gpu = self.device.type == "cuda"
        if on_gpu:
            from parallax_b200.ops import cuda as _cuda

            _cuda.raise_if_status(self.device)      # word mirrored after the previous batch
        arrays = self.planner.plan_arrays(seqs)
        if arrays is None:
            return None, None
        hidden = None
        if hidden_of is not None:
            hidden = torch.cat([hidden_of[id(s)] for s in arrays["ordered"]], dim=0)
        extra = None
        if self.lora is not None and any(getattr(s.req, "lora_slot", -1) >= 0 for s in arrays["ordered"]):
            import numpy as np

            rows = np.full(arrays["pos"].shape[0], -1, dtype=np.int32)      # adapter slot of every token row
            o = 0
            for s in arrays["ordered"]:
                rows[o:o + s.num_tokens] = getattr(s.req, "lora_slot", -1)
                o += s.num_tokens
            extra = {"lora_ids": rows}
        if self.group is not None:
            # every rank of the node runs the stage on this plan; rank 0 (here) keeps the result
            out = self.group.forward(arrays, hidden, want_logits=bool(arrays["owners"]),
                                     lora_ids=None if extra is None else extra["lora_ids"])
            if on_gpu:
                _cuda.status_copy_async(self.device)
            return arrays, out
        fb = self.builder.build(arrays["ids"] if self.is_first else None, arrays["pos"], arrays["slots"],
                                arrays["p_q"], arrays["p_ctx"], arrays["p_tables"], arrays["d_ctx"],
                                arrays["d_tables"], arrays["logit_rows"], arrays["seq_rows"], extra=extra)
        with torch.inference_mode():
            if self.is_last:
                h = self.worker.model.embed_tokens(fb) if self.is_first else hidden
                h = self.worker.model.forward_layers(h, fb)
                out = (h, self.worker.model.logits(h, fb) if arrays["owners"] else None)
            else:
                out = (self.worker.run(fb, hidden), None)
        if on_gpu:
            _cuda.status_copy_async(self.device)    # read back with this batch's outputs
        return arrays, out

    def _sample(self, logits: torch.Tensor, owners: list[ScheduledSeq]):
        from parallax_b200.engine.sampling import apply_penalties, build_penalties

        # on the last peer the mirror requests know the prompt; generated tokens arrive with the packets
        logits = apply_penalties(logits, build_penalties([s.req for s in owners]))
        sps = [s.req.sampling_params for s in owners]
        if all(sp.is_greedy for sp in sps):
            ids, lp = ops.argmax(logits, want_logprob=True)
            out = ids.tolist(), lp.exp().tolist()
            self._raise_if_device_error()
            return self._constrain(logits, owners, *out)
        dev = logits.device
        t = torch.tensor([0.0 if sp.is_greedy else sp.temperature for sp in sps], dtype=torch.float32, device=dev)
        k = torch.tensor([sp.top_k if sp.top_k > 0 else 0 for sp in sps], dtype=torch.int32, device=dev)
        p = torch.tensor([sp.top_p for sp in sps], dtype=torch.float32, device=dev)
        mp = torch.tensor([sp.min_p for sp in sps], dtype=torch.float32, device=dev)
        u = torch.rand(len(sps), generator=self._gen, device=dev, dtype=torch.float32)
        ids, pr = ops.sample(logits, t, k, p, mp, u, want_prob=True)
        out = ids.tolist(), pr.tolist()
        self._raise_if_device_error()
        return self._constrain(logits, owners, *out)

    def _constrain(self, logits: torch.Tensor, owners: list[ScheduledSeq], ids: list, probs: list):
        """Rows of requests with a JSON schema: the best candidate (or a draw among the valid ones) whose text
        keeps the request's document valid replaces the sampled token; ``None`` where nothing fits (the request
        ends). The matcher advances with every token picked here: this peer is the only one that samples."""
        if not any(s.req.sampling_params.json_schema for s in owners):
            return ids, probs
        from parallax_b200.engine.structured import JsonSchemaMatcher, TokenChooser

        tok = self.tokenizer
        if tok is None:
            raise RuntimeError("a constrained request reached a peer that has no tokenizer")
        chooser = TokenChooser(tok.token_text, sorted(getattr(tok, "eos_token_ids", ()) or ()))
        for row, s in enumerate(owners):
            sp = s.req.sampling_params
            if not sp.json_schema:
                continue
            g = self._grammars.get(s.req.request_id)
            if g is None:
                g = self._grammars[s.req.request_id] = JsonSchemaMatcher(sp.json_schema)
            choice = chooser.choose(g, logits[row], 0.0 if sp.is_greedy else sp.temperature, self._py_rng)
            if choice is None:
                ids[row] = None
                continue
            text = tok.token_text(int(choice))
            if text and not g.done:
                g.advance(text)
            ids[row] = int(choice)
            probs[row] = float(torch.softmax(logits[row].float(), dim=-1)[int(choice)])
        return ids, probs

    def _raise_if_device_error(self) -> None:
        """After a synchronising read of a batch's outputs: fail the batch if one of its kernels gave up."""
        if self.device.type == "cuda":
            from parallax_b200.ops import cuda as _cuda

            _cuda.raise_if_status(self.device)

    def _hidden_packets(self, arrays, h: torch.Tensor) -> list[IntermediateRequest]:
        """One packet per sequence carrying its slice of the stage output."""
        out, o = [], 0
        for s in arrays["ordered"]:
            n = s.num_tokens
            pk = IntermediateRequest.from_request(s.req, hidden_states=h[o:o + n], chunk_start=s.start,
                                                  num_tokens=n) if s.is_prefill else \
                IntermediateRequest.from_request(s.req, hidden_states=h[o:o + 1])
            if s.is_prefill:
                pk.is_last_chunk = s.produces_token
                pk.is_chunked = s.req.is_chunked
            out.append(pk)
            o += n
        return out

    # ------------------------------------------------------------------ adapters
    def _acquire_lora(self, req: Request) -> None:
        req.lora_slot = getattr(req, "lora_slot", -1)
        if req.lora_path and req.lora_slot < 0:
            if self.lora is None:
                raise ValueError("this node was started without LoRA support (--enable-lora)")
            req.lora_slot = self.lora.acquire(req.lora_path)       # loads the adapter if it is not resident

    def _release_lora(self, req: Optional[Request]) -> None:
        if req is not None and self.lora is not None and getattr(req, "lora_slot", -1) >= 0:
            self.lora.release(req.lora_path)
            req.lora_slot = -1

    # ------------------------------------------------------------------ first peer
    def add_request(self, req: Request) -> None:
        assert self.is_first, "requests enter the pipeline at the first peer"
        req.sampling_params.verify()
        req.max_total_length = min(req.max_total_length, self.planner.max_total_length)
        self._acquire_lora(req)
        req.grammar = None
        if req.sampling_params.json_schema:
            if self.tokenizer is None:
                raise ValueError("json_schema needs a node that knows its tokenizer")
            from parallax_b200.engine.structured import JsonSchemaMatcher

            req.grammar = JsonSchemaMatcher(req.sampling_params.json_schema)
        self.scheduler.enque_request(req)

    def has_work(self) -> bool:
        return self.scheduler.num_queued_requests > 0 or self.scheduler.num_running_requests > 0

    def step_first(self):
        """Form and run one batch on the first peer.

        Returns ``(packets_for_next_peer, events, releases)``: ``events`` are
        ``(request, token or None)`` for requests that progressed or finished locally (single-peer
        pipelines sample here); ``releases`` are request ids every other peer must free."""
        assert self.is_first
        events, releases = [], []
        for req in self.scheduler.get_timed_out_requests():
            req.update_status(RequestStatus.FINISHED_ABORT)
            self._finish_first(req, events, releases)
        seqs = [s for s in self.scheduler.form_batch()]
        for req in self.scheduler.pop_rejected():
            events.append((req, None))
        live = []
        for s in seqs:
            if s.req.abort:
                s.req.update_status(RequestStatus.FINISHED_ABORT)
                self._finish_first(s.req, events, releases)
            else:
                live.append(s)
        if not live:
            return [], events, releases
        arrays, out = self._run(live, None)
        for s in live:
            if s.req.is_finished:
                self._finish_first(s.req, events, releases)
        if arrays is None:
            return [], events, releases
        h, logits = out
        for s in arrays["ordered"]:
            if s.is_prefill:
                s.req.num_computed_tokens = s.start + s.num_tokens
                self.cache.insert_full_blocks_to_cache(s.req.request_id, s.req.num_computed_tokens)
        if self.is_last:
            toks, probs = self._sample(logits, arrays["owners"]) if arrays["owners"] else ([], [])
            idx = {id(s): i for i, s in enumerate(arrays["owners"])}
            for s in arrays["ordered"]:
                i = idx.get(id(s))
                if i is not None and toks[i] is None:          # no token keeps the constrained document valid
                    s.req.update_status(RequestStatus.FINISHED_EOS)
                self._commit(s.req, None if i is None else toks[i], None if i is None else probs[i], events, releases)
            return [], events, releases
        packets = self._hidden_packets(arrays, h)
        for s in arrays["ordered"]:
            if s.is_prefill and not s.produces_token:
                self.scheduler.enque_request(s.req)   # next chunk may start right away
        return packets, events, releases

    def _finish_first(self, req: Request, events, releases) -> None:
        self.scheduler.evict_request(req.request_id)
        self.cache.free_request(req.request_id)
        self._release_lora(req)
        self._grammars.pop(req.request_id, None)
        events.append((req, None))
        releases.append(req.request_id)

    def _commit(self, req: Request, tok, prob, events, releases) -> None:
        if tok is not None:
            req.commit_new_token(int(tok), prob if req.return_probs else None)
            self.cache.update_request_tokens(req.request_id, [int(tok)])
            g = getattr(req, "grammar", None)
            if g is not None and not req.is_finished:
                # the document grows by the token's text; it ends the request once it is complete
                text = self.tokenizer.token_text(int(tok))
                if not text or not g.advance(text) or g.done:
                    req.update_status(RequestStatus.FINISHED_EOS)
        if self.scheduler.check_and_update_request_status(req):
            self.cache.free_request(req.request_id)
            self._release_lora(req)
            self._grammars.pop(req.request_id, None)
            releases.append(req.request_id)
            events.append((req, tok))
        else:
            self.scheduler.enque_request(req)
            if tok is not None:
                events.append((req, tok))

    def receive_tokens(self, packets: list[IntermediateRequest]):
        """First peer: tokens (or aborts) coming back from the last peer."""
        assert self.is_first
        events, releases = [], []
        for pk in packets:
            req = self.scheduler.get_running_request(pk.request_id)
            if req is None:
                continue
            if pk.status == RequestStatus.FINISHED_EOS and pk.next_token_id is None:
                req.update_status(RequestStatus.FINISHED_EOS)       # the sampling peer ended a constrained request
                self._commit(req, None, None, events, releases)
                continue
            if pk.abort or pk.status in (RequestStatus.FINISHED_ABORT, RequestStatus.ERROR):
                if req.num_cached_tokens > 0 and not req.output_ids:
                    # a later peer refused a prompt whose first part this peer skipped as cached: it does not
                    # hold that prefix (any more - it may have restarted). Forget the cached prefixes here, so
                    # that the next request sends whole prompts down the pipeline again.
                    logger.warning("request %s was refused downstream with %d cached prompt tokens: dropping this "
                                   "peer's cached prefixes", req.request_id, req.num_cached_tokens)
                    self.cache.invalidate_prefix_cache()
                req.abort = True
                self._commit(req, None, None, events, releases)
                continue
            self._commit(req, pk.next_token_id, pk.token_prob, events, releases)
        return events, releases

    # ------------------------------------------------------------------ later peers
    def release(self, request_ids) -> None:
        for rid in request_ids:
            self._release_lora(self.mirror.pop(rid, None))
            self._grammars.pop(rid, None)
            self.cache.free_request(rid)

    def _admit_packet(self, pk: IntermediateRequest) -> Optional[ScheduledSeq]:
        rid = pk.request_id
        m = self.mirror.get(rid)
        if pk.is_prefill:
            end = pk.current_position
            ids = list(pk.input_ids or [])
            if m is None:
                m = Request(request_id=rid, input_ids=ids, sampling_params=pk.sampling_params,
                            routing_table=pk.routing_table, return_probs=pk.return_probs,
                            max_total_length=self.planner.max_total_length, lora_path=pk.lora_path)
                ok, matched = self.cache.allocate_request(rid, end, token_ids=ids, namespace=pk.lora_path)
                if not ok or matched < pk.chunk_start:
                    if ok:
                        self.cache.free_request(rid)
                    return None
                try:
                    self._acquire_lora(m)
                except Exception as e:
                    logger.warning("request %s: adapter %r cannot be served here: %s", rid, pk.lora_path, e)
                    self.cache.free_request(rid)
                    return None
                self.mirror[rid] = m
            else:
                m.input_ids, m.prompt_len = ids, len(ids)
                known = self.cache.reqs[rid].tokens
                if known is not None:
                    self.cache.update_request_tokens(rid, ids[len(known):])
                if not self.cache.extend_request(rid, end):
                    return None
            m.is_chunked = pk.is_chunked
            return ScheduledSeq(m, end - pk.chunk_start, pk.chunk_start, True, pk.is_last_chunk)
        if m is None:
            return None
        m.status = RequestStatus.DECODING
        n_out = pk.current_position - m.prompt_len
        m.output_ids = [0] * max(n_out - 1, 0) + [int(pk.next_token_id or 0)]
        return ScheduledSeq(m, 1, pk.current_position - 1, False, True)

    def process_packets(self, packets: list[IntermediateRequest]) -> list[IntermediateRequest]:
        """Run this peer's layers on a batch of incoming packets.

        Returns hidden-state packets for the next peer, or (on the last peer) token packets for
        the first peer. Requests this peer cannot serve come back as abort packets."""
        assert not self.is_first
        out: list[IntermediateRequest] = []
        seqs = []
        for pk in packets:
            if pk.abort or pk.is_finished:
                self.release([pk.request_id])
                continue
            s = self._admit_packet(pk)
            if s is None:
                bad = IntermediateRequest(pk.request_id, pk.current_position, RequestStatus.FINISHED_ABORT,
                                          routing_table=pk.routing_table)
                bad.abort = True
                out.append(bad)
                self.release([pk.request_id])
                continue
            seqs.append((s, pk))
        if not seqs:
            return out
        # plan order is prefill first, then decode: order the hidden states the same way
        seqs.sort(key=lambda sp: 0 if sp[0].is_prefill else 1)
        hidden_of = {id(s): pk.hidden_states.to(device=self.device, dtype=self.worker.dtype) for s, pk in seqs}
        arrays, res = self._run([s for s, _ in seqs], hidden_of)
        for s, pk in seqs:
            if s.req.is_finished:   # KV exhausted while appending a decode slot
                bad = IntermediateRequest(pk.request_id, pk.current_position, RequestStatus.FINISHED_ABORT,
                                          routing_table=pk.routing_table)
                bad.abort = True
                out.append(bad)
                self.release([pk.request_id])
        if arrays is None:
            return out
        h, logits = res
        for s in arrays["ordered"]:
            if s.is_prefill:
                self.cache.insert_full_blocks_to_cache(s.req.request_id, s.start + s.num_tokens)
        if not self.is_last:
            return out + self._hidden_packets(arrays, h)
        if arrays["owners"]:
            toks, probs = self._sample(logits, arrays["owners"])
            for s, t, p in zip(arrays["owners"], toks, probs):
                r = s.req
                if t is None:      # no token keeps the constrained document valid: the request ends with what it has
                    out.append(IntermediateRequest(r.request_id, r.total_length, RequestStatus.FINISHED_EOS,
                                                   routing_table=r.routing_table, sampling_params=r.sampling_params))
                    continue
                out.append(IntermediateRequest(r.request_id, r.total_length + 1, RequestStatus.DECODING,
                                               next_token_id=int(t), routing_table=r.routing_table,
                                               sampling_params=r.sampling_params, token_prob=float(p),
                                               return_probs=r.return_probs))
        return out
