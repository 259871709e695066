"""Multi-GPU engine inside one box: pipeline stages x lanes, one process per GPU. The lanes of a stage
are either tensor-parallel ranks (one batch, sharded weights) or expert-parallel ranks with
data-parallel attention (every lane runs its own requests with the whole attention stack and a slice
of the experts; the MoE layers exchange token rows over NVLink peer memory).

Rank layout: ``rank = pp_rank * lanes + lane``. Rank 0 owns the scheduler and the logical KV
plan; every step it publishes the packed step inputs (a few hundred KB of indices) to all
ranks through a shared-memory ring, so that every rank can enqueue its kernels without waiting
on a device-to-host copy. Activations move stage to stage with NCCL point-to-point on NVLink -
each tensor-parallel rank sends its own row shard to its counterpart in the next stage - and
only the sampled token ids travel back to rank 0.

Every hop has a two-rank communicator of its own (forward hops and the token return never
queue behind one another), receives are posted on a side stream into a ring of buffers as soon
as the plan is known, and the compute stream only waits for the event that marks the arrival.
Several micro-batches are kept in flight (``pp`` by default): rank 0 issues plan k+1 before it
reads the tokens of plan k. On rank 0 the stage's kernel launches run in a thread of their own,
so planning and committing micro-batches overlaps with enqueuing the stage's work.

This replaces the reference's stage transport (hidden states -> safetensors bytes -> protobuf
-> ZMQ -> libp2p RPC -> ZMQ, with a GPU<->CPU copy on every hop;
``src/parallax/p2p/message_util.py:202-219``, ``src/parallax/p2p/server.py:628-711``) for the
case where all stages live on one NVSwitch domain.
"""

from __future__ import annotations

import logging
import os
import queue
import threading
import time
from collections import deque
from dataclasses import dataclass
from typing import Optional

import numpy as np
import torch
import torch.distributed as dist

from parallax_b200 import ops
from parallax_b200.engine.batch import BatchBuilder
from parallax_b200.engine.engine import Planner
from parallax_b200.engine.request import Request, RequestStatus
from parallax_b200.engine.worker import StageWorker
from parallax_b200.models.config import ModelConfig
from parallax_b200.parallel.tp_comm import CollectiveTPComm, FusedTPComm

logger = logging.getLogger(__name__)


def _ret_len(lane_plan: dict) -> int:
    """Length of the int32 message a sampling rank returns for one lane plan."""
    n = lane_plan["n_logits"]
    return n + 1 + (n if lane_plan.get("want_prob") else 0)


def cu_launch_count() -> int:
    from parallax_b200.ops import cuda as cu

    return cu.launch_count


def split_layers(num_layers: int, pp: int) -> list[tuple[int, int]]:
    """Contiguous split, as even as the layer count allows (what water-filling yields for identical
    GPUs). The remainder layers go to the stages in the middle: the first stage also hosts the
    scheduler and the embedding, the last one the lm_head and the sampler."""
    base, rem = divmod(num_layers, pp)
    extra = [0] * pp
    order = list(range(1, pp - 1)) + [0, pp - 1] if pp > 2 else list(range(pp))
    for i in order[:rem]:
        extra[i] = 1
    out, s = [], 0
    for i in range(pp):
        n = base + extra[i]
        out.append((s, s + n))
        s += n
    return out


@dataclass
class Topology:
    world: int
    rank: int
    pp: int
    tp: int
    ep: int = 1

    @property
    def lanes(self) -> int:
        return self.tp * self.ep

    @property
    def pp_rank(self) -> int:
        return self.rank // self.lanes

    @property
    def lane(self) -> int:
        return self.rank % self.lanes

    @property
    def tp_rank(self) -> int:
        return self.lane if self.tp > 1 else 0

    @property
    def ep_rank(self) -> int:
        return self.lane if self.ep > 1 else 0

    @property
    def is_first_stage(self) -> bool:
        return self.pp_rank == 0

    @property
    def is_last_stage(self) -> bool:
        return self.pp_rank == self.pp - 1

    @property
    def last_stage_root(self) -> int:
        return (self.pp - 1) * self.lanes

    @property
    def token_senders(self) -> list[int]:
        """Ranks that sample and return tokens to rank 0: the first lane of the last stage with tensor
        parallelism (all its lanes hold the same logits), every lane of the last stage with expert
        parallelism (each lane runs its own requests)."""
        if self.ep > 1:
            return [self.last_stage_root + l for l in range(self.lanes)]
        return [self.last_stage_root]


class _RecvSlot:
    """One buffer of the receive ring and the event after which it may be overwritten."""

    __slots__ = ("buf", "free")

    def __init__(self):
        self.buf: Optional[torch.Tensor] = None
        self.free = None


class _SchedulerGroup:
    """The schedulers of all expert-parallel lanes behind the few calls a serving loop makes."""

    def __init__(self, scheds):
        self.scheds = scheds

    @property
    def num_running_requests(self) -> int:
        return sum(s.num_running_requests for s in self.scheds)

    @property
    def num_queued_requests(self) -> int:
        return sum(s.num_queued_requests for s in self.scheds)

    def running_requests(self):
        return [r for s in self.scheds for r in s.running_requests()]

    def evict_request(self, rid: str):
        for s in self.scheds:
            r = s.evict_request(rid)
            if r is not None:
                return r
        return None


class _CacheGroup:
    def __init__(self, caches):
        self.caches = caches

    def free_request(self, rid: str) -> None:
        for c in self.caches:
            if c.has_request(rid):
                c.free_request(rid)


class DistEngine:
    def __init__(self, cfg: ModelConfig, pp: int, tp: int, device, dtype=None, page_size: int = 16,
                 num_blocks: Optional[int] = None, kv_fraction: float = 0.85, max_batch_size: int = 8,
                 max_num_tokens_per_batch: int = 16384, micro_batch_ratio: Optional[int] = None,
                 chunked_prefill_size: Optional[int] = 1024, max_prefill_tokens_per_batch: Optional[int] = None,
                 enable_prefix_cache: bool = True,
                 max_total_length: int = 32768, request_timeout_s: Optional[float] = 600, eos_token_id=None,
                 seed: int = 0, weights: Optional[dict] = None, fused: Optional[bool] = None,
                 max_in_flight: Optional[int] = None, weights_prefiltered: bool = False,
                 liveness_timeout_s: float = 10.0, step_timeout_s: float = 600.0, align_rows: int = 0,
                 executor_thread: Optional[bool] = None, ep: int = 1, ep_local_init: Optional[bool] = None,
                 kv_cache_dtype: Optional[str] = None, linear_prefix_slots: Optional[int] = None,
                 lora: Optional[dict] = None, tokenizer=None):
        assert dist.is_initialized(), "init the default process group first (nccl on GPUs, gloo on CPU)"
        self.cfg = cfg
        self.device = torch.device(device)
        world, rank = dist.get_world_size(), dist.get_rank()
        assert tp == 1 or ep == 1, "a stage's lanes are either tensor-parallel or expert-parallel"
        assert world == pp * tp * ep, f"world size {world} != pp*tp*ep = {pp * tp * ep}"
        self.topo = topo = Topology(world, rank, pp, tp, ep)
        lanes = topo.lanes
        on_gpu = self.device.type == "cuda"
        data_backend = "nccl" if on_gpu else "gloo"
        # ---- groups (every rank creates every group, in the same order)
        self.ctrl = dist.new_group(list(range(world)), backend="gloo")
        # one two-rank communicator per stage hop and tensor-parallel lane, one for the token return
        self.hop_in = self.hop_out = None
        for s in range(pp - 1):
            for t in range(lanes):
                a, b = s * lanes + t, (s + 1) * lanes + t
                g = dist.new_group([a, b], backend=data_backend)
                if rank == a:
                    self.hop_out = g
                elif rank == b:
                    self.hop_in = g
        self.ret: dict = {}          # token-return communicators: sender rank -> group (on rank 0 and on the sender)
        for snd in topo.token_senders:
            if snd != 0:
                g = dist.new_group([0, snd], backend=data_backend)
                if rank in (0, snd):
                    self.ret[snd] = g
        self.tp_group = self.ep_group = None
        for s in range(pp if lanes > 1 else 0):
            g = dist.new_group(list(range(s * lanes, (s + 1) * lanes)), backend=data_backend)
            if s == topo.pp_rank:
                if tp > 1:
                    self.tp_group = g
                else:
                    self.ep_group = g
        self.max_in_flight = max_in_flight or pp
        # ---- step plans travel through shared memory (all ranks live on one box); the name is agreed once
        from parallax_b200.parallel.ctrl_channel import CtrlChannel

        max_blocks = (max_total_length + page_size - 1) // page_size + 1
        ratio = micro_batch_ratio or pp
        # expert-parallel lanes split the requests and the per-step token budget among them
        self.n_plans = ep
        lane_batch = -(-max_batch_size // ep)
        lane_tokens = max(-(-max_num_tokens_per_batch // ep), lane_batch + 256) if ep > 1 else max_num_tokens_per_batch
        micro_seqs = max(1, max_batch_size // max(1, ratio))
        # the largest plan: ids, positions (4 B) and slots (8 B) per token, one block table row per sequence
        slot_bytes = 16 * (ep * lane_tokens + max_batch_size) + 4 * micro_seqs * (max_blocks + 8) + (64 << 10)
        slot_bytes = max(1 << 18, (slot_bytes + 4095) // 4096 * 4096)
        n_slots = max(8, self.max_in_flight + 6)
        box = [None]
        if rank == 0:
            box[0] = f"pxl_ctrl_{os.getpid()}_{int(time.time() * 1e3) % 100000000}"
            self.chan = CtrlChannel(box[0], create=True, n_readers=world - 1, slots=n_slots, slot_bytes=slot_bytes)
        dist.broadcast_object_list(box, src=0, group=self.ctrl)      # also orders attach after create
        if rank != 0:
            self.chan = CtrlChannel(box[0], create=False, n_readers=world - 1, reader_index=rank - 1, slots=n_slots,
                                    slot_bytes=slot_bytes)
        start, end = split_layers(cfg.num_hidden_layers, pp)[topo.pp_rank]
        comm = None
        from parallax_b200.models.registry import family_of

        family = family_of(cfg.architecture)
        if tp > 1:
            # the fused all-gather / reduce-scatter GEMMs are built for the GQA decoder's shapes; the other
            # families run the same layout over library collectives
            use_fused = (on_gpu if fused is None else fused) and family == "decoder"
            if use_fused:
                comm = FusedTPComm(self.tp_group, tp, topo.tp_rank, self.device, max_num_tokens_per_batch,
                                   cfg.hidden_size, max_n=cfg.hidden_size,
                                   max_k=max(cfg.hidden_size, cfg.intermediate_size // tp, cfg.q_size // tp))
            else:
                comm = CollectiveTPComm(self.tp_group, tp, topo.tp_rank, align=128 if on_gpu else 1)
        ep_comm = None
        if ep > 1:
            from parallax_b200.parallel.ep import EPComm

            ep_comm = EPComm(self.ep_group, ep, topo.ep_rank, self.device, max_rows=lane_tokens + lane_batch,
                             fused=on_gpu if fused is None else fused)
            if ep_local_init is None:
                # generate only the local experts when the full expert set would not fit beside the KV cache
                per_layer = cfg.num_experts * 3 * cfg.moe_intermediate_size * cfg.hidden_size * 2
                ep_local_init = per_layer * (end - start) > (48 << 30)
        self.ep_comm = ep_comm
        stage_ep = (topo.ep_rank, ep, ep_comm)
        if tp > 1 and family != "decoder" and cfg.is_moe:
            from parallax_b200.parallel.ep import EPComm
            from parallax_b200.parallel.tp_comm import padded_rows_per_rank

            # the experts of such a stage are split over its tensor-parallel ranks; each rank brings its own rows
            rows = padded_rows_per_rank(max_num_tokens_per_batch, tp, 128 if on_gpu else 1)
            stage_ep = (topo.tp_rank, tp, EPComm(self.tp_group, tp, topo.tp_rank, self.device, max_rows=rows,
                                                 fused=on_gpu if fused is None else fused))
        if weights is not None and not weights_prefiltered:
            from parallax_b200.loader.filter import filter_weights_for_range

            weights = filter_weights_for_range(weights, start, end, cfg.num_hidden_layers, cfg.tie_word_embeddings)
        # the rotary table covers every position a request may reach, whatever length the checkpoint's
        # config advertises (positions beyond that length are the caller's choice, as with the reference's
        # on-the-fly rotary embedding); a table cut at the advertised length was read out of bounds
        max_positions = max_total_length + 8
        # hybrid models: the prefix cache keeps snapshots of the recurrent state at block boundaries in extra
        # state slots behind the requests' own (the same layout on every rank; rank 0 decides the copies and
        # every rank carries them out in plan order, see `slot_pre` / `slot_post` in the step plan)
        hybrid_prefix = 0
        if cfg.has_linear_layers and enable_prefix_cache and ep == 1:
            hybrid_prefix = 32 if linear_prefix_slots is None else max(int(linear_prefix_slots), 0)
        if cfg.has_linear_layers and not hybrid_prefix:
            enable_prefix_cache = False
        self.worker = StageWorker(cfg, start, end, self.device, dtype, page_size, num_blocks=num_blocks,
                                  kv_fraction=kv_fraction, seed=seed, weights=weights, max_positions=max_positions,
                                  tp_rank=topo.tp_rank, tp_size=tp, tp_group=self.tp_group, comm=comm,
                                  num_linear_slots=(max(max_batch_size * 2, 16) + hybrid_prefix) if cfg.has_linear_layers else 0,
                                  ep_rank=stage_ep[0], ep_size=stage_ep[1], ep_comm=stage_ep[2],
                                  ep_local_init=bool(ep_local_init) and weights is None,
                                  kv_cache_dtype=kv_cache_dtype)
        # every rank must agree on the number of KV blocks
        nb = torch.tensor([self.worker.num_blocks], dtype=torch.int64)
        dist.all_reduce(nb, op=dist.ReduceOp.MIN, group=self.ctrl)
        self.num_blocks = int(nb)
        self.liveness_timeout_s, self.step_timeout_s = liveness_timeout_s, step_timeout_s
        self._recv_stream = torch.cuda.Stream(self.device) if on_gpu else None
        self._ret_stream = torch.cuda.Stream(self.device) if on_gpu else None
        self._recv_ring = [_RecvSlot() for _ in range(self.max_in_flight + 2)]
        self._recv_n = 0
        self._warm_links()
        self.planner = None
        self.planners: list = []
        if rank == 0:
            for _ in range(self.n_plans):
                pl = Planner(cfg, self.num_blocks, page_size, lane_batch if ep > 1 else max_batch_size, lane_tokens,
                             ratio, chunked_prefill_size, enable_prefix_cache, max_total_length, request_timeout_s,
                             eos_token_id, linear_prefix_slots=hybrid_prefix)
                if pl.cache.needs_slots:
                    # a request that matched a snapshot starts from a copy of it: queued for the next plan
                    pl.cache.on_copy_slot = lambda dst, src: self._slot_pre.append((int(dst), int(src)))
                pl.scheduler.max_prefill_tokens_per_batch = max_prefill_tokens_per_batch
                pl.scheduler.align_rows = align_rows
                self.planners.append(pl)
            self.planner = self.planners[0]
        self.builders = [BatchBuilder(self.device, lane_tokens + max_batch_size, max_batch_size,
                                      max_blocks) for _ in range(self.max_in_flight + 1)]
        self._bi = 0
        # per-request LoRA adapters: every rank keeps the adapter slots of its own layers; rank 0 decides which
        # adapter lives in which slot and sends the loads (slot, name, path) with the next step plan
        self.lora = None
        self._lora_loads: list = []
        if lora:
            from parallax_b200.loader.lora import LoRAManager, LoRAStack, TPLoRAStack

            if not hasattr(self.worker.model, "lora") or family != "decoder":
                raise ValueError("per-request LoRA in the multi-GPU engine is available for the GQA decoder families")
            n_slots, max_rank = int(lora.get("max_loaded") or 4), int(lora.get("max_rank") or 64)
            # tensor-parallel ranks keep their slice of every adapter; expert-parallel lanes run whole attention
            # layers (the adapters' targets) on their own requests, so each keeps whole adapters
            self.worker.model.lora = (TPLoRAStack if tp > 1 else LoRAStack)(self.worker.model, n_slots, max_rank)
            if rank == 0:
                self.lora = LoRAManager([], n_slots, lora.get("paths"),
                                        on_load=lambda slot, name, path: self._lora_loads.append((int(slot), name, path)))
        self._slot_pre: list = []        # rank 0: state-slot copies (dst, src) that the next plan carries
        # JSON-schema constrained requests: rank 0 keeps a matcher per request to know when the document is
        # complete; the rank that samples keeps its own copy (built from the schema that rides with the
        # request's first constrained plan) and advances it with the tokens it picks
        self.tokenizer = tokenizer
        self._grammar_known: set = set()        # rank 0: request ids whose schema has travelled
        self._grammar_drops: list = []          # rank 0: finished constrained requests, for the next plan
        self._grammars: dict = {}               # sampling rank: request id -> matcher
        self._py_rng = __import__("random").Random(seed + 777)
        self.in_flight: deque = deque()
        self._pending_sends: deque = deque()
        self._side_events: list = []
        self._rng = np.random.default_rng(seed + 12345)
        self.steps = 0
        self.keep_logits = False
        self.last_logits = None
        self.marks: list = []
        self._busy_events: list = []     # (start, end, rows) of every micro-batch's compute since the last mark
        self.h2d_bytes = 0
        self.host_s = {"plan": 0.0, "publish": 0.0, "launch": 0.0, "wait": 0.0, "commit": 0.0}
        # token return: pinned host buffers (tokens + the last stage's status word), reused round-robin
        self._ret_host = [torch.empty(2 * max_batch_size + 1, dtype=torch.int32, pin_memory=on_gpu)
                          for _ in range((self.max_in_flight + 2) * self.n_plans)] if rank == 0 else []
        self._ret_n = 0
        # rank 0: the stage's launches run in their own thread (on GPUs; CPU ranks keep one thread)
        self._exec_thread = None
        self._exec_q: "queue.Queue" = queue.Queue()
        self._exec_err: list = []
        use_thread = on_gpu if executor_thread is None else executor_thread
        if rank == 0 and use_thread and world > 1:
            self._exec_thread = threading.Thread(target=self._executor_loop, name="pxl-stage0-exec", daemon=True)
            self._exec_thread.start()

    # ------------------------------------------------------------------ links
    def _prev(self) -> int:
        return self.topo.rank - self.topo.lanes

    def _next(self) -> int:
        return self.topo.rank + self.topo.lanes

    def _warm_links(self) -> None:
        """Open every point-to-point connection once, in an order that all ranks share, so that
        connection set-up (which blocks the host until the peer arrives) never meets the
        serving loop, where the ranks post their transfers at different times."""
        topo = self.topo
        x = torch.zeros(8, dtype=self.worker.dtype, device=self.device)
        if not topo.is_first_stage:
            dist.recv(x, src=self._prev(), group=self.hop_in)
        if not topo.is_last_stage:
            dist.send(x, dst=self._next(), group=self.hop_out)
        t = torch.zeros(8, dtype=torch.int32, device=self.device)
        for snd in topo.token_senders:
            if snd == 0:
                continue
            if topo.rank == snd:
                dist.send(t, dst=0, group=self.ret[snd])
            elif topo.rank == 0:
                dist.recv(t, src=snd, group=self.ret[snd])
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)

    def _recv_hidden(self, rows: int) -> torch.Tensor:
        """Post the receive of a micro-batch's activations into the next ring buffer. On a GPU the
        receive lives on a side stream (it can complete while earlier micro-batches still compute)
        and the compute stream waits for its event only."""
        H = self.cfg.hidden_size
        slot = self._recv_ring[self._recv_n % len(self._recv_ring)]
        self._recv_n += 1
        if slot.buf is None or slot.buf.shape[0] < rows:
            slot.buf = torch.empty((max(rows, 256), H), dtype=self.worker.dtype, device=self.device)
            slot.free = None
            if self.device.type == "cuda" and self.topo.tp == 1:
                # The memory comes from the compute stream's pool: it may be a block that a tensor of an
                # earlier micro-batch gave back while kernels that use it are still queued there. Stream
                # order protects such reuse on the compute stream only, and the first writer of this buffer
                # is the receive on the side stream - so that receive waits for everything queued so far.
                slot.free = torch.cuda.Event()
                slot.free.record(torch.cuda.current_stream(self.device))
                slot.buf.record_stream(self._recv_stream)
        hidden = slot.buf[:rows]
        if self.device.type != "cuda" or self.topo.tp > 1:
            # tensor-parallel stages keep the receive in stream order: their fused GEMM + collective kernels
            # spread one CTA over every SM and wait on each other, so no other kernel may sit on an SM
            # beside them (a receive that waits for its sender would)
            dist.recv(hidden, src=self._prev(), group=self.hop_in)
            slot.free = None
            return hidden
        arrived = torch.cuda.Event()
        with torch.cuda.stream(self._recv_stream):
            if slot.free is not None:
                self._recv_stream.wait_event(slot.free)     # the compute that last read this buffer is done
            work = dist.irecv(hidden, src=self._prev(), group=self.hop_in)
            work.wait()
            arrived.record()
        torch.cuda.current_stream(self.device).wait_event(arrived)
        slot.free = torch.cuda.Event()       # recorded by the caller after the compute that reads the buffer
        return hidden

    # ------------------------------------------------------------------ rank-0 API
    @property
    def scheduler(self):
        return self.planner.scheduler if self.n_plans == 1 else _SchedulerGroup([p.scheduler for p in self.planners])

    @property
    def cache(self):
        return self.planner.cache if self.n_plans == 1 else _CacheGroup([p.cache for p in self.planners])

    def add_request(self, req: Request) -> None:
        req.sampling_params.verify()
        req.max_total_length = min(req.max_total_length, self.planner.max_total_length)
        req.lora_slot = -1
        if getattr(req, "lora_path", None):
            if self.lora is None:
                raise ValueError("this engine was started without LoRA support (--enable-lora)")
            req.lora_slot = self.lora.acquire(req.lora_path)       # the load travels with the next plan
        req.grammar = None
        if req.sampling_params.json_schema:
            if self.tokenizer is None:
                raise ValueError("json_schema needs an engine that knows its tokenizer (DistEngine(tokenizer=...))")
            from parallax_b200.engine.structured import JsonSchemaMatcher

            req.grammar = JsonSchemaMatcher(req.sampling_params.json_schema)
        # expert-parallel lanes: the request stays with the least loaded lane for its whole life
        pl = min(self.planners, key=lambda p: p.scheduler.num_queued_requests + p.scheduler.num_running_requests)
        pl.scheduler.enque_request(req)

    def abort_request(self, rid: str) -> Optional[Request]:
        """Returns the request if it was still waiting for admission (it ends here, without a step)."""
        for pl in self.planners:
            try:
                return pl.scheduler.cancel_request(rid)
            except ValueError:
                pass
        return None

    @property
    def stages(self):
        """Layer span served by the whole group (what :class:`EngineLoop` reports latency over)."""
        class _Span:
            start_layer, end_layer = 0, self.cfg.num_hidden_layers
        return [_Span]

    def has_work(self) -> bool:
        return bool(self.in_flight) or any(p.scheduler.num_queued_requests > 0 or p.scheduler.num_running_requests > 0
                                           for p in self.planners)

    # ------------------------------------------------------------------ one micro-batch on this rank
    def _sample(self, lp: dict, out: torch.Tensor, constrain: bool = False) -> torch.Tensor:
        if lp.get("pen") is not None:
            from parallax_b200.engine.sampling import apply_penalties

            out = apply_penalties(out, lp["pen"])
        want_prob = bool(lp.get("want_prob"))
        probs = None
        if lp["greedy"]:
            if want_prob:
                tokens, logp = ops.argmax(out, want_logprob=True)
                probs = logp.exp()
            else:
                tokens = ops.argmax(out)
        else:
            dev = out.device
            sp = lp["sampling"]
            args = (out, torch.tensor(sp["t"], dtype=torch.float32, device=dev),
                    torch.tensor(sp["k"], dtype=torch.int32, device=dev),
                    torch.tensor(sp["p"], dtype=torch.float32, device=dev),
                    torch.tensor(sp["mp"], dtype=torch.float32, device=dev),
                    torch.tensor(sp["u"], dtype=torch.float32, device=dev))
            if want_prob:
                tokens, probs = ops.sample(*args, want_prob=True)
            else:
                tokens = ops.sample(*args)
        if constrain and lp.get("grammar"):
            tokens = self._constrain(lp, out, tokens)
            if want_prob:      # the constrained rows' tokens changed: their probability under the step's logits
                rows = torch.tensor([int(g[0]) for g in lp["grammar"]], dtype=torch.long, device=out.device)
                picked = tokens[rows].long().clamp_min(0)
                probs = probs.clone()
                probs[rows] = torch.softmax(out[rows].float(), dim=-1).gather(1, picked.view(-1, 1)).view(-1)
        return (tokens, probs) if want_prob else tokens

    def _constrain(self, lp: dict, logits: torch.Tensor, tokens: torch.Tensor) -> torch.Tensor:
        """Sampling rank: rows of requests with a JSON schema get the best candidate (or a draw among the
        valid candidates) whose text keeps the request's document valid; -1 where no token fits, which
        ends the request on rank 0. A request is never in two micro-batches at once, so this rank's
        matcher, advanced with every token picked here, is the document's state."""
        from parallax_b200.engine.structured import JsonSchemaMatcher, TokenChooser

        tok = self.tokenizer
        if tok is None:
            raise RuntimeError("a constrained request reached a sampling rank that has no tokenizer")
        chooser = TokenChooser(tok.token_text, sorted(getattr(tok, "eos_token_ids", ()) or ()))
        rows, vals = [], []
        for row, rid, schema, temp in lp["grammar"]:
            g = self._grammars.get(rid)
            if g is None:
                g = self._grammars[rid] = JsonSchemaMatcher(schema)
            choice = chooser.choose(g, logits[row], temp, self._py_rng)
            if choice is not None:
                text = tok.token_text(int(choice))
                if text and not g.done:
                    g.advance(text)
            rows.append(int(row))
            vals.append(-1 if choice is None else int(choice))
        tokens = tokens.clone()
        tokens[torch.tensor(rows, dtype=torch.long, device=tokens.device)] = torch.tensor(
            vals, dtype=tokens.dtype, device=tokens.device)
        return tokens

    def _execute(self, plan: dict):
        """Run this rank's part of one planned micro-batch. Returns, on rank 0, one handle per plan of
        the step on its sampled tokens (see :meth:`_collect`), else None."""
        topo, w = self.topo, self.worker
        on_gpu = self.device.type == "cuda"
        lane_plans = plan["lanes"]
        for slot, name, path in plan.get("lora_load") or ():
            from parallax_b200.loader.lora import LoRAAdapter

            w.model.lora.load(slot, LoRAAdapter.load(path, name))     # this rank's layers of the adapter
        for rid in plan.get("grammar_drop") or ():
            self._grammars.pop(rid, None)
        lp = lane_plans[topo.lane if self.n_plans > 1 else 0]
        if self.ep_comm is not None:
            self.ep_comm.step_max_rows = plan.get("max_rows")
        tokens = None
        is_sender = topo.rank in topo.token_senders
        if lp is None:
            # expert-parallel lane without a token in this step: it still joins every MoE exchange
            with torch.inference_mode():
                w.model.ep_idle_step()
        else:
            b = self.builders[self._bi]
            self._bi = (self._bi + 1) % len(self.builders)
            fb = b.build(lp["ids"] if topo.is_first_stage else None, lp["pos"], lp["slots"], lp["p_q"],
                         lp["p_ctx"], lp["p_tables"], lp["d_ctx"], lp["d_tables"], lp["logit_rows"],
                         lp.get("seq_rows"),
                         extra={"lora_ids": lp["lora_ids"]} if lp.get("lora_ids") is not None else None)
            if lp.get("lora_ids") is not None:
                fb.extras["lora_ids_host"] = lp["lora_ids"]
            self.h2d_bytes += fb.h2d_bytes
            T = fb.num_tokens
            hidden = None
            slot_free = None
            if not topo.is_first_stage:
                rows = w.model.comm.rows_per_rank(T) if topo.tp > 1 else T
                hidden = self._recv_hidden(rows)
                slot_free = self._recv_ring[(self._recv_n - 1) % len(self._recv_ring)].free
            ev0 = None
            if on_gpu and self.marks and len(self._busy_events) < 100000:
                ev0 = torch.cuda.Event(enable_timing=True)      # only between benchmark marks
                ev0.record()
            for dst, src in lp.get("slot_pre") or ():
                w.pool.copy_slot(dst, src)                 # resume from a snapshot of the recurrent state
            with torch.inference_mode():
                out = w.run(fb, hidden)
            for dst, src in lp.get("slot_post") or ():
                w.pool.copy_slot(dst, src)                 # snapshot at the block boundary this step reached
            if slot_free is not None:
                slot_free.record()
            if ev0 is not None:
                ev1 = torch.cuda.Event(enable_timing=True)
                ev1.record()
                self._busy_events.append((ev0, ev1, T))
            n_logits = lp["n_logits"]
            if self.keep_logits and topo.is_last_stage:
                self.last_logits = out
            if not topo.is_last_stage:
                out = out if out.is_contiguous() else out.contiguous()
                self._pending_sends.append((dist.isend(out, dst=self._next(), group=self.hop_out), out))
            elif n_logits > 0:
                with torch.inference_mode():        # (penalties update the stage's logits in place)
                    tokens = self._sample(lp, out, constrain=is_sender)
                probs = None
                if lp.get("want_prob"):
                    tokens, probs = tokens
                if is_sender:
                    # the status word of the sampling rank rides with the tokens; the tokens' probabilities
                    # (fp32 bit patterns) follow it when some request of the step asked for them
                    packed = torch.empty(_ret_len(lp), dtype=torch.int32, device=self.device)
                    packed[:n_logits].copy_(tokens)
                    if probs is not None:
                        packed[n_logits + 1:].copy_(probs.float().contiguous().view(torch.int32))
                    if on_gpu:
                        from parallax_b200.ops import cuda as cu

                        packed[n_logits:n_logits + 1].copy_(cu.status_tensor(self.device))
                    else:
                        packed[n_logits:n_logits + 1].zero_()
                    tokens = packed
                    if topo.rank != 0:
                        self._pending_sends.append((dist.isend(packed, dst=0, group=self.ret[topo.rank]), packed))
        while len(self._pending_sends) > 2 * self.max_in_flight + 2:
            self._pending_sends.popleft()[0].wait()
        if on_gpu and not (is_sender and lp is not None and lp["n_logits"] > 0):
            # ranks whose status word does not ride with tokens: mirror it to the host, look one step later
            from parallax_b200.ops import cuda as cu

            code = cu.status_mirror(self.device)
            if code and topo.rank != 0:
                self.chan.report_status(code)
            cu.status_copy_async(self.device)
        if topo.rank != 0:
            return None
        # ---- rank 0: one handle per plan of the step
        handles = []
        for i, p_i in enumerate(lane_plans):
            if p_i is None or p_i["n_logits"] == 0:
                handles.append(None)
                continue
            m = _ret_len(p_i)        # tokens, status word, and the probabilities if they were asked for
            snd = topo.token_senders[i]
            host = self._ret_host[self._ret_n % len(self._ret_host)]
            self._ret_n += 1
            if snd != 0:
                # post the receive now, in the same order in which the sender posts its sends
                if not on_gpu:
                    t = torch.empty(m, dtype=torch.int32, device=self.device)
                    handles.append(("recv", (t, dist.irecv(t, src=snd, group=self.ret[snd]), None, None)))
                    continue
                # on a side stream: reading the tokens later must not wait for the compute of the
                # micro-batches that were queued behind this one
                ev = torch.cuda.Event()
                with torch.cuda.stream(self._ret_stream):
                    t = torch.empty(m, dtype=torch.int32, device=self.device)   # from the side stream's pool
                    work = dist.irecv(t, src=snd, group=self.ret[snd])
                    work.wait()
                    host[:m].copy_(t, non_blocking=True)
                    ev.record()
                handles.append(("recv", (t, None, host[:m], ev)))
            elif on_gpu:
                ev = torch.cuda.Event()
                host[:m].copy_(tokens, non_blocking=True)
                ev.record()
                handles.append(("recv", (tokens, None, host[:m], ev)))
            else:
                handles.append(("have", tokens))
        return handles

    # ------------------------------------------------------------------ rank 0: executor thread
    def _executor_loop(self) -> None:
        if self.device.type == "cuda":
            torch.cuda.set_device(self.device)
        while True:
            item = self._exec_q.get()
            if item is None:
                return
            kind, payload, box = item
            try:
                if kind == "step":
                    box.append(self._execute(payload))
                elif kind == "mark":
                    self._on_mark()
                    box.append(None)
                else:       # "drain": everything queued before has been enqueued on the device
                    box.append(None)
            except BaseException as exc:      # surfaced by the scheduling thread at its next collect
                self._exec_err.append(exc)
                box.append(("error", exc))
            finally:
                done = getattr(box, "done", None)
                if done is not None:
                    done.set()

    class _Box(list):
        """Result slot of a queued executor job."""

        def __init__(self):
            super().__init__()
            self.done = threading.Event()

    def _submit(self, kind: str, payload=None) -> "_Box":
        box = DistEngine._Box()
        if self._exec_thread is None:
            if kind == "step":
                box.append(self._execute(payload))
            elif kind == "mark":
                self._on_mark()
                box.append(None)
            else:
                box.append(None)
            box.done.set()
        else:
            self._exec_q.put((kind, payload, box))
        return box

    def _drain_executor(self) -> None:
        self._submit("drain").done.wait()
        if self._exec_err:
            raise self._exec_err.pop(0)

    # ------------------------------------------------------------------ device-time probes
    def _on_mark(self) -> None:
        ev = None
        if self.device.type == "cuda":
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
        self.marks.append((ev, time.perf_counter(), cu_launch_count(), self.h2d_bytes))
        self._busy_prev, self._busy_events = self._busy_events, []

    def _on_elapsed(self) -> dict:
        """Device time between the last two marks (max over ranks) and the kernels launched /
        bytes copied to the device between them (sum over ranks)."""
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        (e0, t0, l0, h0), (e1, t1, l1, h1) = self.marks[-2], self.marks[-1]
        ms = e0.elapsed_time(e1) if e0 is not None else (t1 - t0) * 1e3
        mx = torch.tensor([ms], dtype=torch.float64)
        dist.all_reduce(mx, op=dist.ReduceOp.MAX, group=self.ctrl)
        sm = torch.tensor([float(l1 - l0), float(h1 - h0)], dtype=torch.float64)
        dist.all_reduce(sm, op=dist.ReduceOp.SUM, group=self.ctrl)
        # how long each rank's GPU computed between the marks (the rest of device_ms it waited for its
        # neighbours or its host) and the largest micro-batch it saw
        busy = torch.zeros(self.topo.world, dtype=torch.float64)
        rows = torch.zeros(self.topo.world, dtype=torch.float64)
        for a, b, n_rows in getattr(self, "_busy_prev", []):
            busy[self.topo.rank] += a.elapsed_time(b)
            rows[self.topo.rank] = max(float(rows[self.topo.rank]), float(n_rows))
        dist.all_reduce(busy, op=dist.ReduceOp.SUM, group=self.ctrl)
        dist.all_reduce(rows, op=dist.ReduceOp.SUM, group=self.ctrl)
        return {"device_ms": float(mx[0]), "launches": int(sm[0]), "h2d_bytes": int(sm[1]), "wall_s": t1 - t0,
                "busy_ms_per_rank": [round(float(x), 2) for x in busy], "max_rows_per_rank": [int(x) for x in rows]}

    def mark(self) -> None:
        """Rank 0: every rank records a CUDA event at this point of its stream."""
        self.chan.publish({"cmd": "mark"})
        self._submit("mark").done.wait()

    def elapsed(self) -> dict:
        self._drain_executor()
        self.chan.publish({"cmd": "elapsed"})
        return self._on_elapsed()

    # ------------------------------------------------------------------ follower loop
    def serve_one(self) -> bool:
        """Ranks other than 0: take the next message of rank 0 and act on it. False after "stop"."""
        plan = self.chan.receive()
        cmd = plan.get("cmd")
        if cmd == "stop":
            return False
        if cmd == "mark":
            self._on_mark()
        elif cmd == "elapsed":
            self._on_elapsed()
        elif cmd == "refit":
            from parallax_b200.utils.weight_refit import apply_refit_to_stage

            apply_refit_to_stage(self.worker, self.cfg, plan["refit"])
        else:
            self._execute(plan)
            self.steps += 1
        return True

    def apply_refit(self, refit: dict) -> int:
        """Rank 0, between steps: every rank applies a refit request (``index_map`` + ``paths`` of content-addressed
        blocks on disk) to its own layers and slices, at the same place in the order of plans; the work already
        queued on the devices still runs with the old weights. Cached prefixes are dropped. Returns the number
        of tensors rank 0 used."""
        from parallax_b200.utils.weight_refit import apply_refit_to_stage

        assert self.topo.rank == 0
        self._drain_executor()
        self.chan.publish({"cmd": "refit", "refit": refit})
        used = apply_refit_to_stage(self.worker, self.cfg, refit)
        for pl in self.planners:
            pl.cache.invalidate_prefix_cache()
        return used

    def finish_sends(self) -> None:
        for work, _ in self._pending_sends:
            work.wait()
        self._pending_sends.clear()

    def serve_forever(self) -> None:
        """Ranks other than 0: execute published plans until rank 0 says stop."""
        assert self.topo.rank != 0
        while self.serve_one():
            pass
        self.finish_sends()
        self._status_all_ranks()
        self.chan.close()

    def _status_all_ranks(self) -> list[int]:
        """Device status word of every rank (0 = healthy), gathered over the control group."""
        code = 0
        if self.device.type == "cuda":
            from parallax_b200.ops import cuda as cu

            torch.cuda.synchronize(self.device)
            code = int(cu.status_tensor(self.device).item())
        codes = torch.zeros(self.topo.world, dtype=torch.int64)
        codes[self.topo.rank] = code
        dist.all_reduce(codes, group=self.ctrl)
        return codes.tolist()

    def shutdown(self) -> None:
        """Rank 0: stop the other ranks; raises if any rank's kernels reported a device error."""
        if self.topo.rank == 0:
            if self._exec_thread is not None:
                self._drain_executor()
                self._exec_q.put(None)
                self._exec_thread.join(10.0)
                self._exec_thread = None
            self.chan.publish({"cmd": "stop"})
            codes = self._status_all_ranks()       # also a barrier: every reader has seen the stop message
            self.chan.close()
            if any(codes):
                from parallax_b200.ops import _lib

                raise _lib.KernelError("device status per rank: " + ", ".join(
                    f"rank {i}: {_lib.describe(c)}" for i, c in enumerate(codes) if c))

    # ------------------------------------------------------------------ rank-0 step
    def _release_lora(self, req: Request) -> None:
        if self.lora is not None and getattr(req, "lora_slot", -1) >= 0:
            self.lora.release(req.lora_path)
            req.lora_slot = -1

    def _release_grammar(self, req: Request) -> None:
        """A constrained request ended (however): the sampling rank forgets its matcher with the next plan."""
        if getattr(req, "grammar", None) is not None and req.request_id in self._grammar_known:
            self._grammar_known.discard(req.request_id)
            self._grammar_drops.append(req.request_id)

    def _drop(self, pl, req: Request) -> None:
        pl.scheduler.evict_request(req.request_id)
        pl.cache.free_request(req.request_id)
        self._release_lora(req)
        self._release_grammar(req)
        self._side_events.append((req, None))

    def _plan_one(self, pl):
        """Form and plan the next micro-batch of one planner: ``(arrays, lane plan)`` or None."""
        sched = pl.scheduler
        seqs = sched.form_batch()
        for req in sched.pop_rejected():
            self._side_events.append((req, None))
        live = []
        for s in seqs:
            if s.req.abort:
                s.req.update_status(RequestStatus.FINISHED_ABORT)
                self._drop(pl, s.req)
            else:
                live.append(s)
        if not live:
            return None
        arrays = pl.plan_arrays(live)
        for s in live:
            if s.req.is_finished:      # aborted by KV exhaustion during planning
                self._drop(pl, s.req)
        if arrays is None:
            return None
        owners = arrays["owners"]
        sps = [s.req.sampling_params for s in owners]
        greedy = all(sp.is_greedy for sp in sps)
        lp = {k: arrays[k] for k in ("ids", "pos", "slots", "p_q", "p_ctx", "p_tables", "d_ctx", "d_tables",
                                     "logit_rows", "seq_rows")}
        lp.update(n_logits=len(owners), greedy=greedy)
        if any(s.req.return_probs for s in owners):
            lp["want_prob"] = True
        if self.lora is not None and any(getattr(s.req, "lora_slot", -1) >= 0 for s in arrays["ordered"]):
            rows = np.full(arrays["pos"].shape[0], -1, dtype=np.int32)      # adapter slot of every token row
            o = 0
            for s in arrays["ordered"]:
                rows[o:o + s.num_tokens] = getattr(s.req, "lora_slot", -1)
                o += s.num_tokens
            lp["lora_ids"] = rows
        if any(getattr(s.req, "grammar", None) is not None for s in owners):
            rows = []
            for row, s in enumerate(owners):
                if getattr(s.req, "grammar", None) is None:
                    continue
                rid, sp = s.req.request_id, s.req.sampling_params
                first = rid not in self._grammar_known
                self._grammar_known.add(rid)
                rows.append((row, rid, sp.json_schema if first else None, 0.0 if sp.is_greedy else sp.temperature))
            lp["grammar"] = rows
        from parallax_b200.engine.sampling import build_penalties

        pen = build_penalties([s.req for s in owners])
        if pen is not None:
            lp["pen"] = pen
        if not greedy:
            lp["sampling"] = {"t": [0.0 if sp.is_greedy else sp.temperature for sp in sps],
                              "k": [sp.top_k if sp.top_k > 0 else 0 for sp in sps], "p": [sp.top_p for sp in sps],
                              "mp": [sp.min_p for sp in sps], "u": self._rng.random(len(sps)).tolist()}
        return arrays, lp

    def _issue(self) -> bool:
        t0 = time.perf_counter()
        planned = [self._plan_one(pl) for pl in self.planners]
        if all(x is None for x in planned):
            return False
        lane_plans = [None if x is None else x[1] for x in planned]
        # prefill bookkeeping that does not depend on the sampled token: the next chunk of a long
        # prompt may enter the pipeline right behind this one. The chunk's full blocks are published now:
        # whoever matches them is planned later and every rank runs the plans in order. For hybrid models
        # this also decides the state snapshots of the step (taken on every rank right after its forward).
        for pl, x in zip(self.planners, planned):
            if x is None:
                continue
            post: list = []
            snap = (lambda src, dst: post.append((int(dst), int(src)))) if pl.cache.needs_slots else None
            for s in x[0]["ordered"]:
                if s.is_prefill:
                    s.req.num_computed_tokens = s.start + s.num_tokens
                    pl.cache.insert_full_blocks_to_cache(s.req.request_id, s.req.num_computed_tokens,
                                                         snapshot_linear=snap)
                    if not s.produces_token:
                        pl.scheduler.enque_request(s.req)
            if pl.cache.needs_slots:
                x[1]["slot_pre"], self._slot_pre = self._slot_pre, []
                x[1]["slot_post"] = post
        plan = {"cmd": "step", "lanes": lane_plans,
                "max_rows": max(int(lp["pos"].shape[0]) for lp in lane_plans if lp is not None)}
        if self._lora_loads:
            plan["lora_load"], self._lora_loads = self._lora_loads, []
        if self._grammar_drops:
            plan["grammar_drop"], self._grammar_drops = self._grammar_drops, []
        t1 = time.perf_counter()
        self.chan.publish(plan)
        t2 = time.perf_counter()
        res = self._submit("step", plan)
        t3 = time.perf_counter()
        hs = self.host_s
        hs["plan"] += t1 - t0
        hs["publish"] += t2 - t1
        hs["launch"] += t3 - t2
        self.in_flight.append(([None if x is None else x[0] for x in planned], res))
        return True

    def _wait_return(self, ev, work) -> None:
        """Wait for the tokens of the oldest micro-batch while watching the other ranks' heartbeats:
        a rank that stopped (crashed process, stuck host loop) turns into an exception here instead
        of an endless wait, and the serving loop fails the affected requests."""
        t0 = time.monotonic()
        sleep = 0.0
        waiter = None
        if ev is None:
            # gloo receive handles only complete inside wait(): block in a helper thread and watch it
            err: list = []

            def _wait():
                try:
                    work.wait()
                except Exception as exc:      # e.g. the peer's connection was reset
                    err.append(exc)

            waiter = threading.Thread(target=_wait, daemon=True)
            waiter.start()
        while True:
            if waiter is not None:
                waiter.join(0.0 if sleep == 0.0 else 0.01)
                done = not waiter.is_alive()
            else:
                done = ev.query()
            if done:
                if waiter is not None and err:
                    raise RuntimeError(f"the last pipeline stage stopped responding: {err[0]}")
                return
            if sleep:
                time.sleep(sleep)
            elif self._exec_thread is not None:
                time.sleep(0)          # hand the interpreter to the thread that launches rank 0's stage
            waited = time.monotonic() - t0
            if waited > 0.002:
                sleep = 0.0002
            elif self._exec_thread is not None:
                sleep = 0.00005
            if waited > self.liveness_timeout_s / 4:
                stale = self.chan.stale_readers(self.liveness_timeout_s)
                if stale:
                    raise RuntimeError(f"rank(s) {[i + 1 for i in stale]} stopped responding "
                                       f"(no heartbeat for {self.liveness_timeout_s:.0f} s)")
            if waited > self.step_timeout_s:
                raise TimeoutError(f"no tokens came back within {self.step_timeout_s:.0f} s")

    def _check_device_status(self, sender_codes: dict) -> None:
        """Fail the step if any rank's kernels gave up (bounded wait ran out, bad table entry)."""
        bad = {r: c for r, c in sender_codes.items() if c}
        for idx, code in self.chan.failed_readers().items():
            bad[idx + 1] = code
        if self.device.type == "cuda":
            from parallax_b200.ops import cuda as cu

            code = cu.status_mirror(self.device)
            if code:
                bad[0] = code
                try:
                    cu.raise_if_status(self.device)
                except ops.KernelError:
                    pass
        if bad:
            from parallax_b200.ops import _lib

            raise ops.KernelError("device status: " + ", ".join(f"rank {r}: {_lib.describe(c)}"
                                                                for r, c in sorted(bad.items())))

    def _collect(self) -> list:
        arrays_list, box = self.in_flight.popleft()
        out = []
        tw = time.perf_counter()
        box.done.wait()
        if self._exec_err:
            raise self._exec_err.pop(0)
        handles = box[0]
        tokens_of: list = []
        probs_of: dict = {}
        codes = {}
        for i, arrays in enumerate(arrays_list):
            toks = []
            if arrays is not None and arrays["owners"]:
                kind, t = handles[i]
                if kind == "recv":
                    t, work, host, ev = t
                    self._wait_return(ev, work)
                    if ev is not None:
                        t = host
                vals = t.tolist()
                n = len(arrays["owners"])
                toks = vals[:n]
                codes[self.topo.token_senders[i]] = int(vals[n])
                if len(vals) > n + 1:      # the tokens' probabilities follow the status word as fp32 bit patterns
                    probs_of[i] = np.array(vals[n + 1:], dtype=np.int32).view(np.float32).tolist()
            tokens_of.append(toks)
        self.host_s["wait"] += time.perf_counter() - tw
        self._check_device_status(codes)
        tc = time.perf_counter()
        now = time.time()
        for lane, (pl, arrays, toks) in enumerate(zip(self.planners, arrays_list, tokens_of)):
            if arrays is None:
                continue
            sched, cache = pl.scheduler, pl.cache
            probs = probs_of.get(lane)
            for j, (s, tok) in enumerate(zip(arrays["owners"], toks)):
                req = s.req
                tok = int(tok)
                g = getattr(req, "grammar", None)
                if tok >= 0:
                    req.commit_new_token(tok, probs[j] if (probs is not None and req.return_probs) else None, now=now)
                    cache.append_request_token(req.request_id, tok)
                if g is not None and not req.is_finished:
                    # the document grows by the token's text; it ends the request once it is complete,
                    # and so does a step in which no token fitted (-1 from the sampling rank)
                    text = self.tokenizer.token_text(tok) if tok >= 0 else None
                    if not text or not g.advance(text) or g.done:
                        req.update_status(RequestStatus.FINISHED_EOS)
                if sched.check_and_update_request_status(req):
                    cache.free_request(req.request_id)
                    self._release_lora(req)
                    self._release_grammar(req)
                else:
                    sched.enque_request(req, now=now)
                out.append((req, tok if tok >= 0 else None))
        self.host_s["commit"] += time.perf_counter() - tc
        return out

    def step(self) -> list:
        """Rank 0: issue micro-batches while the pipeline has room, then collect the oldest."""
        assert self.topo.rank == 0
        out = []
        for pl in self.planners:
            for req in pl.scheduler.get_timed_out_requests():
                req.update_status(RequestStatus.FINISHED_ABORT)
                pl.scheduler.evict_request(req.request_id)
                pl.cache.free_request(req.request_id)
                self._release_lora(req)
                self._release_grammar(req)
                out.append((req, None))
        issued = False
        while len(self.in_flight) < self.max_in_flight:
            if not self._issue():
                break
            issued = True
        if self.in_flight and (len(self.in_flight) >= self.max_in_flight or not issued):
            out += self._collect()
        if self._side_events:
            out += self._side_events
            self._side_events = []
        self.steps += 1
        return out

    def generate(self, prompts, sampling_params, max_steps: int = 1 << 30) -> list[list[int]]:
        from parallax_b200.engine.request import SamplingParams

        reqs = [Request(input_ids=list(p), sampling_params=SamplingParams.from_dict(sampling_params.to_dict()),
                        max_total_length=self.planner.max_total_length) for p in prompts]
        for r in reqs:
            self.add_request(r)
        n = 0
        while self.has_work() and n < max_steps:
            self.step()
            n += 1
        return [r.output_ids for r in reqs]
