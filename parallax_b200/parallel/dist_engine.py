"""Multi-GPU engine inside one box: pipeline stages x tensor-parallel ranks, one process per GPU.

Rank layout: ``rank = pp_rank * tp + tp_rank``. Rank 0 owns the scheduler and the logical KV
plan; every step it broadcasts the packed step inputs (a few hundred KB of indices) to all
ranks over a CPU control group, so that every rank can enqueue its kernels without waiting on
a device-to-host copy. Activations move stage to stage with NCCL point-to-point on NVLink -
each tensor-parallel rank sends its own row shard to its counterpart in the next stage - and
only the sampled token ids travel back to rank 0, on a separate communicator so that the
return path never queues behind the forward path. Several micro-batches are kept in flight
(``pp`` by default) to fill the pipeline: rank 0 issues plan k+1 before it reads the tokens of
plan k.

This replaces the reference's stage transport (hidden states -> safetensors bytes -> protobuf
-> ZMQ -> libp2p RPC -> ZMQ, with a GPU<->CPU copy on every hop;
``src/parallax/p2p/message_util.py:202-219``, ``src/parallax/p2p/server.py:628-711``) for the
case where all stages live on one NVSwitch domain.
"""

from __future__ import annotations

import logging
import os
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


def cu_launch_count() -> int:
    from parallax_b200.ops import cuda as cu

    return cu.launch_count


def split_layers(num_layers: int, pp: int) -> list[tuple[int, int]]:
    """Even contiguous split (what water-filling yields for identical GPUs); earlier stages get
    the remainder layers because the last stage also runs the lm_head."""
    base, rem = divmod(num_layers, pp)
    out, s = [], 0
    for i in range(pp):
        n = base + (1 if i < rem else 0)
        out.append((s, s + n))
        s += n
    return out


@dataclass
class Topology:
    world: int
    rank: int
    pp: int
    tp: int

    @property
    def pp_rank(self) -> int:
        return self.rank // self.tp

    @property
    def tp_rank(self) -> int:
        return self.rank % self.tp

    @property
    def is_first_stage(self) -> bool:
        return self.pp_rank == 0

    @property
    def is_last_stage(self) -> bool:
        return self.pp_rank == self.pp - 1

    @property
    def last_stage_root(self) -> int:
        return (self.pp - 1) * self.tp


class DistEngine:
    def __init__(self, cfg: ModelConfig, pp: int, tp: int, device, dtype=None, page_size: int = 16,
                 num_blocks: Optional[int] = None, kv_fraction: float = 0.85, max_batch_size: int = 8,
                 max_num_tokens_per_batch: int = 16384, micro_batch_ratio: Optional[int] = None,
                 chunked_prefill_size: Optional[int] = 1024, max_prefill_tokens_per_batch: Optional[int] = None,
                 enable_prefix_cache: bool = True,
                 max_total_length: int = 32768, request_timeout_s: Optional[float] = 600, eos_token_id=None,
                 seed: int = 0, weights: Optional[dict] = None, fused: Optional[bool] = None,
                 max_in_flight: Optional[int] = None, weights_prefiltered: bool = False,
                 liveness_timeout_s: float = 10.0, step_timeout_s: float = 600.0):
        assert dist.is_initialized(), "init the default process group first (nccl on GPUs, gloo on CPU)"
        self.cfg = cfg
        self.device = torch.device(device)
        world, rank = dist.get_world_size(), dist.get_rank()
        assert world == pp * tp, f"world size {world} != pp*tp = {pp * tp}"
        self.topo = Topology(world, rank, pp, tp)
        on_gpu = self.device.type == "cuda"
        # groups (every rank creates every group, in the same order)
        self.ctrl = dist.new_group(list(range(world)), backend="gloo")
        self.ret = dist.new_group(list(range(world)), backend="nccl" if on_gpu else "gloo")
        self.tp_group = None
        for s in range(pp if tp > 1 else 0):
            g = dist.new_group(list(range(s * tp, (s + 1) * tp)), backend="nccl" if on_gpu else "gloo")
            if s == self.topo.pp_rank:
                self.tp_group = g
        # step plans travel through shared memory (all ranks live on one box); the name is agreed once
        from parallax_b200.parallel.ctrl_channel import CtrlChannel

        box = [None]
        if rank == 0:
            box[0] = f"pxl_ctrl_{os.getpid()}_{int(time.time() * 1e3) % 100000000}"
            self.chan = CtrlChannel(box[0], create=True, n_readers=world - 1)
        dist.broadcast_object_list(box, src=0, group=self.ctrl)      # also orders attach after create
        if rank != 0:
            self.chan = CtrlChannel(box[0], create=False, n_readers=world - 1, reader_index=rank - 1)
        start, end = split_layers(cfg.num_hidden_layers, pp)[self.topo.pp_rank]
        comm = None
        if tp > 1:
            use_fused = on_gpu if fused is None else fused
            if use_fused:
                comm = FusedTPComm(self.tp_group, tp, self.topo.tp_rank, self.device, max_num_tokens_per_batch,
                                   cfg.hidden_size, max_n=cfg.hidden_size,
                                   max_k=max(cfg.hidden_size, cfg.intermediate_size // tp, cfg.q_size // tp))
            else:
                comm = CollectiveTPComm(self.tp_group, tp, self.topo.tp_rank, align=128 if on_gpu else 1)
        if weights is not None and not weights_prefiltered:
            from parallax_b200.loader.filter import filter_weights_for_range

            weights = filter_weights_for_range(weights, start, end, cfg.num_hidden_layers, cfg.tie_word_embeddings)
        max_positions = min(cfg.max_position_embeddings, max_total_length + 8)
        self.worker = StageWorker(cfg, start, end, self.device, dtype, page_size, num_blocks=num_blocks,
                                  kv_fraction=kv_fraction, seed=seed, weights=weights, max_positions=max_positions,
                                  tp_rank=self.topo.tp_rank, tp_size=tp, tp_group=self.tp_group, comm=comm,
                                  num_linear_slots=max(max_batch_size * 2, 16) if cfg.has_linear_layers else 0)
        if cfg.has_linear_layers:
            enable_prefix_cache = False
        # every rank must agree on the number of KV blocks
        nb = torch.tensor([self.worker.num_blocks], dtype=torch.int64)
        dist.all_reduce(nb, op=dist.ReduceOp.MIN, group=self.ctrl)
        self.num_blocks = int(nb)
        self.max_in_flight = max_in_flight or pp
        self.liveness_timeout_s, self.step_timeout_s = liveness_timeout_s, step_timeout_s
        self._ret_stream = torch.cuda.Stream(self.device) if on_gpu else None
        self._warm_links()
        ratio = micro_batch_ratio or pp
        self.planner = None
        if rank == 0:
            self.planner = Planner(cfg, self.num_blocks, page_size, max_batch_size, max_num_tokens_per_batch, ratio,
                                   chunked_prefill_size, enable_prefix_cache, max_total_length, request_timeout_s,
                                   eos_token_id)
            self.planner.scheduler.max_prefill_tokens_per_batch = max_prefill_tokens_per_batch
        max_blocks = (max_total_length + page_size - 1) // page_size + 1
        self.builders = [BatchBuilder(self.device, max_num_tokens_per_batch + max_batch_size, max_batch_size,
                                      max_blocks) for _ in range(self.max_in_flight + 1)]
        self._bi = 0
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

    def _warm_links(self) -> None:
        """Open every point-to-point connection once, in an order that all ranks share, so that
        connection set-up (which blocks the host until the peer arrives) never meets the
        serving loop, where the ranks post their transfers at different times."""
        topo = self.topo
        x = torch.zeros(8, dtype=self.worker.dtype, device=self.device)
        if not topo.is_first_stage:
            dist.recv(x, src=topo.rank - topo.tp)
        if not topo.is_last_stage:
            dist.send(x, dst=topo.rank + topo.tp)
        if topo.last_stage_root != 0:
            t = torch.zeros(8, dtype=torch.int32, device=self.device)
            if topo.rank == topo.last_stage_root:
                dist.send(t, dst=0, group=self.ret)
            elif topo.rank == 0:
                dist.recv(t, src=topo.last_stage_root, group=self.ret)
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)

    # ------------------------------------------------------------------ rank-0 API
    @property
    def scheduler(self):
        return self.planner.scheduler

    @property
    def cache(self):
        return self.planner.cache

    def add_request(self, req: Request) -> None:
        req.sampling_params.verify()
        req.max_total_length = min(req.max_total_length, self.planner.max_total_length)
        self.scheduler.enque_request(req)

    def abort_request(self, rid: str) -> None:
        try:
            self.scheduler.cancel_request(rid)
        except ValueError:
            pass

    @property
    def stages(self):
        """Layer span served by the whole group (what :class:`EngineLoop` reports latency over)."""
        class _Span:
            start_layer, end_layer = 0, self.cfg.num_hidden_layers
        return [_Span]

    def has_work(self) -> bool:
        return bool(self.in_flight) or self.scheduler.num_queued_requests > 0 or self.scheduler.num_running_requests > 0

    # ------------------------------------------------------------------ plan broadcast
    def _bcast(self, plan: Optional[dict]) -> dict:
        if self.topo.rank == 0:
            self.chan.publish(plan)
            return plan
        return self.chan.receive()

    def _execute(self, plan: dict):
        """Run this rank's part of one planned micro-batch. Returns the sampled-token tensor on
        rank 0 (after the return hop) or None."""
        topo, w = self.topo, self.worker
        b = self.builders[self._bi]
        self._bi = (self._bi + 1) % len(self.builders)
        fb = b.build(plan["ids"] if topo.is_first_stage else None, plan["pos"], plan["slots"], plan["p_q"],
                     plan["p_ctx"], plan["p_tables"], plan["d_ctx"], plan["d_tables"], plan["logit_rows"],
                     plan.get("seq_rows"))
        self.h2d_bytes += fb.h2d_bytes
        T, H = fb.num_tokens, self.cfg.hidden_size
        hidden = None
        if not topo.is_first_stage:
            rows = w.model.comm.rows_per_rank(T) if topo.tp > 1 else T
            hidden = torch.empty((rows, H), dtype=w.dtype, device=self.device)
            dist.recv(hidden, src=topo.rank - topo.tp)
        ev0 = ev1 = None
        if self.device.type == "cuda" and self.marks and len(self._busy_events) < 100000:
            ev0 = torch.cuda.Event(enable_timing=True)      # only between benchmark marks
            ev0.record()
        with torch.inference_mode():
            out = w.run(fb, hidden)
        if ev0 is not None:
            ev1 = torch.cuda.Event(enable_timing=True)
            ev1.record()
            self._busy_events.append((ev0, ev1, T))
        tokens = None
        if self.keep_logits and topo.is_last_stage:
            self.last_logits = out
        if not topo.is_last_stage:
            self._pending_sends.append((dist.isend(out.contiguous(), dst=topo.rank + topo.tp), out))
        elif plan["n_logits"] > 0:
            if plan["greedy"]:
                tokens = ops.argmax(out)
            else:
                dev = out.device
                sp = plan["sampling"]
                tokens = ops.sample(out, torch.tensor(sp["t"], dtype=torch.float32, device=dev),
                                    torch.tensor(sp["k"], dtype=torch.int32, device=dev),
                                    torch.tensor(sp["p"], dtype=torch.float32, device=dev),
                                    torch.tensor(sp["mp"], dtype=torch.float32, device=dev),
                                    torch.tensor(sp["u"], dtype=torch.float32, device=dev))
            if topo.rank == topo.last_stage_root and topo.last_stage_root != 0:
                self._pending_sends.append((dist.isend(tokens, dst=0, group=self.ret), tokens))
        while len(self._pending_sends) > 2 * self.max_in_flight:
            self._pending_sends.popleft()[0].wait()
        if topo.rank != 0 or plan["n_logits"] == 0:
            return None
        if topo.last_stage_root != 0:
            # post the receive now, in the same order in which the last stage posts its sends
            if self.device.type != "cuda":
                t = torch.empty(plan["n_logits"], dtype=torch.int32, device=self.device)
                return ("recv", (t, dist.irecv(t, src=topo.last_stage_root, group=self.ret), None, None))
            # on a side stream: reading the tokens later must not wait for the compute of the
            # micro-batches that were queued behind this one
            host = torch.empty(plan["n_logits"], dtype=torch.int32, pin_memory=True)
            ev = torch.cuda.Event()
            with torch.cuda.stream(self._ret_stream):
                t = torch.empty(plan["n_logits"], dtype=torch.int32, device=self.device)   # from the side stream's pool
                work = dist.irecv(t, src=topo.last_stage_root, group=self.ret)
                work.wait()
                host.copy_(t, non_blocking=True)
                ev.record()
            return ("recv", (t, None, host, ev))
        return ("have", tokens)

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
        self._bcast({"cmd": "mark"})
        self._on_mark()

    def elapsed(self) -> dict:
        self._bcast({"cmd": "elapsed"})
        return self._on_elapsed()

    # ------------------------------------------------------------------ follower loop
    def serve_forever(self) -> None:
        """Ranks other than 0: execute broadcast plans until rank 0 says stop."""
        assert self.topo.rank != 0
        while True:
            plan = self._bcast(None)
            if plan.get("cmd") == "stop":
                break
            if plan.get("cmd") == "mark":
                self._on_mark()
                continue
            if plan.get("cmd") == "elapsed":
                self._on_elapsed()
                continue
            self._execute(plan)
            self.steps += 1
        for work, _ in self._pending_sends:
            work.wait()
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
            self._bcast({"cmd": "stop"})
            codes = self._status_all_ranks()       # also a barrier: every reader has seen the stop message
            self.chan.close()
            if any(codes):
                from parallax_b200.ops import _lib

                raise _lib.KernelError("device status per rank: " + ", ".join(
                    f"rank {i}: {_lib.describe(c)}" for i, c in enumerate(codes) if c))

    # ------------------------------------------------------------------ rank-0 step
    def _drop(self, req: Request) -> None:
        self.scheduler.evict_request(req.request_id)
        self.cache.free_request(req.request_id)
        self._side_events.append((req, None))

    def _issue(self) -> bool:
        t0 = time.perf_counter()
        sched = self.scheduler
        seqs = sched.form_batch()
        for req in sched.pop_rejected():
            self._side_events.append((req, None))
        live = []
        for s in seqs:
            if s.req.abort:
                s.req.update_status(RequestStatus.FINISHED_ABORT)
                self._drop(s.req)
            else:
                live.append(s)
        if not live:
            return False
        arrays = self.planner.plan_arrays(live)
        for s in live:
            if s.req.is_finished:      # aborted by KV exhaustion during planning
                self._drop(s.req)
        if arrays is None:
            return False
        owners = arrays["owners"]
        sps = [s.req.sampling_params for s in owners]
        greedy = all(sp.is_greedy for sp in sps)
        plan = {k: arrays[k] for k in ("ids", "pos", "slots", "p_q", "p_ctx", "p_tables", "d_ctx", "d_tables",
                                       "logit_rows", "seq_rows")}
        plan.update(cmd="step", n_logits=len(owners), greedy=greedy)
        if not greedy:
            plan["sampling"] = {"t": [0.0 if sp.is_greedy else sp.temperature for sp in sps],
                                "k": [sp.top_k if sp.top_k > 0 else 0 for sp in sps], "p": [sp.top_p for sp in sps],
                                "mp": [sp.min_p for sp in sps], "u": self._rng.random(len(sps)).tolist()}
        t1 = time.perf_counter()
        self._bcast(plan)
        t2 = time.perf_counter()
        res = self._execute(plan)
        t3 = time.perf_counter()
        hs = self.host_s
        hs["plan"] += t1 - t0
        hs["publish"] += t2 - t1
        hs["launch"] += t3 - t2
        # prefill bookkeeping that does not depend on the sampled token: the next chunk of a long
        # prompt may enter the pipeline right behind this one
        for s in arrays["ordered"]:
            if s.is_prefill:
                s.req.num_computed_tokens = s.start + s.num_tokens
                self.cache.insert_full_blocks_to_cache(s.req.request_id, s.req.num_computed_tokens)
                if not s.produces_token:
                    sched.enque_request(s.req)
        self.in_flight.append((arrays, res))
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
            import threading

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
            waited = time.monotonic() - t0
            if waited > 0.002:
                sleep = 0.0002
            if waited > self.liveness_timeout_s / 4:
                stale = self.chan.stale_readers(self.liveness_timeout_s)
                if stale:
                    raise RuntimeError(f"rank(s) {[i + 1 for i in stale]} stopped responding "
                                       f"(no heartbeat for {self.liveness_timeout_s:.0f} s)")
            if waited > self.step_timeout_s:
                raise TimeoutError(f"no tokens came back within {self.step_timeout_s:.0f} s")

    def _collect(self) -> list:
        arrays, res = self.in_flight.popleft()
        out = []
        owners = arrays["owners"]
        token_list = []
        if owners:
            kind, t = res
            tw = time.perf_counter()
            if kind == "recv":
                t, work, host, ev = t
                self._wait_return(ev, work)
                if ev is not None:
                    t = host
            token_list = t.tolist()
            self.host_s["wait"] += time.perf_counter() - tw
        sched = self.scheduler
        tc = time.perf_counter()
        now = time.time()
        for s, tok in zip(owners, token_list):
            req = s.req
            tok = int(tok)
            req.commit_new_token(tok, now=now)
            self.cache.append_request_token(req.request_id, tok)
            if sched.check_and_update_request_status(req):
                self.cache.free_request(req.request_id)
            else:
                sched.enque_request(req, now=now)
            out.append((req, tok))
        self.host_s["commit"] += time.perf_counter() - tc
        return out

    def step(self) -> list:
        """Rank 0: issue micro-batches while the pipeline has room, then collect the oldest."""
        assert self.topo.rank == 0
        out = []
        for req in self.scheduler.get_timed_out_requests():
            req.update_status(RequestStatus.FINISHED_ABORT)
            self.scheduler.evict_request(req.request_id)
            self.cache.free_request(req.request_id)
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
