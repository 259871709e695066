"""In-process serving engine: scheduler + KV planner + pipeline stages + sampler.

``Engine`` is the object a user (or the HTTP frontend, or ``bench.py``) drives:

    eng = Engine(named_config("qwen3-8b"), device="cuda:0")
    eng.add_request(Request(input_ids=[...], sampling_params=SamplingParams(max_new_tokens=64)))
    while eng.has_work():
        for req, token in eng.step():
            ...

One ``step()`` is one continuous-batching iteration: admit, form a mixed prefill+decode
batch, plan KV slots, one packed host-to-device copy of the step's index tensors, forward
through every stage, sample on the last stage, one device-to-host copy of the sampled ids,
commit. It is the counterpart of one iteration of the reference's executor run loop
(``src/parallax/server/executor/base_executor.py:634-769``), with the stage hand-off being
a device tensor instead of a serialised network packet.

Stages passed as ``stage_layers=[(0,14),(14,28)]`` run in this process one after another
(used for correctness checks of sharded execution); multi-GPU pipelines use one process
per GPU, see :mod:`parallax_b200.parallel.pipeline`.
"""

from __future__ import annotations

import logging
import time
from typing import Callable, Iterable, Optional

import numpy as np
import torch

from parallax_b200 import ops
from parallax_b200.cache.manager import CacheManager
from parallax_b200.engine.batch import BatchBuilder
from parallax_b200.engine.request import PENDING_TOKEN, Request, RequestStatus, SamplingParams
from parallax_b200.engine.scheduler import BatchScheduler, ScheduledSeq
from parallax_b200.engine.worker import StageWorker
from parallax_b200.models.config import ModelConfig

logger = logging.getLogger(__name__)


def _describe_status(code: int) -> str:
    from parallax_b200.ops import _lib

    return _lib.describe(code)


class _InFlightStep:
    """A launched step whose sampled tokens have not been read yet."""

    __slots__ = ("arrays", "ids", "probs", "fb", "t0", "serial", "slot_index", "index", "host", "trace_events")

    def __init__(self, arrays, ids, probs, fb, t0, serial):
        self.arrays, self.ids, self.probs, self.fb, self.t0, self.serial = arrays, ids, probs, fb, t0, serial
        self.slot_index: list[int] = []      # per owner: index of its placeholder in the request's output_ids
        self.index: dict[str, int] = {}      # request id -> position of its token in `ids`
        self.host = None
        self.trace_events = None


class Planner:
    """Scheduler + logical KV cache: turns ready requests into packed step inputs."""

    def __init__(self, cfg: ModelConfig, num_blocks: int, page_size: int, max_batch_size: int,
                 max_num_tokens_per_batch: int, micro_batch_ratio: int = 1,
                 chunked_prefill_size: Optional[int] = 1024, enable_prefix_cache: bool = True,
                 max_total_length: int = 32768, request_timeout_s: Optional[float] = 600,
                 eos_token_id=None, shared_state=None, linear_prefix_slots: int = 0):
        self.cfg = cfg
        self.page_size = page_size
        max_blocks_per_seq = (max_total_length + page_size - 1) // page_size + 1
        max_requests = max(max_batch_size * 2, 16)
        # hybrid models: a request's recurrent state lives in a slot of its own, and the prefix cache keeps
        # snapshots of that state at block boundaries (`linear_prefix_slots` of them) to resume from
        hybrid_slots = max_requests if (cfg.has_linear_layers and enable_prefix_cache and linear_prefix_slots > 0) else 0
        self.cache = CacheManager(num_blocks, page_size, max_requests=max_requests,
                                  max_blocks_per_seq=max_blocks_per_seq,
                                  enable_prefix_cache=enable_prefix_cache, num_linear_slots=hybrid_slots,
                                  num_prefix_linear_slots=linear_prefix_slots if hybrid_slots else 0)
        self.scheduler = BatchScheduler(
            max_batch_size=max_batch_size, max_num_tokens_per_batch=max_num_tokens_per_batch,
            micro_batch_ratio=micro_batch_ratio, cache_manager=self.cache,
            chunked_prefill_size=chunked_prefill_size, request_timeout_s=request_timeout_s,
            eos_token_id=eos_token_id, max_total_length=max_total_length, shared_state=shared_state)
        self.max_total_length = max_total_length

    def plan_arrays(self, seqs: list[ScheduledSeq], pending_index: Optional[dict] = None):
        """Numpy inputs of a step. Returns None if nothing can run (e.g. all aborted by OOM).

        ``pending_index``: request id -> position of that request's token in the token tensor that the
        previous (still unread) step sampled. Decode rows of those requests get their input id on the
        device: the result carries ``patch_rows`` / ``patch_src`` for :func:`ops.patch_ids`."""
        cache, bs = self.cache, self.page_size
        state_slot = cache.get_slot if cache.needs_slots else cache.get_row     # slot of the recurrent state
        prefill = [s for s in seqs if s.is_prefill]
        decode = []
        for s in seqs:
            if s.is_prefill:
                continue
            if not cache.append_slot(s.req.request_id):
                # out of KV memory while decoding: abort the request (reference behaviour,
                # src/parallax/server/executor/mlx_executor.py:766-784)
                s.req.abort = True
                s.req.update_status(RequestStatus.FINISHED_ABORT)
                continue
            decode.append(s)
        ordered = prefill + decode
        if not ordered:
            return None
        T = sum(s.num_tokens for s in ordered)
        ids = np.empty(T, dtype=np.int32)
        pos = np.empty(T, dtype=np.int32)
        rows_of_tok = np.empty(T, dtype=np.int32)
        logit_rows, owners = [], []
        o = 0
        p_q, p_ctx, p_rows = [], [], []
        patch_rows = patch_src = None
        for s in prefill:
            n, st = s.num_tokens, s.start
            ids[o:o + n] = s.req.input_ids[st:st + n]
            pos[o:o + n] = np.arange(st, st + n, dtype=np.int32)
            row = cache.get_row(s.req.request_id)
            rows_of_tok[o:o + n] = row
            p_q.append(n)
            p_ctx.append(st + n)
            p_rows.append(row)
            if s.produces_token:
                logit_rows.append(o + n - 1)
                owners.append(s)
            o += n
        # decode rows: one Python pass collecting plain lists, then whole-array numpy stores (a numpy
        # scalar store per field and request costs several times more with hundreds of requests)
        nd = len(decode)
        if nd:
            reqs_d = [s.req for s in decode]
            d_ctx = np.fromiter((r.prompt_len + len(r.output_ids) for r in reqs_d), dtype=np.int32, count=nd)
            d_rows = np.fromiter((cache.get_row(r.request_id) for r in reqs_d), dtype=np.int32, count=nd)
            ids[o:o + nd] = np.fromiter((r.output_ids[-1] for r in reqs_d), dtype=np.int32, count=nd)
            if pending_index:
                hit = [(o + i, pending_index[r.request_id]) for i, r in enumerate(reqs_d)
                       if r.output_ids[-1] == PENDING_TOKEN and r.request_id in pending_index]
                if hit:
                    patch_rows, patch_src = (np.asarray(x, dtype=np.int32) for x in zip(*hit))
            pos[o:o + nd] = d_ctx - 1
            rows_of_tok[o:o + nd] = d_rows
            logit_rows.extend(range(o, o + nd))
            owners.extend(decode)
            o += nd
        else:
            d_rows = np.empty(0, dtype=np.int32)
            d_ctx = np.empty(0, dtype=np.int32)
        slots = cache.tables[rows_of_tok, pos // bs].astype(np.int64) * bs + (pos % bs)
        maxb_p = (max(p_ctx) + bs - 1) // bs if prefill else 0
        maxb_d = (int(d_ctx.max()) + bs - 1) // bs if len(decode) else 0
        p_tables = cache.tables[np.asarray(p_rows, dtype=np.int64), :maxb_p] if prefill else None
        d_tables = cache.tables[d_rows, :maxb_d] if len(decode) else None
        if cache.needs_slots:
            seq_rows = np.fromiter((state_slot(s.req.request_id) for s in ordered), dtype=np.int32, count=len(ordered))
        else:
            seq_rows = np.concatenate([np.asarray(p_rows, dtype=np.int32), d_rows])
        return dict(ordered=ordered, ids=ids, pos=pos, slots=slots, p_q=p_q, p_ctx=p_ctx,
                    p_tables=p_tables, d_ctx=d_ctx, d_tables=d_tables,
                    logit_rows=np.asarray(logit_rows, dtype=np.int32), owners=owners, seq_rows=seq_rows,
                    patch_rows=patch_rows, patch_src=patch_src)


class Engine:
    def __init__(
        self,
        cfg: ModelConfig,
        device="cuda:0",
        dtype=None,
        stage_layers: Optional[list[tuple[int, int]]] = None,
        page_size: int = 16,
        num_blocks: Optional[int] = None,
        kv_fraction: float = 0.85,
        max_batch_size: int = 8,
        max_num_tokens_per_batch: int = 16384,
        micro_batch_ratio: int = 1,
        chunked_prefill_size: Optional[int] = 1024,
        enable_prefix_cache: bool = True,
        max_total_length: int = 32768,
        request_timeout_s: Optional[float] = 600,
        eos_token_id=None,
        seed: int = 0,
        weights: Optional[dict] = None,
        max_kv_tokens: Optional[int] = None,
        shared_state=None,
        wire_hook: Optional[Callable] = None,
        trace=None,
        async_scheduling: Optional[bool] = None,
        linear_prefix_slots: Optional[int] = None,
        lora: Optional[dict] = None,
        kv_cache_dtype: Optional[str] = None,
        tokenizer=None,
        return_routed_experts: bool = False,
    ):
        """``tokenizer`` (anything with ``token_text(id)`` and ``eos_token_ids``) is only needed for requests
        with a ``json_schema``: constrained decoding checks candidate tokens by their text."""
        self.tokenizer = tokenizer
        self.cfg = cfg
        self.device = torch.device(device)
        self.page_size = page_size
        stage_layers = stage_layers or [(0, cfg.num_hidden_layers)]
        # the rotary table covers every position a request may reach, whatever length the checkpoint's
        # config advertises (positions beyond that length are the caller's choice, as with the reference's
        # on-the-fly rotary embedding); a table cut at the advertised length was read out of bounds
        max_positions = max_total_length + 8
        self.stages: list[StageWorker] = []
        max_requests = max(max_batch_size * 2, 16)
        # hybrid models resume a shared prefix from a snapshot of the recurrent state taken at a block
        # boundary (a recurrent state cannot be rebuilt from cached KV pages); the snapshots live in extra
        # state slots behind the requests' own
        self.linear_prefix_slots = 0
        if cfg.has_linear_layers and enable_prefix_cache:
            self.linear_prefix_slots = linear_prefix_slots if linear_prefix_slots is not None else 32
            if self.linear_prefix_slots <= 0:
                enable_prefix_cache = False
        for (s, e) in stage_layers:
            w = None
            if weights is not None:
                from parallax_b200.loader.filter import filter_weights_for_range

                w = filter_weights_for_range(weights, s, e, cfg.num_hidden_layers, cfg.tie_word_embeddings)
            self.stages.append(StageWorker(cfg, s, e, self.device, dtype, page_size, num_blocks=num_blocks,
                                           kv_fraction=kv_fraction / len(stage_layers), seed=seed, weights=w,
                                           max_kv_tokens=max_kv_tokens, max_positions=max_positions,
                                           num_linear_slots=(max_requests + self.linear_prefix_slots)
                                           if cfg.has_linear_layers else 0, kv_cache_dtype=kv_cache_dtype))
        nb = min(st.num_blocks for st in self.stages)
        self.planner = Planner(cfg, nb, page_size, max_batch_size, max_num_tokens_per_batch,
                               micro_batch_ratio, chunked_prefill_size, enable_prefix_cache,
                               max_total_length, request_timeout_s, eos_token_id, shared_state,
                               linear_prefix_slots=self.linear_prefix_slots)
        self.scheduler = self.planner.scheduler
        self.cache = self.planner.cache
        if self.cache.needs_slots:
            # a request that matched a snapshot starts from a copy of it (enqueued before its first step)
            self.cache.on_copy_slot = self._copy_state_slot
        max_blocks = self.cache.max_blocks_per_seq
        self.builder = BatchBuilder(self.device, max_num_tokens_per_batch + max_batch_size,
                                    max_batch_size, max_blocks)
        # launch step s before reading the tokens of step s-1 (GPU devices by default; PXL_SYNC_ENGINE=1 turns it off)
        import os as _os

        if async_scheduling is None:
            async_scheduling = self.device.type == "cuda" and not _os.environ.get("PXL_SYNC_ENGINE")
        self.async_scheduling = bool(async_scheduling)
        self._in_flight: Optional[_InFlightStep] = None
        self._host_slots = []
        if self.device.type == "cuda":
            for _ in range(3):
                self._host_slots.append({"ids": torch.empty(max(max_batch_size, 16), dtype=torch.int32, pin_memory=True),
                                         "probs": torch.empty(max(max_batch_size, 16), dtype=torch.float32, pin_memory=True),
                                         "event": torch.cuda.Event()})
        # per-request LoRA adapters: {"max_loaded": slots, "max_rank": r, "paths": {name: dir}}
        self.lora = None
        if lora:
            from parallax_b200.loader.lora import LoRAManager, LoRAStack

            stacks = []
            for st in self.stages:
                if not hasattr(st.model, "lora"):
                    raise ValueError(f"per-request LoRA adapters are not available for {cfg.architecture}")
                st.model.lora = LoRAStack(st.model, int(lora.get("max_loaded") or 4), int(lora.get("max_rank") or 64))
                stacks.append(st.model.lora)
            self.lora = LoRAManager(stacks, int(lora.get("max_loaded") or 4), lora.get("paths"))
        # routed-experts record for rollout replay: finished requests carry `routed_experts`
        # ([tokens with K/V][MoE layers][top-k]); a model without MoE layers leaves it off
        self.return_routed_experts = False
        if return_routed_experts:
            on = [st.model.enable_routed_capture(nb * page_size) for st in self.stages
                  if hasattr(st.model, "enable_routed_capture")]
            self.return_routed_experts = any(on)
        self.wire_hook = wire_hook  # optional transform applied to hidden states between stages
        self._gen = torch.Generator(device=self.device)
        self._gen.manual_seed(seed + 12345)
        import random as _random

        self._py_rng = _random.Random(seed + 777)          # draws among valid candidates of constrained requests
        self.last_step_stats: dict = {}
        self.total_steps = 0
        self.keep_logits = False
        self.last_logits: Optional[torch.Tensor] = None
        from parallax_b200.utils.trace import StepTracer

        self.tracer = StepTracer(trace) if isinstance(trace, str) else (trace or StepTracer.from_env())

    # ------------------------------------------------------------------ requests
    def add_request(self, req: Request) -> None:
        req.sampling_params.verify()
        req.max_total_length = min(req.max_total_length, self.planner.max_total_length)
        req.lora_slot = -1
        if req.lora_path:
            if self.lora is None:
                raise ValueError("this engine was started without LoRA support (--enable-lora)")
            req.lora_slot = self.lora.acquire(req.lora_path)     # loads the adapter if it is not resident
        req.grammar = None
        if req.sampling_params.json_schema:
            if self.tokenizer is None:
                raise ValueError("json_schema needs an engine that knows its tokenizer (Engine(tokenizer=...))")
            from parallax_b200.engine.structured import JsonSchemaMatcher

            req.grammar = JsonSchemaMatcher(req.sampling_params.json_schema)
        self.scheduler.enque_request(req)

    def update_weights(self, tensors: dict) -> int:
        """Online refit of this engine's stages from HF-named tensors (whole layers; see
        ``DecoderStage.reload_layers``). Cached prefixes were computed with the old weights and are dropped.
        Call between steps. Returns the number of tensors used."""
        used = sum(st.model.update_weights(tensors) for st in self.stages)
        self.cache.invalidate_prefix_cache()
        return used

    def apply_refit(self, refit: dict) -> int:
        """A refit request in the scheduler's format (``index_map``: weight -> content id, ``paths``: content id ->
        readable file): every stage takes the blocks of its layers, checks them against their ids and reloads.
        Call between steps (``EngineLoop.call`` does). Returns the number of tensors used."""
        from parallax_b200.utils.weight_refit import apply_refit_to_stage

        used = sum(apply_refit_to_stage(st, self.cfg, refit) for st in self.stages)
        self.cache.invalidate_prefix_cache()
        return used

    def abort_request(self, rid: str) -> Optional[Request]:
        """Returns the request if it was still waiting for admission (it ends here, without a step)."""
        try:
            return self.scheduler.cancel_request(rid)
        except ValueError:
            return None

    def has_work(self) -> bool:
        return (self._in_flight is not None or self.scheduler.num_queued_requests > 0
                or self.scheduler.num_running_requests > 0)

    # ------------------------------------------------------------------ sampling
    def _sample(self, logits: torch.Tensor, owners: list[ScheduledSeq]):
        from parallax_b200.engine.sampling import apply_penalties, build_penalties

        sps = [s.req.sampling_params for s in owners]
        want_prob = any(s.req.return_probs for s in owners)
        logits = apply_penalties(logits, build_penalties([s.req for s in owners]))
        if any(getattr(s.req, "grammar", None) is not None for s in owners):
            ids, probs = self._sample_rows(logits, owners, sps, want_prob)
            return self._constrain(logits, owners, ids), probs
        return self._sample_rows(logits, owners, sps, want_prob)

    def _constrain(self, logits: torch.Tensor, owners: list[ScheduledSeq], ids: torch.Tensor) -> torch.Tensor:
        """Rows of requests with a JSON schema: the best candidate token (or a draw among the valid ones)
        whose text keeps the request's document valid replaces what the sampler picked. Such steps are
        committed before the next one is planned, so the matcher is always up to date here."""
        from parallax_b200.engine.structured import TokenChooser

        tok = self.tokenizer
        chooser = TokenChooser(tok.token_text, sorted(getattr(tok, "eos_token_ids", ()) or ()))
        picks = []
        for row, s in enumerate(owners):
            g = getattr(s.req, "grammar", None)
            if g is None:
                continue
            sp = s.req.sampling_params
            choice = chooser.choose(g, logits[row], 0.0 if sp.is_greedy else sp.temperature, self._py_rng)
            if choice is None:
                s.req.grammar_stuck = True          # nothing valid: the request ends with what it has
                choice = 0
            picks.append((row, int(choice)))
        if picks:
            rows = torch.tensor([r for r, _t in picks], dtype=torch.long, device=ids.device)
            vals = torch.tensor([t for _r, t in picks], dtype=ids.dtype, device=ids.device)
            ids = ids.clone()
            ids[rows] = vals
        return ids

    def _sample_rows(self, logits: torch.Tensor, owners: list[ScheduledSeq], sps, want_prob: bool):
        if all(sp.is_greedy for sp in sps):
            if want_prob:
                ids, lp = ops.argmax(logits, want_logprob=True)
                return ids, lp.exp()
            return ops.argmax(logits), None
        dev = logits.device
        temperature = torch.tensor([0.0 if sp.is_greedy else sp.temperature for sp in sps],
                                   dtype=torch.float32, device=dev)
        top_k = torch.tensor([sp.top_k if sp.top_k > 0 else 0 for sp in sps], dtype=torch.int32, device=dev)
        top_p = torch.tensor([sp.top_p for sp in sps], dtype=torch.float32, device=dev)
        min_p = torch.tensor([sp.min_p for sp in sps], dtype=torch.float32, device=dev)
        u = torch.rand(len(sps), generator=self._gen, device=dev, dtype=torch.float32)
        if want_prob:
            return ops.sample(logits, temperature, top_k, top_p, min_p, u, want_prob=True)
        return ops.sample(logits, temperature, top_k, top_p, min_p, u), None

    def _copy_state_slot(self, dst: int, src: int) -> None:
        for st in self.stages:
            st.pool.copy_slot(dst, src)

    def _snapshot_state(self, src_slot: int, dst_slot: int) -> None:
        """Keep the recurrent state of a request as of the block boundary it just reached."""
        self._copy_state_slot(dst_slot, src_slot)

    # ------------------------------------------------------------------ device status word
    def _queue_status_read(self) -> None:
        """The kernels' status word rides back with the step's tokens (one pinned int, no extra
        synchronisation)."""
        if self.device.type == "cuda":
            from parallax_b200.ops import cuda as _cuda

            _cuda.status_copy_async(self.device)

    def _step_status(self) -> int:
        """Status word as of the end of the step that was just read back (0 = healthy); clears it."""
        if self.device.type != "cuda":
            return 0
        from parallax_b200.ops import cuda as _cuda

        code = _cuda.status_mirror(self.device)
        if code:
            try:
                _cuda.raise_if_status(self.device)
            except ops.KernelError:
                pass
        return code

    # ------------------------------------------------------------------ one step
    def _routed_experts(self, req: Request):
        """The request's routing record, read by the KV slots of its tokens (one device-to-host copy at the
        end of the request): ``[tokens][MoE layers of all stages][top-k]``."""
        rid = req.request_id
        if not self.cache.has_request(rid):
            return None
        n = min(self.cache.get_context_length(rid), req.prompt_len + max(len(req.output_ids) - 1, 0))
        table = self.cache.get_block_table(rid)
        if n <= 0 or not table:
            return None
        ps = self.page_size
        slots = (torch.tensor(table, dtype=torch.int64).view(-1, 1) * ps + torch.arange(ps).view(1, -1)).flatten()[:n]
        slots = slots.to(self.device)
        parts = [st.model.routed_experts_of(slots) for st in self.stages if getattr(st.model, "routed_buf", None) is not None]
        return torch.cat(parts, dim=1).cpu().tolist()

    def _release(self, req: Request) -> None:
        if self.return_routed_experts and req.is_finished and getattr(req, "routed_experts", None) is None:
            req.routed_experts = self._routed_experts(req)
        self.cache.free_request(req.request_id)
        if self.lora is not None and getattr(req, "lora_slot", -1) >= 0:
            self.lora.release(req.lora_path)
            req.lora_slot = -1

    @torch.inference_mode()
    def step(self, events=None) -> list[tuple[Request, Optional[int]]]:
        """Run one engine iteration. Returns ``(request, new_token or None)`` for every
        request that produced a token or finished.

        With ``async_scheduling`` the step that is launched here is NOT the one whose tokens are
        returned: the engine plans and launches step s from sequence lengths alone (the decode rows take
        their input ids on the device from the tokens step s-1 sampled), and only then reads and commits
        the tokens of step s-1, while the GPU already works on step s. The events of a call therefore lag
        one step; :meth:`flush` returns the last ones. A request that ends on an EOS / stop token has
        one wasted row in the step that was launched before the token was read.

        ``events``: optional ``(start, end)`` CUDA events recorded on the compute stream right
        before the step's host-to-device copy and right after sampling (device-time probes)."""
        out: list[tuple[Request, Optional[int]]] = []
        t_step = time.perf_counter()
        sched = self.scheduler
        for req in sched.get_timed_out_requests():
            req.update_status(RequestStatus.FINISHED_ABORT)
            sched.evict_request(req.request_id)
            self._release(req)
            out.append((req, None))
        seqs = sched.form_batch()
        for req in sched.pop_rejected():
            out.append((req, None))
        # requests aborted by the client while waiting for their turn
        live = []
        for s in seqs:
            if s.req.abort:
                s.req.update_status(RequestStatus.FINISHED_ABORT)
                sched.evict_request(s.req.request_id)
                self._release(s.req)
                out.append((s.req, None))
            else:
                live.append(s)
        prev = self._in_flight
        # penalties count the tokens a request has produced: their rows need the previous step's values on
        # the host, so such a step is not launched ahead of them
        needs_values = any(s.req.sampling_params.has_penalties or getattr(s.req, "grammar", None) is not None
                           for s in live)
        if needs_values and prev is not None:
            self._in_flight = None
            out += self._commit(prev)
            prev = None
            live = [s for s in live if not s.req.is_finished]      # ended on the token that was just read
        arrays = self.planner.plan_arrays(live, prev.index if prev is not None else None) if live else None
        for s in live:
            if s.req.is_finished:  # aborted by KV exhaustion during planning
                sched.evict_request(s.req.request_id)
                self._release(s.req)
                out.append((s.req, None))
        if arrays is None:
            if prev is not None:
                self._in_flight = None
                out += self._commit(prev)
            return out
        t0 = time.perf_counter()
        tr = self.tracer
        if tr is not None:
            tr.span("schedule+plan", t_step, t0)
            if events is None and self.device.type == "cuda":
                events = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
        if events is not None:
            events[0].record()
        extra = None
        if arrays["patch_rows"] is not None:
            extra = {"patch_rows": arrays["patch_rows"], "patch_src": arrays["patch_src"]}
        if self.lora is not None and any(getattr(s.req, "lora_slot", -1) >= 0 for s in arrays["ordered"]):
            rows = np.full(arrays["pos"].shape[0], -1, dtype=np.int32)     # adapter slot of every token row
            o = 0
            for s in arrays["ordered"]:
                rows[o:o + s.num_tokens] = getattr(s.req, "lora_slot", -1)
                o += s.num_tokens
            extra = dict(extra or {}, lora_ids=rows)
        fb = self.builder.build(arrays["ids"], arrays["pos"], arrays["slots"], arrays["p_q"],
                                arrays["p_ctx"], arrays["p_tables"], arrays["d_ctx"], arrays["d_tables"],
                                arrays["logit_rows"], arrays["seq_rows"], extra=extra)
        if "patch_rows" in fb.extras:
            ops.patch_ids(fb.input_ids, fb.extras["patch_rows"], prev.ids, fb.extras["patch_src"])
        owners = arrays["owners"]
        h = None
        for i, st in enumerate(self.stages):
            h = st.run(fb, h)
            if self.wire_hook is not None and i + 1 < len(self.stages):
                h = self.wire_hook(h)
        if self.keep_logits:
            self.last_logits = h
        ids = probs = None
        if owners:
            ids, probs = self._sample(h, owners)
        if events is not None:
            events[1].record()
        cur = _InFlightStep(arrays, ids, probs, fb, t0, self.total_steps)
        self._read_back(cur)
        t_launched = time.perf_counter()
        self._advance_requests(cur)
        self.total_steps += 1
        self.last_step_stats = {
            "tokens": fb.num_tokens, "prefill_tokens": fb.num_prefill_tokens, "decode": fb.num_decode,
            "h2d_bytes": fb.h2d_bytes, "d2h_bytes": 4 * len(owners) * (2 if probs is not None else 1) + 4,
            "new_tokens": len(owners),
        }
        if tr is not None:
            tr.span("build+launch", t0, t_launched, tokens=fb.num_tokens, prefill=fb.num_prefill_tokens, decode=fb.num_decode)
            if events is not None:
                cur.trace_events = events
        # the tokens of the step before this one (its GPU work ended when this step's began)
        self._in_flight = cur
        if prev is not None:
            out += self._commit(prev)
        if not self.async_scheduling or needs_values:
            self._in_flight = None
            out += self._commit(cur)
        self.last_step_stats["wall_s"] = time.perf_counter() - t0
        return out

    # ------------------------------------------------------------------ the two halves of a step's bookkeeping
    def _read_back(self, cur: "_InFlightStep") -> None:
        """Enqueue the device-to-host copy of the step's tokens (and probabilities) and of the status
        word; an event marks their arrival."""
        n = len(cur.arrays["owners"])
        if self.device.type != "cuda":
            return
        from parallax_b200.ops import cuda as _cuda

        slot = self._host_slots[cur.serial % len(self._host_slots)]
        if n:
            if slot["ids"].numel() < n:
                slot["ids"] = torch.empty(max(n, 2 * slot["ids"].numel()), dtype=torch.int32, pin_memory=True)
                slot["probs"] = torch.empty(slot["ids"].numel(), dtype=torch.float32, pin_memory=True)
            slot["ids"][:n].copy_(cur.ids, non_blocking=True)
            if cur.probs is not None:
                slot["probs"][:n].copy_(cur.probs, non_blocking=True)
        _cuda.status_copy_async(self.device)
        slot["event"].record()
        cur.host = slot

    def _advance_requests(self, cur: "_InFlightStep") -> None:
        """Everything about the launched step that does not need the sampled values: prompt progress,
        publishing the chunk's full KV blocks to the prefix cache (a request that matches them can only be
        scheduled in a later step, which the stream orders after this one), a placeholder for each token
        that is on its way, and the requests' readiness for the next step."""
        sched, cache = self.scheduler, self.cache
        now = time.time()
        owner_ids = {id(s) for s in cur.arrays["owners"]}
        for s in cur.arrays["ordered"]:
            req = s.req
            if s.is_prefill:
                req.num_computed_tokens = s.start + s.num_tokens
                cache.insert_full_blocks_to_cache(req.request_id, req.num_computed_tokens,
                                                  snapshot_linear=self._snapshot_state if cache.needs_slots else None)
            if id(s) in owner_ids:
                k = req.reserve_token()
                cur.slot_index.append(k)
                cur.index[req.request_id] = len(cur.slot_index) - 1
                if not sched.ends_by_length_after(req, k + 1):
                    sched.enque_request(req, now=now)      # decodes on: ready for the next step
            else:
                sched.enque_request(req, now=now)          # next prompt chunk

    def _commit(self, st: "_InFlightStep") -> list:
        """Read the tokens of a launched step, fill them in and finish the requests that end on them."""
        out = []
        owners = st.arrays["owners"]
        tr = self.tracer
        t_wait = time.perf_counter()
        token_list, prob_list = [], None
        if self.device.type == "cuda":
            st.host["event"].synchronize()
            if owners:
                token_list = st.host["ids"][:len(owners)].tolist()
                if st.probs is not None:
                    prob_list = st.host["probs"][:len(owners)].tolist()
        elif owners:
            token_list = st.ids.tolist()
            prob_list = st.probs.tolist() if st.probs is not None else None
        code = self._step_status()
        sched, cache = self.scheduler, self.cache
        if code:
            # a kernel of the step gave up (bounded wait ran out, bad table entry): its outputs are
            # undefined. Nothing of it is committed; the serving loop fails the batch.
            for s, k in zip(owners, st.slot_index):
                del s.req.output_ids[k:]
            self._in_flight = None
            fb = st.fb
            raise ops.KernelError(f"device status after step {st.serial}: {_describe_status(code)} "
                                  f"[{fb.num_tokens} rows: {fb.num_prefill_tokens} prompt rows in "
                                  f"{fb.num_prefill_seqs} slices, {fb.num_decode} decode rows, {fb.num_logits} logit rows]")
        t_synced = time.perf_counter()
        now = time.time()
        for i, s in enumerate(owners):
            req = s.req
            k = st.slot_index[i]
            tok = int(token_list[i])
            if req.is_finished:           # ended earlier (EOS seen after this row was launched, abort)
                if k < len(req.output_ids) and req.output_ids[k] == PENDING_TOKEN:
                    # aborted (client, time-out, KV memory) while this token was on its way: it was computed,
                    # so it takes its place in the record (the request's stream has ended already)
                    req.fill_token(k, tok, prob_list[i] if prob_list else None, now=now)
                continue
            req.fill_token(k, tok, prob_list[i] if prob_list else None, now=now)
            cache.append_request_token(req.request_id, tok)
            why = sched.finish_reason(req, k + 1, tok)
            g = getattr(req, "grammar", None)
            if g is not None and why is None:
                # the document grows by the token's text; it ends the request once it is complete
                text = self.tokenizer.token_text(tok)
                stuck = getattr(req, "grammar_stuck", False) or not text or not g.advance(text)
                if stuck or g.done:
                    why = RequestStatus.FINISHED_EOS
                if stuck:
                    del req.output_ids[k:]      # no candidate fitted: the stand-in token is not part of the reply
                    tok = None
            if why is not None:
                del req.output_ids[k + 1:]      # a placeholder of the step that is already running
                req.update_status(why)
                sched.evict_request(req.request_id)
                self._release(req)
            out.append((req, tok))
        for s in st.arrays["ordered"]:
            if s.is_prefill and not s.produces_token and s.req.abort and not s.req.is_finished:
                s.req.update_status(RequestStatus.FINISHED_ABORT)
                sched.evict_request(s.req.request_id)
                self._release(s.req)
                out.append((s.req, None))
        if tr is not None:
            tr.span("wait for tokens", t_wait, t_synced)
            tr.span("commit", t_synced, time.perf_counter())
            if st.trace_events is not None:
                tr.device_span(st.serial + 1, st.trace_events[0], st.trace_events[1], st.t0, tokens=st.fb.num_tokens)
        return out

    def flush(self) -> list:
        """Read and commit the step that is still in flight (asynchronous scheduling); returns its events
        like :meth:`step`. A no-op otherwise."""
        st, self._in_flight = self._in_flight, None
        return self._commit(st) if st is not None else []

    # ------------------------------------------------------------------ convenience
    def generate(self, prompts: Iterable[list[int]], sampling_params: Optional[SamplingParams] = None,
                 max_steps: int = 1 << 30) -> list[list[int]]:
        """Blocking helper: run the prompts to completion and return the generated ids."""
        reqs = []
        for p in prompts:
            sp = sampling_params or SamplingParams()
            r = Request(input_ids=list(p), sampling_params=SamplingParams.from_dict(sp.to_dict()),
                        max_total_length=self.planner.max_total_length)
            reqs.append(r)
            self.add_request(r)
        steps = 0
        while self.has_work() and steps < max_steps:
            self.step()
            steps += 1
        if self.device.type == "cuda":
            from parallax_b200.ops import cuda as _cuda

            _cuda.check_status(self.device)
        return [r.output_ids for r in reqs]
