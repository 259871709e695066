"""Per-node continuous-batching scheduler.

Two phases per step, like the reference's local scheduler
(``src/parallax/server/scheduler.py:251-392``): (1) admit waiting requests into the running
set while ``max_batch_size`` and the KV pool allow (allocation includes the prefix-cache
match); (2) form the next micro-batch from *ready* running requests — prefills first in
admission order, each costing ``min(remaining prompt, chunked_prefill_size)`` tokens, then
ready decodes — bounded by ``micro_batch_size = max_batch_size // micro_batch_ratio``
sequences and ``max_num_tokens_per_batch`` tokens. A request that is in flight in the
pipeline is not ready again until its token came back, which is what keeps several
micro-batches in flight across stages.

Unlike the reference, several requests may be mid-way through a chunked prefill at once and
prefill chunks share a forward pass with decodes.
"""

from __future__ import annotations

import logging
import time
from collections import OrderedDict, deque
from dataclasses import dataclass
from typing import Iterable, Optional

from parallax_b200.engine.request import _FINISHED as _FINISHED_STATES
from parallax_b200.engine.request import Request, RequestStatus

logger = logging.getLogger(__name__)


def _normalize_token_ids(x) -> set[int]:
    if x is None:
        return set()
    if isinstance(x, int):
        return {x}
    return {int(t) for t in x}


@dataclass(slots=True)
class ScheduledSeq:
    req: Request
    num_tokens: int        # tokens run in this step
    start: int             # sequence position of the first token run in this step
    is_prefill: bool
    produces_token: bool   # last prompt chunk or decode step => a token is sampled


class BatchScheduler:
    def __init__(
        self,
        max_batch_size: int = 8,
        max_num_tokens_per_batch: int = 16384,
        micro_batch_ratio: int = 1,
        cache_manager=None,
        chunked_prefill_size: Optional[int] = 1024,
        request_timeout_s: Optional[float] = 600,
        eos_token_id=None,
        max_total_length: int = 32768,
        is_first_peer: bool = True,
        prefill_priority: int = 0,
        shared_state=None,
        max_prefill_tokens_per_batch: Optional[int] = None,
        align_rows: int = 0,
    ):
        self.max_batch_size = max_batch_size
        self.max_num_tokens_per_batch = max_num_tokens_per_batch
        self.micro_batch_size = max(1, max_batch_size // max(1, micro_batch_ratio))
        self.cache_manager = cache_manager
        self.chunked_prefill_size = chunked_prefill_size
        # prompt tokens one batch may carry in total (None = only the token budget limits them): with
        # micro-batches rotating through a pipeline this keeps them even, a long prompt is spread over
        # consecutive micro-batches instead of stalling every stage behind one heavy batch
        self.max_prefill_tokens_per_batch = max_prefill_tokens_per_batch
        # when > 0, a batch whose last prompt slice is cut anyway is cut so that the batch's total rows
        # (prompt tokens + decode rows) are a multiple of this: the GEMMs work on 128-row tiles, so 300
        # rows cost as much tensor time as 384 while 256 cost a third less
        self.align_rows = align_rows
        self.request_timeout_s = request_timeout_s
        self.eos_token_ids = _normalize_token_ids(eos_token_id)
        self.max_total_length = max_total_length
        # ready decode rows keep their place in a step when prompt tokens would fill the budget (see form_batch);
        # False restores prompts-first, which benchmarks use while they build a closed loop's steady state
        self.decode_first = True
        self.is_first_peer = is_first_peer
        self.prefill_priority = prefill_priority
        self.shared_state = shared_state
        self._wait_queue: deque[Request] = deque()
        self._running: "OrderedDict[str, Request]" = OrderedDict()
        self._last_reported = -1
        self._rejected: list[Request] = []

    # ------------------------------------------------------------------ queues
    @property
    def num_queued_requests(self) -> int:
        return len(self._wait_queue)

    @property
    def num_running_requests(self) -> int:
        return len(self._running)

    def running_requests(self) -> Iterable[Request]:
        return self._running.values()

    def get_running_request(self, rid: str) -> Optional[Request]:
        return self._running.get(rid)

    def enque_request(self, req: Request, now: Optional[float] = None) -> None:
        """New requests go to the wait queue; a running request coming back from the
        pipeline becomes ready for its next step (and moves to the end of the ready order)."""
        if req.is_finished:
            return
        if now is None:
            now = time.time()
        running = self._running.get(req.request_id)
        if running is not None:
            running.ready_for_next_step = True
            running.last_updated_time = now
            self._running.move_to_end(req.request_id)
            return
        req.last_updated_time = now
        self._wait_queue.append(req)

    def evict_request(self, rid: str) -> Optional[Request]:
        return self._running.pop(rid, None)

    def cancel_request(self, rid: str) -> Optional[Request]:
        """A running request is flagged and ends at its next step; one that still waits for admission is taken
        out of the queue and returned (status CANCELLED): it produces no further event by itself."""
        req = self._running.get(rid)
        if req is not None:
            req.abort = True
            return None
        for r in list(self._wait_queue):
            if r.request_id == rid:
                self._wait_queue.remove(r)
                r.update_status(RequestStatus.CANCELLED)
                return r
        raise ValueError(f"Attempted to cancel non-existent request {rid}.")

    # ------------------------------------------------------------------ phase 1
    def admit_requests(self) -> None:
        while self._wait_queue and len(self._running) < self.max_batch_size:
            req = self._wait_queue.popleft()
            rid = req.request_id
            if rid in self._running:
                continue
            # a request may not outgrow what the engine was sized for (block tables, rotary table)
            req.max_total_length = min(req.max_total_length, self.max_total_length)
            if req.total_length > self.max_total_length:
                req.update_status(RequestStatus.FINISHED_ABORT)
                req.abort = True
                self._rejected.append(req)
                continue
            if self.cache_manager is not None and not self.cache_manager.has_request(rid):
                ok, matched = self.cache_manager.allocate_request(rid, req.total_length, token_ids=req.input_ids,
                                                                  namespace=getattr(req, "lora_path", None))
                if not ok:
                    # out of KV memory: keep FIFO order and stop admitting
                    self._wait_queue.appendleft(req)
                    break
                req.num_cached_tokens = matched
                req.num_computed_tokens = max(req.num_computed_tokens, matched)
            self._running[rid] = req
            req.ready_for_next_step = True
            req.last_updated_time = time.time()
        self._report_metrics()

    def pop_rejected(self) -> list[Request]:
        out, self._rejected = self._rejected, []
        return out

    def _report_metrics(self) -> None:
        if self.shared_state is None:
            return
        cur = len(self._running)
        if cur != self._last_reported:
            try:
                self.shared_state.update_metrics(current_requests=cur)
            except Exception:  # metrics must never break serving
                pass
            self._last_reported = cur

    # ------------------------------------------------------------------ timeouts
    def get_timed_out_requests(self) -> list[Request]:
        if not self.request_timeout_s:
            return []
        now = time.time()
        out = []
        for req in self._running.values():
            if req.last_updated_time is not None and now - req.last_updated_time > self.request_timeout_s:
                req.abort = True
                out.append(req)
        return out

    # ------------------------------------------------------------------ phase 2
    def form_batch(self) -> list[ScheduledSeq]:
        self.admit_requests()
        if not self._running:
            return []
        budget = self.max_num_tokens_per_batch
        batch: list[ScheduledSeq] = []
        prefills, decodes = [], []
        for req in self._running.values():
            st = req.status
            if not req.ready_for_next_step or st in _FINISHED_STATES:
                continue
            (prefills if st == RequestStatus.PREFILLING else decodes).append(req)
        used = 0
        chunk = self.chunked_prefill_size
        prefill_cap = self.max_prefill_tokens_per_batch
        cm = self.cache_manager
        starting: set = set()      # first blocks that prompts of this batch are about to compute
        # Decode rows ride along first: prompt slices are cut to fill whatever room is left, so a backlog of
        # prompt tokens (long prompts, many arrivals) would otherwise take the whole budget step after step
        # and no running request would get its next token until the backlog is gone. (The reference fills
        # prefills first as well, src/parallax/server/scheduler.py:357-379, but never cuts a slice to fit.)
        # Only tokens are reserved: sequence slots go to prompts first, as before (a step takes few prompts
        # and the running set never exceeds the slots of an unsplit batch).
        budget_p = budget - (min(len(decodes), self.micro_batch_size, budget) if self.decode_first else 0)
        for req in prefills:
            if len(batch) >= self.micro_batch_size:
                break
            if prefill_cap is not None and used >= prefill_cap:
                break
            if cm is not None and cm.prefix_cache is not None and req.num_computed_tokens == req.num_cached_tokens \
                    and not req.output_ids:
                # a prompt that has not started: blocks published since its admission are reused, and if
                # another prompt of this very batch computes its first missing block it waits one step
                # (the block is published when that batch is launched) instead of computing it twice
                matched = cm.rematch_request(req.request_id)
                if matched > req.num_cached_tokens:
                    req.num_cached_tokens = matched
                    req.num_computed_tokens = max(req.num_computed_tokens, matched)
                key = cm.next_block_key(req.request_id, req.num_computed_tokens)
                if key is not None:
                    if key in starting:
                        continue
                    starting.add(key)
            remaining = req.remaining_prefill
            if remaining <= 0:
                # whole prompt is cached: recompute the last token to obtain logits
                req.num_computed_tokens = req.prompt_len - 1
                remaining = 1
            cost = remaining if not chunk else min(remaining, chunk)
            room = budget_p - used
            if prefill_cap is not None:
                room = min(room, prefill_cap - used)
            if room <= 0:
                break
            if cost > room:
                if not chunk and prefill_cap is None and used > 0 and cost <= budget_p:
                    continue        # unsliced prompts wait for a step with enough room of their own
                # a slice of the prompt; also without chunked prefill when the prompt is longer than any
                # step's budget, which would otherwise wait for ever
                cost = room
            last = cost == remaining
            if not last:
                req.is_chunked = True
            batch.append(ScheduledSeq(req, cost, req.num_computed_tokens, True, last))
            used += cost
        room = min(self.micro_batch_size - len(batch), budget - used)
        n_dec = min(len(decodes), room) if room > 0 else 0
        if self.align_rows > 1 and batch and prefill_cap is not None:
            # trim the last prompt slice so that the step's rows fill whole tiles (only when the slice
            # stays a slice: the rest of the prompt follows in the next batch)
            extra = (used + n_dec) % self.align_rows
            last = batch[-1]
            if extra and last.num_tokens > extra and used + n_dec > self.align_rows:
                last.num_tokens -= extra
                last.produces_token = False
                last.req.is_chunked = True
                used -= extra
        if n_dec > 0:
            for req in decodes[:n_dec]:
                batch.append(ScheduledSeq(req, 1, req.prompt_len + len(req.output_ids) - 1, False, True))
        now = time.time()
        for s in batch:
            s.req.ready_for_next_step = False
            s.req.last_updated_time = now
        return batch

    # ------------------------------------------------------------------ finish rules
    def finish_reason(self, req: Request, n_out: int, last_token: Optional[int]) -> Optional[RequestStatus]:
        """Why the request ends after its ``n_out``-th generated token ``last_token`` (None = it goes on):
        abort, EOS / stop ids (honouring ``min_new_tokens``), ``max_new_tokens``, total length."""
        if req.abort:
            return RequestStatus.FINISHED_ABORT
        sp = req.sampling_params
        if n_out and n_out > sp.min_new_tokens and last_token is not None:
            if (not sp.ignore_eos and last_token in self.eos_token_ids) or \
                    (sp.stop_token_ids and last_token in sp.stop_token_ids):
                return RequestStatus.FINISHED_EOS
        if n_out >= sp.max_new_tokens or req.prompt_len + n_out >= req.max_total_length:
            return RequestStatus.FINISHED_MAX_LENGTH
        return None

    def ends_by_length_after(self, req: Request, n_out: int) -> bool:
        """Whether the request is over after ``n_out`` generated tokens whatever those tokens are."""
        return n_out >= req.sampling_params.max_new_tokens or req.prompt_len + n_out >= req.max_total_length

    def check_and_update_request_status(self, req: Request) -> bool:
        """EOS / stop ids (honouring ``min_new_tokens``) / max_new / max_total / abort."""
        if req.status in _FINISHED_STATES:
            self.evict_request(req.request_id)
            return True
        if req.abort:
            req.update_status(RequestStatus.FINISHED_ABORT)
            self.evict_request(req.request_id)
            return True
        if not self.is_first_peer:
            return False
        # runs once per request and step: plain attribute reads instead of the Request properties
        sp = req.sampling_params
        out = req.output_ids
        n_out = len(out)
        finished = False
        if n_out > sp.min_new_tokens and n_out:
            last = out[-1]
            if (not sp.ignore_eos and last in self.eos_token_ids) or (sp.stop_token_ids and last in sp.stop_token_ids):
                req.update_status(RequestStatus.FINISHED_EOS)
                finished = True
        if not finished and (n_out >= sp.max_new_tokens or req.prompt_len + n_out >= req.max_total_length):
            req.update_status(RequestStatus.FINISHED_MAX_LENGTH)
            finished = True
        if finished:
            self.evict_request(req.request_id)
        return finished
