"""Device-side description of one forward step (a mixed prefill + decode batch).

Token rows are laid out as ``[prefill tokens of seq 0, seq 1, ..., decode tokens]``. All
index tensors are packed into ONE pinned host buffer and shipped with a single
host-to-device copy per step; the views below alias a device mirror of that buffer.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import numpy as np
import torch


@dataclass
class ForwardBatch:
    num_tokens: int = 0
    num_prefill_tokens: int = 0
    num_prefill_seqs: int = 0
    num_decode: int = 0
    input_ids: Optional[torch.Tensor] = None      # int32 [T] (first stage only)
    positions: Optional[torch.Tensor] = None      # int32 [T]
    slot_mapping: Optional[torch.Tensor] = None   # int64 [T]
    # prefill part
    p_cu_q: Optional[torch.Tensor] = None         # int32 [Bp+1]
    p_ctx_lens: Optional[torch.Tensor] = None     # int32 [Bp]
    p_block_tables: Optional[torch.Tensor] = None  # int32 [Bp, MB]
    p_max_q: int = 0
    p_max_ctx: int = 0
    # decode part
    d_ctx_lens: Optional[torch.Tensor] = None     # int32 [Bd]
    d_block_tables: Optional[torch.Tensor] = None  # int32 [Bd, MB]
    d_max_ctx: int = 0
    # rows whose logits are needed (last token of finished prefills + every decode row)
    logit_rows: Optional[torch.Tensor] = None     # int32 [n_logits]
    num_logits: int = 0
    # every sequence of the step (prefill sequences, then one per decode row)
    seq_cu: Optional[torch.Tensor] = None         # int32 [B+1] token ranges
    seq_slots: Optional[torch.Tensor] = None      # int32 [B] request rows (state slots of linear-attention layers)
    h2d_bytes: int = 0
    # model-specific extras (e.g. linear-attention state slots)
    extras: dict = field(default_factory=dict)


class BatchBuilder:
    """Packs per-step index arrays into one pinned buffer and mirrors it on the device."""

    def __init__(self, device: torch.device, max_tokens: int, max_seqs: int, max_blocks_per_seq: int):
        self.device = device
        self.max_tokens = max_tokens
        self.max_seqs = max_seqs
        self.max_blocks = max_blocks_per_seq
        # int32 words: ids T, positions T, slots 2T (as int64), cu_q S+1, p_ctx S, d_ctx S,
        # logit_rows S, block tables 2*S*MB (prefill and decode parts never overlap, but keep
        # room for both so that offsets are static)
        words = 4 * max_tokens + 6 * max_seqs + 16 + max_seqs * max_blocks_per_seq + 64
        self.capacity = words
        pin = device.type == "cuda"
        self.host = torch.empty(words, dtype=torch.int32, pin_memory=pin)
        self.host_np = self.host.numpy()
        self.dev = torch.empty(words, dtype=torch.int32, device=device)
        self._copied = None     # CUDA event: the last host-to-device copy out of the pinned buffer has run

    def build(
        self,
        input_ids: Optional[np.ndarray],
        positions: np.ndarray,
        slots: np.ndarray,
        p_q_lens: list[int],
        p_ctx_lens: list[int],
        p_tables: Optional[np.ndarray],
        d_ctx_lens: np.ndarray,
        d_tables: Optional[np.ndarray],
        logit_rows: np.ndarray,
        seq_rows: Optional[np.ndarray] = None,
        extra: Optional[dict] = None,
    ) -> ForwardBatch:
        if self._copied is not None:
            # the pinned buffer is about to be rewritten: the asynchronous copy of its previous
            # content must have executed (a caller may run several steps ahead of the device)
            self._copied.synchronize()
        T = int(positions.shape[0])
        Bp, Bd = len(p_q_lens), int(d_ctx_lens.shape[0])
        Tp = int(sum(p_q_lens))
        h = self.host_np
        off = 0

        def put(arr: np.ndarray, align: int = 4) -> tuple[int, int]:
            nonlocal off
            off = (off + align - 1) // align * align
            n = int(arr.size)
            if off + n > self.capacity:
                raise ValueError("forward batch exceeds the builder capacity")
            h[off:off + n] = arr.reshape(-1)
            start = off
            off += n
            return start, n

        spans = {}
        if input_ids is not None:
            spans["ids"] = put(input_ids.astype(np.int32, copy=False))
        spans["pos"] = put(positions.astype(np.int32, copy=False))
        spans["slots"] = put(slots.astype(np.int64, copy=False).view(np.int32))
        if Bp:
            cu = np.zeros(Bp + 1, dtype=np.int32)
            np.cumsum(np.asarray(p_q_lens, dtype=np.int32), out=cu[1:])
            spans["cu_q"] = put(cu)
            spans["p_ctx"] = put(np.asarray(p_ctx_lens, dtype=np.int32))
            spans["p_bt"] = put(p_tables.astype(np.int32, copy=False))
        if Bd:
            spans["d_ctx"] = put(d_ctx_lens.astype(np.int32, copy=False))
            spans["d_bt"] = put(d_tables.astype(np.int32, copy=False))
        spans["rows"] = put(logit_rows.astype(np.int32, copy=False))
        if seq_rows is not None:
            lens = np.concatenate([np.asarray(p_q_lens, dtype=np.int32), np.ones(Bd, dtype=np.int32)])
            scu = np.zeros(Bp + Bd + 1, dtype=np.int32)
            np.cumsum(lens, out=scu[1:])
            spans["seq_cu"] = put(scu)
            spans["seq_slots"] = put(seq_rows.astype(np.int32, copy=False))
        for name, arr in (extra or {}).items():      # further int32 arrays that ride in the same copy
            spans["x_" + name] = put(np.asarray(arr, dtype=np.int32))
        total = off
        self.dev[:total].copy_(self.host[:total], non_blocking=True)
        if self.device.type == "cuda":
            if self._copied is None:
                self._copied = torch.cuda.Event()
            self._copied.record()

        def view(key):
            s, n = spans[key]
            return self.dev[s:s + n]

        fb = ForwardBatch(num_tokens=T, num_prefill_tokens=Tp, num_prefill_seqs=Bp, num_decode=Bd)
        fb.h2d_bytes = total * 4
        if input_ids is not None:
            fb.input_ids = view("ids")
        fb.positions = view("pos")
        fb.slot_mapping = view("slots").view(torch.int64)
        if Bp:
            fb.p_cu_q = view("cu_q")
            fb.p_ctx_lens = view("p_ctx")
            fb.p_block_tables = view("p_bt").view(Bp, -1)
            fb.p_max_q = int(max(p_q_lens))
            fb.p_max_ctx = int(max(p_ctx_lens))
        if Bd:
            fb.d_ctx_lens = view("d_ctx")
            fb.d_block_tables = view("d_bt").view(Bd, -1)
            fb.d_max_ctx = int(d_ctx_lens.max())
        fb.logit_rows = view("rows")
        if seq_rows is not None:
            fb.seq_cu = view("seq_cu")
            fb.seq_slots = view("seq_slots")
        fb.num_logits = int(logit_rows.shape[0])
        for name in (extra or {}):
            fb.extras[name] = view("x_" + name)
        return fb
