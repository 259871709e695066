"""Free-list allocators for KV blocks and per-request state slots.

Same contract as the reference's ``BlockAllocator`` / ``SlotAllocator``
(``src/parallax/server/cache/allocator.py:8-72``): all-or-nothing multi-block allocation,
``-1`` / empty list on exhaustion, double frees are ignored with a warning.
"""

from __future__ import annotations

import logging

import numpy as np

logger = logging.getLogger(__name__)


class BlockAllocator:
    def __init__(self, num_blocks: int):
        self.num_blocks = int(num_blocks)
        # stack of free ids; low ids are handed out first
        self._free = np.arange(self.num_blocks - 1, -1, -1, dtype=np.int32)
        self._top = self.num_blocks
        self._is_free = np.ones(self.num_blocks, dtype=bool)

    def get_num_free_blocks(self) -> int:
        return self._top

    def allocate(self, n: int = 1) -> list[int]:
        if n <= 0:
            return []
        if n > self._top:
            return []
        out = self._free[self._top - n:self._top][::-1].copy()
        self._top -= n
        self._is_free[out] = False
        return out.tolist()

    def allocate_np(self, n: int) -> np.ndarray | None:
        if n > self._top:
            return None
        out = self._free[self._top - n:self._top][::-1].copy()
        self._top -= n
        self._is_free[out] = False
        return out

    def free(self, blocks) -> None:
        for b in blocks:
            b = int(b)
            if b < 0 or b >= self.num_blocks:
                logger.warning("free of out-of-range block %d ignored", b)
                continue
            if self._is_free[b]:
                logger.warning("double free of block %d ignored", b)
                continue
            self._is_free[b] = True
            self._free[self._top] = b
            self._top += 1


class SlotAllocator:
    def __init__(self, num_slots: int):
        self.num_slots = int(num_slots)
        self._free = list(range(self.num_slots - 1, -1, -1))
        self._used: set[int] = set()

    def get_num_free_slots(self) -> int:
        return len(self._free)

    def allocate(self) -> int:
        if not self._free:
            return -1
        s = self._free.pop()
        self._used.add(s)
        return s

    def free(self, slot: int) -> None:
        if slot not in self._used:
            logger.warning("double free of slot %d ignored", slot)
            return
        self._used.discard(slot)
        self._free.append(slot)
