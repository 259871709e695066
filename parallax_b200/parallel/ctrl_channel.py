"""Single-box control channel: rank 0 publishes step plans, every other rank reads them.

A ring of fixed-size slots in POSIX shared memory; each slot carries a sequence number that the
writer stores last, readers poll it. Per-reader cursors in the same segment give the writer flow
control (a slot is reused only after every reader has consumed it). One plan is a pickled dict of
small numpy arrays (tens of KB), so publishing costs one memcpy instead of a collective per step.

This is the in-box replacement of the reference's python-object broadcast to its tensor-parallel
ranks over ``multiprocessing.Pipe`` (``src/parallax/server/executor/sglang_executor.py:560-571``).
"""

from __future__ import annotations

import pickle
import time
from multiprocessing import shared_memory

import numpy as np

# header bytes: [0:8] reserved, 7 reader cursors (int64), 7 reader heartbeats (int64 ns) from byte 64,
# 7 reader device-status words (int64, 0 = healthy) from byte 128
_HDR = 256
_SLOT_HDR = 16       # seq (int64), nbytes (int64; bit 40 set: the message continues in the next slot)
_MORE = 1 << 40
_CREATED_HERE: set = set()      # segments created by this process


class CtrlChannel:
    def __init__(self, name: str, create: bool, n_readers: int, reader_index: int = -1, slots: int = 32,
                 slot_bytes: int = 1 << 20):
        self.slots, self.slot_bytes, self.n_readers, self.reader_index = slots, slot_bytes, n_readers, reader_index
        size = _HDR + slots * (slot_bytes + _SLOT_HDR)
        if create:
            self.shm = shared_memory.SharedMemory(name=name, create=True, size=size)
            _CREATED_HERE.add(name)
            self.shm.buf[:_HDR] = bytes(_HDR)
            for i in range(slots):
                o = _HDR + i * (slot_bytes + _SLOT_HDR)
                self.shm.buf[o:o + _SLOT_HDR] = bytes(_SLOT_HDR)
        else:
            self.shm = shared_memory.SharedMemory(name=name, create=False)
            if name not in _CREATED_HERE:      # (writer and reader in one process share one tracker entry)
                try:        # the creating process owns the segment; readers must not unlink it at exit
                    from multiprocessing import resource_tracker

                    resource_tracker.unregister(self.shm._name, "shared_memory")
                except Exception:
                    pass
        self.owner = create
        self.cursors = np.ndarray((7,), dtype=np.int64, buffer=self.shm.buf, offset=8)
        self.beats = np.ndarray((7,), dtype=np.int64, buffer=self.shm.buf, offset=64)
        self.status = np.ndarray((7,), dtype=np.int64, buffer=self.shm.buf, offset=128)
        if not create:
            self.beat()
        self.seq = 0      # writer: messages published; reader: messages consumed

    def _slot(self, seq: int):
        o = _HDR + (seq % self.slots) * (self.slot_bytes + _SLOT_HDR)
        hdr = np.ndarray((2,), dtype=np.int64, buffer=self.shm.buf, offset=o)
        return hdr, o + _SLOT_HDR

    # ------------------------------------------------------------------ writer (rank 0)
    def publish(self, obj, timeout_s: float = 600.0) -> None:
        """A message larger than a slot (a step plan that carries a large JSON schema, say) travels as several
        slots in a row; every part but the last has the ``_MORE`` bit set in its length word."""
        data = pickle.dumps(obj, protocol=pickle.HIGHEST_PROTOCOL)
        for o in range(0, max(len(data), 1), self.slot_bytes):
            part = data[o:o + self.slot_bytes]
            self._publish_part(part, o + len(part) < len(data), timeout_s)

    def _publish_part(self, data: bytes, more: bool, timeout_s: float) -> None:
        nxt = self.seq + 1
        t0 = time.monotonic()
        while self.n_readers and nxt - int(self.cursors[: self.n_readers].min()) > self.slots:
            if time.monotonic() - t0 > timeout_s:
                raise TimeoutError("a reader of the control channel stopped consuming")
            time.sleep(0.0002)
        hdr, off = self._slot(nxt)
        self.shm.buf[off:off + len(data)] = data
        hdr[1] = len(data) | (_MORE if more else 0)
        hdr[0] = nxt          # published last: readers poll this word
        self.seq = nxt

    # ------------------------------------------------------------------ readers
    def receive(self, timeout_s: float = 600.0):
        parts = []
        while True:
            data, more = self._receive_part(timeout_s)
            parts.append(data)
            if not more:
                return pickle.loads(parts[0] if len(parts) == 1 else b"".join(parts))

    def _receive_part(self, timeout_s: float):
        nxt = self.seq + 1
        hdr, off = self._slot(nxt)
        t0 = time.monotonic()
        spins = 0
        while int(hdr[0]) != nxt:
            spins += 1
            if spins > 2000:             # stay hot for a moment, then yield the core
                time.sleep(0.0001)
                if spins % 512 == 0:
                    self.beat()          # an idle reader is still alive
                    if time.monotonic() - t0 > timeout_s:
                        raise TimeoutError("no control message from rank 0")
        word = int(hdr[1])
        n = word & (_MORE - 1)
        data = bytes(self.shm.buf[off:off + n])
        self.seq = nxt
        self.cursors[self.reader_index] = nxt
        self.beat()
        return data, bool(word & _MORE)

    # ------------------------------------------------------------------ liveness
    def beat(self) -> None:
        """Reader: publish "alive now" (wall-clock ns; all processes share the box's clock)."""
        if self.reader_index >= 0:
            self.beats[self.reader_index] = time.time_ns()

    def stale_readers(self, max_age_s: float) -> list[int]:
        """Writer: indices of readers whose last heartbeat is older than ``max_age_s`` (0 = never seen)."""
        now = time.time_ns()
        return [i for i in range(self.n_readers) if now - int(self.beats[i]) > max_age_s * 1e9]

    def report_status(self, code: int) -> None:
        """Reader: publish a non-zero device status word (kept until the writer clears it)."""
        if self.reader_index >= 0 and code:
            self.status[self.reader_index] = code

    def failed_readers(self) -> dict[int, int]:
        """Writer: {reader index: status code} of the readers that reported a device error; clears them."""
        out = {}
        for i in range(self.n_readers):
            c = int(self.status[i])
            if c:
                out[i] = c
                self.status[i] = 0
        return out

    def close(self) -> None:
        self.cursors = None
        self.beats = None
        self.status = None
        try:
            self.shm.close()
            if self.owner:
                self.shm.unlink()
        except (FileNotFoundError, BufferError):
            pass
