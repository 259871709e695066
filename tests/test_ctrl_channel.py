"""The in-box control channel: ordered delivery to every reader, flow control, oversize messages, liveness words."""

import os
import threading

import numpy as np

from parallax_b200.parallel.ctrl_channel import CtrlChannel


def test_messages_reach_every_reader_in_order_and_oversize_ones_travel_in_parts():
    name = f"pxl_test_ctrl_{os.getpid()}"
    w = CtrlChannel(name, create=True, n_readers=2, slots=4, slot_bytes=4096)
    readers = [CtrlChannel(name, create=False, n_readers=2, reader_index=i, slots=4, slot_bytes=4096) for i in range(2)]
    big = {"cmd": "step", "schema": "x" * 50_000, "arr": np.arange(3000, dtype=np.int32)}     # 15 slots of a 4-slot ring
    msgs = [{"i": 0}, big, {"i": 2}] + [{"i": k} for k in range(3, 12)]
    got = [[], []]

    def read(i):
        for _ in msgs:
            got[i].append(readers[i].receive(timeout_s=20))

    threads = [threading.Thread(target=read, args=(i,)) for i in range(2)]
    for t in threads:
        t.start()
    for m in msgs:
        w.publish(m, timeout_s=20)          # blocks while a reader is more than the ring behind
    for t in threads:
        t.join(30)
    try:
        for g in got:
            assert len(g) == len(msgs)
            assert g[0] == {"i": 0} and g[2] == {"i": 2} and g[-1] == {"i": 11}
            assert g[1]["schema"] == big["schema"] and np.array_equal(g[1]["arr"], big["arr"])
        assert w.stale_readers(5.0) == []
        readers[1].report_status(105)
        assert w.failed_readers() == {1: 105} and w.failed_readers() == {}
    finally:
        for r in readers:
            r.close()
        w.close()
