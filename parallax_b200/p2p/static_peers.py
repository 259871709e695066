"""Pipeline peers without a scheduler: every node is started with its layer range and the addresses of some other
nodes, and the nodes find the chain themselves.

The reference lets developers skip the scheduler: each node gets ``--start-layer / --end-layer`` and finds the others
through the peer-to-peer overlay seeded with ``--initial-peers``
(``docs/user_guide/quick_start.md`` "Skipping Scheduler", ``src/parallax/p2p/server.py:631-648`` routing by layer
range). Here the overlay is plain HTTP: a node answers ``GET /peer/info`` with its id, address, layer range and the
addresses it knows; starting from the seeds a node walks those answers until it knows every reachable peer. The first
node (the one whose range starts at layer 0) chains peers by layer range into the routing table of each request.
"""

from __future__ import annotations

import logging
import threading
import time
from typing import Callable, Optional

logger = logging.getLogger(__name__)


def _http_get_json(url: str, timeout_s: float = 3.0) -> dict:
    import httpx

    return httpx.get(url, timeout=timeout_s, trust_env=False).json()


class StaticPeers:
    def __init__(self, node_id: str, url: str, start_layer: int, end_layer: int, seeds: list[str],
                 http_get: Callable[[str], dict] = _http_get_json, refresh_s: float = 5.0):
        self.info = {"node_id": node_id, "url": url.rstrip("/"), "start_layer": int(start_layer), "end_layer": int(end_layer)}
        self.seeds = [s if "://" in s else f"http://{s}" for s in seeds if s]
        self.http_get = http_get
        self.refresh_s = refresh_s
        self.known: dict[str, dict] = {node_id: dict(self.info)}      # node id -> info
        self._last = 0.0
        self._lock = threading.Lock()

    # ---- what this node tells others
    def describe(self) -> dict:
        with self._lock:
            urls = sorted({p["url"] for p in self.known.values()} | {s.rstrip("/") for s in self.seeds})
        return dict(self.info, peers=urls)

    # ---- discovery
    def refresh(self, force: bool = False) -> None:
        """Walk ``/peer/info`` from the seeds and from every peer learnt on the way (unreachable ones are skipped)."""
        if not force and time.time() - self._last < self.refresh_s:
            return
        self._last = time.time()
        todo = [s.rstrip("/") for s in self.seeds]
        with self._lock:
            todo += [p["url"] for p in self.known.values()]
        seen = {self.info["url"]}
        while todo:
            url = todo.pop()
            if url in seen:
                continue
            seen.add(url)
            try:
                d = self.http_get(url + "/peer/info")
            except Exception as e:
                logger.debug("peer %s not reachable: %s", url, e)
                continue
            if not isinstance(d, dict) or "node_id" not in d:
                continue
            with self._lock:
                self.known[d["node_id"]] = {k: d[k] for k in ("node_id", "url", "start_layer", "end_layer") if k in d}
                self.known[d["node_id"]].setdefault("url", url)
            todo += [u.rstrip("/") for u in d.get("peers") or []]

    def node_addresses(self) -> dict[str, str]:
        self.refresh()
        with self._lock:
            return {nid: p["url"] for nid, p in self.known.items()}

    def route(self, num_layers: int) -> Optional[list[str]]:
        """Node ids covering ``[0, num_layers)`` in order, or None while some range is missing."""
        for attempt in range(2):
            with self._lock:
                by_start: dict[int, dict] = {}
                for p in self.known.values():
                    if "start_layer" in p and (p["start_layer"] not in by_start or p["node_id"] == self.info["node_id"]):
                        by_start[p["start_layer"]] = p
            table, at = [], 0
            while at < num_layers and at in by_start and by_start[at]["end_layer"] > at:
                table.append(by_start[at]["node_id"])
                at = by_start[at]["end_layer"]
            if at >= num_layers:
                return table
            if attempt == 0:
                self.refresh(force=True)
        return None


class StaticAgent:
    """What :class:`parallax_b200.p2p.node_runtime.NodeRuntime` needs from a node agent, without a scheduler."""

    def __init__(self, peers: StaticPeers):
        self.node_id = peers.info["node_id"]
        self.scheduler = peers              # node_addresses()
        self.peers = peers
        self.on_refit = None
