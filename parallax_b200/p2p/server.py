"""Node-side cluster agent: join, heartbeat, allocation changes, peer-to-peer packet transport.

Replaces the reference's Lattica/libp2p node server (``src/parallax/p2p/server.py:341-958``)
with plain HTTP, which is sufficient inside a rack:

* ``SchedulerClient``   - ``/node/join``, ``/node/update``, ``/node/leave`` on the cluster backend;
* ``NodeAgent``         - joins, publishes the allocation into the node's SharedState, sends a
                          heartbeat every 10 s with load and latency metrics, flags allocation
                          changes (the launcher then restarts the executor with the new layer
                          range) and hands weight-refit requests to the executor;
* ``PeerTransport``     - ships ForwardRequest messages to the next peer's ``/pp_forward`` and
                          abort notices to ``/pp_abort``; keeps 3 refit versions on disk.
"""

from __future__ import annotations

import logging
import os
import threading
import time
import uuid
from typing import Callable, Optional

from parallax_b200.utils.hardware import HardwareInfo
from parallax_b200.utils.shared_state import SharedState

logger = logging.getLogger(__name__)

# seconds between heartbeats (the reference's node_update period); PARALLAX_HEARTBEAT_INTERVAL_S overrides it
HEARTBEAT_INTERVAL_S = float(os.environ.get("PARALLAX_HEARTBEAT_INTERVAL_S", "10"))


class SchedulerClient:
    def __init__(self, scheduler_addr: str, timeout: float = 310.0, http=None):
        base = scheduler_addr if scheduler_addr.startswith("http") else f"http://{scheduler_addr}"
        self.base = base.rstrip("/")
        self.timeout = timeout
        self._http = http

    def _post(self, path: str, payload: dict) -> dict:
        if self._http is not None:
            r = self._http.post(self.base + path, json=payload)
        else:
            import httpx

            r = httpx.post(self.base + path, json=payload, timeout=self.timeout, trust_env=False)
        r.raise_for_status()
        return r.json()

    def node_join(self, info: dict) -> dict:
        return self._post("/node/join", info)

    def node_update(self, info: dict) -> tuple[dict, dict]:
        d = self._post("/node/update", info)
        return d.get("layer_allocation") or {}, d.get("refit_request") or {}

    def node_leave(self, node_id: str) -> dict:
        return self._post("/node/leave", {"node_id": node_id})

    def node_addresses(self) -> dict[str, str]:
        """node id -> base URL of every node the scheduler knows (for peer-to-peer packets)."""
        return self._post("/node/addresses", {})


def _http_rtt_ms(url: str, timeout_s: float = 1.0) -> Optional[float]:
    import httpx

    t0 = time.perf_counter()
    r = httpx.get(url.rstrip("/") + "/health", timeout=timeout_s, trust_env=False)
    if r.status_code >= 500:
        return None
    return (time.perf_counter() - t0) * 1e3


class NodeAgent:
    def __init__(self, scheduler: SchedulerClient, shared_state: SharedState, http_addr: str,
                 node_id: Optional[str] = None, hardware: Optional[HardwareInfo] = None,
                 max_batch_size: int = 8, max_sequence_length: int = 32768, param_mem_ratio: float = 0.65,
                 kvcache_mem_ratio: float = 0.25, start_layer: Optional[int] = None,
                 end_layer: Optional[int] = None, on_refit: Optional[Callable[[dict], None]] = None,
                 heartbeat_interval_s: float = HEARTBEAT_INTERVAL_S,
                 probe: Optional[Callable[[str], Optional[float]]] = None):
        """``probe(url) -> round-trip ms or None``: how the agent measures the way to another node (default: a timed
        ``GET <url>/health``)."""
        self.scheduler = scheduler
        self.probe = probe or _http_rtt_ms
        self._rtt_at: dict[str, float] = {}
        self._rtt_missing = False
        self.state = shared_state
        self.http_addr = http_addr
        self.node_id = node_id or f"node-{uuid.uuid4().hex[:12]}"
        self.hardware = hardware or HardwareInfo.detect()
        self.max_batch_size = max_batch_size
        self.max_sequence_length = max_sequence_length
        self.param_mem_ratio, self.kvcache_mem_ratio = param_mem_ratio, kvcache_mem_ratio
        self.manual_range = (start_layer, end_layer) if start_layer is not None and end_layer is not None else None
        self.on_refit = on_refit
        self.interval = heartbeat_interval_s
        self.rtt_to_nodes: dict[str, float] = {}
        self.last_refit_time = 0.0
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None

    def node_info(self, is_active: bool = True) -> dict:
        hw = self.hardware.dumps()
        hw["node_id"] = self.node_id
        m = self.state.get_metrics()
        info = {"node_id": self.node_id, "http_addr": self.http_addr, "hardware": hw,
                "kvcache_mem_ratio": self.kvcache_mem_ratio, "param_mem_ratio": self.param_mem_ratio,
                "max_concurrent_requests": self.max_batch_size, "max_sequence_length": self.max_sequence_length,
                "is_active": is_active, "current_requests": m.get("current_requests", 0),
                "layer_latency_ms": m.get("layer_latency_ms"), "rtt_to_nodes": self.rtt_to_nodes or None,
                "last_refit_time": self.last_refit_time}
        if self.manual_range is not None:
            info.update(manual_layer_assignment=True, start_layer=self.manual_range[0], end_layer=self.manual_range[1])
        return info

    def _apply_allocation(self, alloc: dict) -> bool:
        """Publish an allocation; True if it differs from what the executor is running."""
        if not alloc:
            return False
        cur = self.state.get_model_info()
        changed = (cur["block_start_index"], cur["block_end_index"], cur["model_name"]) != (
            alloc.get("start_layer"), alloc.get("end_layer"), alloc.get("model_name"))
        if changed:
            first = cur["block_start_index"] is None
            self.state.update(model_name=alloc.get("model_name"), block_start_index=alloc.get("start_layer"),
                              block_end_index=alloc.get("end_layer"), tp_size=alloc.get("tp_size"),
                              enable_weight_refit=alloc.get("enable_weight_refit"),
                              weight_refit_mode=alloc.get("weight_refit_mode"),
                              _layer_allocation_changed=not first)
            if not first:
                self.state.set_status("initializing")
        return changed

    def join(self) -> dict:
        alloc = self.scheduler.node_join(self.node_info(is_active=False))
        self._apply_allocation(alloc)
        return alloc

    def measure_rtts(self, refresh_s: float = 60.0) -> None:
        """Round-trip times to the other nodes of the cluster, which the scheduler needs to price a pipeline's
        hops (the reference reads them from its peer-to-peer layer, ``src/parallax/p2p/server.py:867-905``):
        peers are learnt from the scheduler and probed at most once per ``refresh_s``; one that does not answer
        yet stays unknown and is tried again with the next heartbeat."""
        try:
            peers = self.scheduler.node_addresses() or {}
        except Exception as e:
            logger.debug("no peer addresses yet: %s", e)
            return
        now = time.time()
        missing = False
        for nid, url in peers.items():
            if nid == self.node_id or not url:
                continue
            if nid in self.rtt_to_nodes and now - self._rtt_at.get(nid, 0.0) < refresh_s:
                continue
            ms = None
            try:
                ms = self.probe(url)
            except Exception:
                ms = None
            if ms is None:
                missing = True
                continue
            self.rtt_to_nodes[nid] = float(ms)
            self._rtt_at[nid] = now
        for nid in [n for n in self.rtt_to_nodes if n not in peers]:
            self.rtt_to_nodes.pop(nid, None)
        self._rtt_missing = missing

    def heartbeat_once(self) -> tuple[dict, dict]:
        self.measure_rtts()
        active = self.state.get_status() == "available"
        alloc, refit = self.scheduler.node_update(self.node_info(is_active=active))
        self._apply_allocation(alloc)
        if refit and self.on_refit is not None:
            try:
                self.on_refit(refit)
                self.last_refit_time = float(refit.get("time_stamp", time.time()))
            except Exception as e:
                logger.exception("weight refit failed: %s", e)
        return alloc, refit

    def start(self) -> None:
        def loop():
            wait = 0.5          # the first beat follows the join at once: it carries the first measured hops
            while not self._stop.wait(wait):
                try:
                    self.heartbeat_once()
                except Exception as e:
                    logger.warning("heartbeat failed: %s", e)
                # until every peer has answered a probe (nodes come up at different times) beat faster
                wait = min(self.interval, 2.0) if self._rtt_missing else self.interval

        self._thread = threading.Thread(target=loop, name="NodeHeartbeat", daemon=True)
        self._thread.start()

    def stop(self, leave: bool = True) -> None:
        self._stop.set()
        if leave:
            try:
                self.scheduler.node_leave(self.node_id)
            except Exception:
                pass


class PeerTransport:
    """Sends stage packets to other peers; ``resolve(node_id)`` maps a node id to its base URL."""

    def __init__(self, resolve: Callable[[str], Optional[str]], http=None, notify_url: Optional[str] = None):
        self.resolve = resolve
        self._http = http
        self.notify_url = notify_url

    def _post(self, url: str, body: bytes) -> None:
        if self._http is not None:
            self._http.post(url, content=body, headers={"content-type": "application/msgpack"})
            return
        import httpx

        # a peer that is gone fails the connect at once; one that is busy may take long to answer
        httpx.post(url, content=body, headers={"content-type": "application/msgpack"},
                   timeout=httpx.Timeout(600.0, connect=5.0), trust_env=False)

    def send_forward(self, packets, self_id: str) -> list:
        """Group packets by their next hop in the routing table and ship one message per hop. Returns the packets
        that could not be delivered (the next peer is gone or unknown)."""
        from parallax_b200.p2p.message_util import request_to_proto

        groups: dict[str, list] = {}
        for pk in packets:
            table = pk.routing_table or []
            if self_id in table:
                nxt = table[(table.index(self_id) + 1) % len(table)]
            elif table:
                nxt = table[0]
            else:
                continue
            groups.setdefault(nxt, []).append(pk)
        undelivered = []
        for nid, group in groups.items():
            if not self.send_to(nid, group):
                undelivered.extend(group)
        return undelivered

    def send_to(self, nid: str, group: list) -> bool:
        """Ship packets to one peer. False when the peer has no address or does not answer."""
        from parallax_b200.p2p.message_util import request_to_proto

        url = self.resolve(nid)
        if url is None:
            logger.warning("no address for peer %s; %d packet(s) not delivered", nid, len(group))
            return False
        t0 = time.time()
        blob = request_to_proto(group)
        try:
            self._post(url.rstrip("/") + "/pp_forward", blob)
        except Exception as e:
            logger.warning("peer %s did not take %d packet(s): %s", nid, len(group), e)
            return False
        logger.debug("sent %.2f MB to %s in %.1f ms", len(blob) / 1e6, nid, (time.time() - t0) * 1e3)
        if self.notify_url:
            try:
                self._post(self.notify_url, blob[:0])
            except Exception:
                pass
        return True

    def send_abort(self, request_ids: list[str], routing_table: list[str], self_id: str) -> None:
        from parallax_b200.p2p.message_util import abort_request_to_proto

        blob = abort_request_to_proto(request_ids)
        for nid in routing_table:
            if nid == self_id:
                continue
            url = self.resolve(nid)
            if url:
                try:
                    self._post(url.rstrip("/") + "/pp_abort", blob)
                except Exception as e:
                    logger.warning("abort notice to %s failed: %s", nid, e)
