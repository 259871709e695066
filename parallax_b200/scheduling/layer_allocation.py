"""Layer allocation: which node hosts which contiguous decoder-layer range.

Implements the allocation algorithms of ``src/scheduling/layer_allocation.py`` of the
reference:

* per-layer KV "hosting power" bookkeeping with a min-heap (lightest layer first) used for
  dynamic joins and the global-rebalance trigger (coefficient of variation of layer loads);
* in-place **water-filling** rebalance of one pipeline: find lambda by bisection so that
  ``sum_i min(cap_i, lambda * power_i) = L``, floor, then hand out the remainder by largest
  fractional part (never beyond a node's capacity);
* a **greedy** allocator that builds pipelines from the largest nodes first with a one-step
  look-ahead, and a **dynamic-programming** allocator that picks the number of pipelines k
  maximising ``k^2 / s*(k)``, ``s*(k)`` being the minimum number of stages needed for k
  pipelines;
* turning-point trimming: drop layers that the latency-optimal layer-level path never uses.

On one NVSwitch box every node has the same capacity and zero RTT, so the results reduce to
equal splits; the general algorithms are kept because clusters of boxes are heterogeneous.
"""

from __future__ import annotations

import heapq
import logging
from dataclasses import dataclass, field
from math import floor
from typing import Literal, Optional

from parallax_b200.scheduling.model_info import ModelInfo
from parallax_b200.scheduling.node import Node
from parallax_b200.scheduling.node_management import NodeManager

logger = logging.getLogger(__name__)
INF = float("inf")


@dataclass
class LayerLoad:
    layer_id: int
    current_kv_size: int
    hosting_nodes: set = field(default_factory=set)

    def add_node(self, node: Node) -> None:
        mem = node.per_decoder_layer_kv_cache_memory
        if mem is None:
            raise ValueError("Node must have per_decoder_layer_kv_cache_memory")
        self.hosting_nodes.add(node.node_id)
        self.current_kv_size += mem

    def remove_node(self, node: Node) -> None:
        if node.node_id in self.hosting_nodes:
            mem = node.per_decoder_layer_kv_cache_memory
            if mem is None:
                raise ValueError("Node must have per_decoder_layer_kv_cache_memory")
            self.hosting_nodes.remove(node.node_id)
            self.current_kv_size -= mem

    def __lt__(self, other: "LayerLoad") -> bool:
        return (self.current_kv_size, self.layer_id) < (other.current_kv_size, other.layer_id)


def layer_level_best_path(nodes: list[Node], num_layers: int) -> list[int]:
    """Index (into ``nodes``) of the host chosen for every layer by a layer-level shortest
    path: cost = per-layer latency of the host + RTT whenever the host changes."""
    hosts = [[i for i, n in enumerate(nodes) if n.hosts_layer(l)] for l in range(num_layers)]
    if not hosts or any(not h for h in hosts):
        return []
    cost = {i: nodes[i].layer_latency_ms for i in hosts[0]}
    back: list[dict] = [{i: None for i in hosts[0]}]
    for l in range(1, num_layers):
        cur, bk = {}, {}
        for i in hosts[l]:
            best, arg = INF, None
            for j, c in cost.items():
                if c == INF:
                    continue
                t = c + (0.0 if i == j else nodes[j].get_rtt_to(nodes[i])) + nodes[i].layer_latency_ms
                if t < best:
                    best, arg = t, j
            cur[i], bk[i] = best, arg
        cost = cur
        back.append(bk)
    end = min(cost, key=lambda k: cost[k])
    path = [end]
    for l in range(num_layers - 1, 0, -1):
        prev = back[l][path[-1]]
        if prev is None:
            break
        path.append(prev)
    path.reverse()
    return path


def turning_points_of_path(nodes: list[Node], path: list[int]) -> list[tuple[str, int, str]]:
    """(node_id, layer, 'tail'|'head'): layers a node still hosts after (tail) / before (head)
    the optimal path has left / entered it."""
    out = []
    for l in range(1, len(path)):
        if path[l - 1] != path[l] and nodes[path[l - 1]].hosts_layer(l):
            out.append((nodes[path[l - 1]].node_id, l, "tail"))
    first = {}
    for l, idx in enumerate(path):
        first.setdefault(idx, l)
    for idx, l0 in first.items():
        n = nodes[idx]
        if n.start_layer is not None and l0 > n.start_layer:
            out.append((n.node_id, l0, "head"))
    return out


class BaseLayerAllocator:
    def __init__(self, model_info: ModelInfo, node_management: NodeManager, *,
                 dynamic_pipelines_router: bool = False, rebalance_threshold: float = 0.25,
                 water_filling_max_iterations: int = 40, trim_layers_on_turning_points: bool = False):
        self.model_info = model_info
        self.num_total_layers = model_info.num_layers
        self.node_management = node_management
        self.dynamic_pipelines_router = dynamic_pipelines_router
        self.rebalance_threshold = rebalance_threshold
        self.water_filling_max_iterations = water_filling_max_iterations
        self.trim_layers_on_turning_points = trim_layers_on_turning_points
        self.layer_to_load = {l: LayerLoad(l, 0) for l in range(self.num_total_layers)}
        self.layer_loads_heap: list[LayerLoad] = []
        self._update_layer_loads_heap()

    # ---- primitive moves
    def _update_layer_loads_heap(self) -> None:
        self.layer_loads_heap = list(self.layer_to_load.values())
        heapq.heapify(self.layer_loads_heap)

    def get_lightest_layer(self) -> Optional[LayerLoad]:
        return self.layer_loads_heap[0] if self.layer_loads_heap else None

    def allocate(self, node: Node, start_layer: int, end_layer: int) -> None:
        if end_layer <= start_layer:
            raise ValueError(f"Invalid allocation: start_layer {start_layer} >= end_layer {end_layer}")
        node.set_layer_allocation(start_layer, end_layer)
        self.node_management.activate([node.node_id])
        for l in range(start_layer, end_layer):
            if l not in self.layer_to_load:
                raise ValueError(f"Layer {l} not found in layer_to_load")
            self.layer_to_load[l].add_node(node)
        self._update_layer_loads_heap()

    def deallocate(self, node: Node) -> None:
        if node.start_layer is None or node.end_layer is None:
            return
        for l in range(node.start_layer, node.end_layer):
            if l in self.layer_to_load:
                self.layer_to_load[l].remove_node(node)
        self.node_management.standby([node.node_id])
        self._update_layer_loads_heap()

    def reallocate(self, node: Node, start_layer: int, end_layer: int) -> None:
        self.deallocate(node)
        self.allocate(node, start_layer, end_layer)

    def _end_layer_for(self, node: Node, start: int) -> int:
        first = start == 0
        end = min(start + node.get_decoder_layer_capacity(include_input_embed=first), self.num_total_layers)
        if end == self.num_total_layers:
            cap = node.get_decoder_layer_capacity(include_lm_head=True, include_input_embed=first)
            end = min(start + cap, self.num_total_layers)
        return end

    def dynamic_join(self, node: Node) -> None:
        """Attach a late joiner starting at the layer with the least KV hosting power."""
        lightest = self.get_lightest_layer()
        if lightest is None:
            raise ValueError("No layers to assign")
        start = lightest.layer_id
        self.allocate(node, start, self._end_layer_for(node, start))

    def allocate_from_standby(self) -> bool:  # overridden
        return False

    def allocate_standby_nodes(self) -> bool:
        if self.dynamic_pipelines_router:
            for node in self.node_management.standby_nodes:
                self.dynamic_join(node)
            return True
        return self.allocate_from_standby()

    # ---- rebalance trigger
    def should_global_rebalance(self) -> bool:
        """True when no full pipeline is left, or the per-layer KV hosting power is uneven
        (coefficient of variation above ``rebalance_threshold``)."""
        if not self.node_management.has_full_pipeline(self.num_total_layers):
            return True
        heap = self.layer_loads_heap
        if len(heap) < 2:
            return False
        total_mem = sum(n.hardware.num_gpus * n.hardware.memory_gb for n in self.node_management.nodes)
        if total_mem == 0:
            raise ValueError("Total cluster memory is zero")
        loads = [l.current_kv_size / total_mem for l in heap]
        avg = sum(loads) / len(loads)
        if avg == 0:
            return False
        var = sum((x - avg) ** 2 for x in loads) / len(loads)
        return (var ** 0.5) / avg > self.rebalance_threshold

    # ---- in-pipeline layer split
    def adjust_pipeline_layers(self, pipeline_nodes: list[Node], assume_sorted: bool = False,
                               power_type: Literal["flops", "bandwidth"] = "flops") -> None:
        """Water-filling split of all layers over the nodes of ONE pipeline."""
        L = self.num_total_layers
        if not pipeline_nodes or L <= 0:
            raise ValueError("No nodes or total layers is non-positive")
        nodes = pipeline_nodes if assume_sorted else sorted(
            pipeline_nodes, key=lambda n: n.get_decoder_layer_capacity(), reverse=True)
        n = len(nodes)
        for node in nodes:
            if node.start_layer is not None and node.end_layer is not None:
                self.deallocate(node)
        caps, power = [], []
        for i, node in enumerate(nodes):
            if i == 0:
                # (a pipeline of one node stores the embedding and the head)
                cap = node.get_decoder_layer_capacity(include_input_embed=True, include_lm_head=n == 1)
            elif i == n - 1:
                cap = node.get_decoder_layer_capacity(include_lm_head=True)
            else:
                cap = node.get_decoder_layer_capacity()
            if cap <= 0:
                raise ValueError(f"Node {node.node_id} has non-positive capacity: {cap}")
            caps.append(cap)
            power.append(node.hardware.tflops_fp16 if power_type == "flops" else node.hardware.memory_bandwidth_gbps)
        if sum(caps) < L:
            raise ValueError(f"Total capacity {sum(caps)} is less than total layers {L}")

        def filled(lam: float) -> float:
            return sum(min(caps[i], lam * power[i]) for i in range(n))

        lo, hi = 0.0, max(caps[i] / power[i] for i in range(n))
        for _ in range(self.water_filling_max_iterations):
            mid = 0.5 * (lo + hi)
            if filled(mid) >= L:
                hi = mid
            else:
                lo = mid
        target = [min(caps[i], hi * power[i]) for i in range(n)]
        counts = [min(caps[i], int(floor(target[i]))) for i in range(n)]
        remaining = L - sum(counts)
        if remaining < 0:
            raise ValueError(f"Remaining {remaining} is negative")
        # largest fractional part first; ties go to the earlier (larger) node
        for _, negi in sorted(((target[i] - counts[i], -i) for i in range(n)), reverse=True):
            if remaining == 0:
                break
            i = -negi
            if caps[i] - counts[i] > 0:
                counts[i] += 1
                remaining -= 1
        for i in range(n):  # anything still left goes wherever room remains
            if remaining == 0:
                break
            take = min(caps[i] - counts[i], remaining)
            counts[i] += take
            remaining -= take
        start = 0
        for node, c in zip(nodes, counts):
            if c <= 0:
                continue
            self.allocate(node, start, start + c)
            start += c
        if start != L:
            raise ValueError(f"Assignment did not cover all layers: assigned {start} of {L}")

    def adjust_pipeline_layers_greedy(self, pipeline_nodes: list[Node]) -> None:
        """Fill nodes front to back up to their capacity (no balancing)."""
        L = self.num_total_layers
        if not pipeline_nodes or L <= 0:
            raise ValueError("No nodes or total layers is non-positive")
        for node in pipeline_nodes:
            if node.start_layer is not None and node.end_layer is not None:
                self.deallocate(node)
        start, remaining = 0, L
        for node in pipeline_nodes:
            first = start == 0
            base = node.get_decoder_layer_capacity(include_input_embed=first)
            if base >= remaining:
                take = min(node.get_decoder_layer_capacity(include_input_embed=first, include_lm_head=True), remaining)
            else:
                take = min(base, remaining)
            if take <= 0:
                continue
            self.allocate(node, start, start + take)
            start += take
            remaining -= take
            if remaining == 0:
                break
        if remaining != 0:
            raise ValueError(f"Greedy assignment did not cover all layers: remaining {remaining}")

    def adjust_for_turning_points(self, num_layers: int) -> list[tuple[str, int, str]]:
        """Trim layers that the latency-optimal layer-level path does not use."""
        nodes = self.node_management.active_nodes
        if num_layers <= 0 or not nodes:
            return []
        path = layer_level_best_path(nodes, num_layers)
        if not path:
            return []
        turning = turning_points_of_path(nodes, path)
        by_id = {n.node_id: n for n in nodes}
        for nid, layer, kind in turning:
            n = by_id[nid]
            if kind == "tail":
                self.reallocate(n, n.start_layer, layer)
            else:
                self.reallocate(n, layer, n.end_layer)
        return turning


class GreedyLayerAllocator(BaseLayerAllocator):
    """Largest nodes first; one-step look-ahead keeps a big node for the next pipeline when a
    smaller one can finish the current pipeline just as well."""

    def __init__(self, *, look_ahead_enable: bool = True,
                 pipeline_rebalance_strategy: Literal["greedy", "water_filling"] = "water_filling", **kw):
        super().__init__(**kw)
        self._look_ahead_enable = look_ahead_enable
        self._pipeline_rebalance_strategy = pipeline_rebalance_strategy

    def allocate_from_standby(self) -> bool:
        L = self.model_info.num_layers
        pool = sorted(self.node_management.standby_nodes, key=lambda n: n.get_decoder_layer_capacity(), reverse=True)
        assigned_any = False
        while pool:
            total_cap = sum(n.get_decoder_layer_capacity() for n in pool)
            if total_cap < L:
                break
            members: list[Node] = []
            remaining, cap_left = L, total_cap
            while remaining > 0 and pool:
                first = not members
                pick = -1
                if self._look_ahead_enable and first and cap_left - remaining >= L + 1:
                    for i, cand in enumerate(pool):
                        c = cand.get_decoder_layer_capacity(include_lm_head=True)
                        if c >= remaining and cap_left - c >= L:
                            pick = i  # last match = smallest node that still closes the pipeline
                node = pool.pop(pick) if pick != -1 else pool.pop(0)
                members.append(node)
                cap = node.get_decoder_layer_capacity(include_input_embed=first)
                if remaining - cap <= 0:
                    cap = node.get_decoder_layer_capacity(include_input_embed=first, include_lm_head=True)
                remaining -= cap
                cap_left -= cap
            if remaining > 0 or not members:
                break
            if self._pipeline_rebalance_strategy == "greedy":
                self.adjust_pipeline_layers_greedy(members)
            else:
                self.adjust_pipeline_layers(members, assume_sorted=False)
            assigned_any = True
        if not assigned_any or not self.node_management.has_full_pipeline(self.num_total_layers):
            return False
        if self.trim_layers_on_turning_points:
            self.adjust_for_turning_points(self.num_total_layers)
        if self.dynamic_pipelines_router:
            self.allocate_standby_nodes()
        return True


class DynamicProgrammingLayerAllocator(BaseLayerAllocator):
    """Choose the number of pipelines k that maximises k^2 / s*(k)."""

    def __init__(self, *, alpha: float = 2.0, **kw):
        super().__init__(**kw)
        self.alpha = alpha

    def _min_stages(self, nodes: list[Node], k_target: int):
        """(s*, decisions): minimum stage count to build ``k_target`` pipelines from ``nodes``
        taken in order, and the per-state decision table for reconstruction."""
        L = self.model_info.num_layers
        n = len(nodes)
        cap = [x.get_decoder_layer_capacity() for x in nodes]
        cap_head = [x.get_decoder_layer_capacity(include_input_embed=True) for x in nodes]
        cap_tail = [x.get_decoder_layer_capacity(include_lm_head=True) for x in nodes]
        cap_solo = [x.get_decoder_layer_capacity(include_input_embed=True, include_lm_head=True) for x in nodes]
        suffix = [0] * (n + 1)
        for i in range(n - 1, -1, -1):
            suffix[i] = suffix[i + 1] + cap[i]
        memo: dict = {}
        decision: dict = {}

        def solve(i: int, open_res: tuple, done: int) -> float:
            key = (i, open_res, done)
            if key in memo:
                return memo[key]
            if done == k_target and not open_res:
                decision[key] = ("done",)
                memo[key] = 0
                return 0
            if i == n:
                memo[key] = INF
                return INF
            to_start = k_target - done - len(open_res)
            if (to_start < 0 or suffix[i] < sum(open_res) + max(0, to_start) * L
                    or done + len(open_res) + (n - i) < k_target):
                memo[key] = INF
                return INF
            best, act = solve(i + 1, open_res, done), ("skip",)
            for j, r in enumerate(open_res):  # extend open pipeline j with node i
                left = r - cap[i]
                closes = False
                if left <= 0:
                    left = r - cap_tail[i]  # the closing stage also stores norm + lm_head
                    closes = left <= 0
                rest = list(open_res)
                if closes:
                    rest.pop(j)
                    c = 1 + solve(i + 1, tuple(rest), done + 1)
                else:
                    rest[j] = left
                    rest.sort()
                    c = 1 + solve(i + 1, tuple(rest), done)
                if c < best:
                    best, act = c, ("assign", j, closes)
            if to_start > 0:  # open a new pipeline at node i
                # a node is a pipeline of its own only if the head fits beside the embedding as well; one that
                # falls short of that by the head alone opens a pipeline and leaves its last layer to the next node
                left = 0 if cap_solo[i] >= L else max(L - cap_head[i], 1)
                if left <= 0:
                    c = 1 + solve(i + 1, open_res, done + 1)
                    if c < best:
                        best, act = c, ("start", 0, True)
                else:
                    c = 1 + solve(i + 1, tuple(sorted(open_res + (left,))), done)
                    if c < best:
                        best, act = c, ("start", left, False)
            decision[key] = act
            memo[key] = best
            return best

        import sys
        old = sys.getrecursionlimit()
        sys.setrecursionlimit(max(old, 4 * n + 1000))
        try:
            s = solve(0, tuple(), 0)
        finally:
            sys.setrecursionlimit(old)
        return s, decision, (cap, cap_tail)

    def _reconstruct(self, nodes: list[Node], k: int, decision: dict, caps) -> list[list[Node]]:
        cap, cap_tail = caps
        pipelines: list[list[Node]] = [[] for _ in range(k)]
        open_list: list[tuple[int, list[Node]]] = []
        i = done = 0
        while i < len(nodes) and done < k:
            open_list.sort(key=lambda x: x[0])
            act = decision.get((i, tuple(r for r, _ in open_list), done))
            if act is None:
                break
            if act[0] == "assign":
                j, closes = act[1], act[2]
                r, seq = open_list[j]
                seq.append(nodes[i])
                left = r - cap[i]
                if left <= 0:
                    left = r - cap_tail[i]
                if closes or left <= 0:
                    pipelines[done].extend(seq)
                    open_list.pop(j)
                    done += 1
                else:
                    open_list[j] = (left, seq)
            elif act[0] == "start":
                if act[2]:
                    pipelines[done].append(nodes[i])
                    done += 1
                else:
                    open_list.append((act[1], [nodes[i]]))
            i += 1
        return pipelines

    def allocate_from_standby(self) -> bool:
        L = self.model_info.num_layers
        nodes = sorted(self.node_management.standby_nodes, key=lambda n: n.get_decoder_layer_capacity(), reverse=True)
        total_cap = sum(n.get_decoder_layer_capacity() for n in nodes)
        if L <= 0 or not nodes or total_cap < L:
            logger.warning("[DPLayerAllocator] Insufficient resources: nodes=%d layers=%d cap=%d",
                           len(nodes), L, total_cap)
            return False
        best = None
        for k in range(1, min(len(nodes), total_cap // L) + 1):
            s, decision, caps = self._min_stages(nodes, k)
            if s < INF:
                score = (k ** self.alpha) / s
                if best is None or score > best[0]:
                    best = (score, k, decision, caps)
        if best is None:
            return False
        _, k, decision, caps = best
        for members in self._reconstruct(nodes, k, decision, caps):
            if members:
                self.adjust_pipeline_layers(members, assume_sorted=False)
        if not self.node_management.has_full_pipeline(self.num_total_layers):
            return False
        if self.trim_layers_on_turning_points:
            self.adjust_for_turning_points(self.num_total_layers)
        if self.dynamic_pipelines_router:
            self.allocate_standby_nodes()
        return True
