"""Block-granular radix prefix cache.

One tree node represents one FULL KV block (``block_size`` tokens) and is keyed by the
block's token tuple under its parent. Matching walks whole blocks only; requests pin the
nodes they use through lock reference counts; unpinned leaves are evicted in LRU order and
report the freed block (and, for hybrid linear-attention models, the state slot snapshot)
through callbacks. Behavioural counterpart:
``src/parallax/server/block_radix_cache.py:74-310``.

Eviction does not walk the tree: the number of unpinned nodes is kept as a counter, and a lazy
min-heap holds every node at the moment it becomes an unpinned leaf (inserted, unpinned, or left
without children). Entries are checked when popped - a node that was touched, pinned, extended or
deleted since is skipped or pushed back with its current time stamp - so evicting k blocks costs
O(k log n) however large the tree is.
"""

from __future__ import annotations

import heapq
import itertools
import time
from typing import Callable, Optional


class BlockNode:
    __slots__ = ("key", "block_id", "parent", "children", "lock_ref", "last_access", "linear_slot",
                 "alive")

    def __init__(self, key: Optional[tuple], block_id: int, parent: Optional["BlockNode"]):
        self.key = key
        self.block_id = block_id
        self.parent = parent
        self.children: dict[tuple, BlockNode] = {}
        self.lock_ref = 0
        self.last_access = 0.0
        self.linear_slot: Optional[int] = None
        self.alive = True


class BlockRadixCache:
    def __init__(
        self,
        block_size: int,
        on_evict_block: Optional[Callable[[int], None]] = None,
        on_evict_linear_slot: Optional[Callable[[int], None]] = None,
        require_linear_slot: bool = False,
    ):
        self.block_size = block_size
        self.on_evict_block = on_evict_block
        self.on_evict_linear_slot = on_evict_linear_slot
        self.require_linear_slot = require_linear_slot
        self.root = BlockNode(None, -1, None)
        self.root.lock_ref = 1
        self.request_to_nodes: dict[str, list[BlockNode]] = {}
        self.num_nodes = 0
        self._clock = itertools.count()
        self.hits = 0
        self.queries = 0
        self._unpinned = 0                 # nodes with lock_ref == 0 (what eviction could free)
        self._lru: list = []               # lazy heap of (last_access, tie, node) candidates
        self._tie = itertools.count()

    def _offer(self, node: BlockNode) -> None:
        """The node may have become an unpinned leaf: make it a candidate for eviction."""
        if node is not self.root and node.alive and node.lock_ref == 0 and not node.children:
            heapq.heappush(self._lru, (node.last_access, next(self._tie), node))
            if len(self._lru) > 4 * self.num_nodes + 4096:
                self._compact()

    def _compact(self) -> None:
        """Drop stale heap entries (a node is offered again every time it is unpinned; without eviction
        pressure nothing pops the old entries). Linear, but only after the heap grew to several times the
        tree, so its cost is amortised over that many offers."""
        seen, keep = set(), []
        for _stamp, tie, n in self._lru:
            if n.alive and n.lock_ref == 0 and not n.children and id(n) not in seen:
                seen.add(id(n))
                keep.append((n.last_access, tie, n))
        heapq.heapify(keep)
        self._lru = keep

    # ------------------------------------------------------------------ lookup
    def _tick(self) -> float:
        return time.monotonic() + next(self._clock) * 1e-9

    def root_of(self, namespace=None) -> BlockNode:
        """Root of the tree for a namespace. KV blocks depend on everything that shaped them, not only on the
        tokens: requests that run under a LoRA adapter must not share blocks with the base model or with
        another adapter, so each adapter name gets a tree of its own under a permanent pseudo-node."""
        if namespace is None:
            return self.root
        key = ("namespace", namespace)
        node = self.root.children.get(key)
        if node is None:
            node = BlockNode(key, -1, self.root)
            node.lock_ref = 1                      # never evicted, never counted
            self.root.children[key] = node
        return node

    def get_path(self, token_ids, namespace=None) -> list[BlockNode]:
        """Nodes along the longest fully matching block path (no side effects)."""
        bs = self.block_size
        node, path = self.root_of(namespace), []
        for i in range(0, len(token_ids) - bs + 1, bs):
            child = node.children.get(tuple(token_ids[i:i + bs]))
            if child is None:
                break
            path.append(child)
            node = child
        return path

    def match_prefix(self, token_ids, namespace=None) -> tuple[list[int], int]:
        """Longest cached prefix in whole blocks: (block ids, matched token count).

        With ``require_linear_slot`` the match is cut back to the deepest node that carries
        a linear-state snapshot, because a hybrid model can only resume from such a node.
        """
        self.queries += 1
        path = self.get_path(token_ids, namespace)
        if self.require_linear_slot:
            while path and path[-1].linear_slot is None:
                path.pop()
        now = self._tick()
        for n in path:
            n.last_access = now
        if path:
            self.hits += 1
        return [n.block_id for n in path], len(path) * self.block_size

    def get_node_for_token_ids(self, token_ids) -> Optional[BlockNode]:
        path = self.get_path(token_ids)
        if len(path) * self.block_size == len(token_ids) and path:
            return path[-1]
        return None

    # ------------------------------------------------------------------ insert
    def insert_block(self, prefix_nodes: list[BlockNode], block_tokens, block_id: int,
                     linear_slot: Optional[int] = None, namespace=None) -> tuple[BlockNode, bool]:
        """Insert one full block under the path ``prefix_nodes``.

        Returns (node, inserted). If the block is already cached the existing node is
        returned with ``inserted=False`` and the caller keeps ownership of ``block_id``.
        """
        assert len(block_tokens) == self.block_size
        parent = prefix_nodes[-1] if prefix_nodes else self.root_of(namespace)
        key = tuple(block_tokens)
        node = parent.children.get(key)
        if node is not None:
            node.last_access = self._tick()
            if linear_slot is not None and node.linear_slot is None:
                node.linear_slot = linear_slot
                return node, False
            return node, False
        node = BlockNode(key, block_id, parent)
        node.last_access = self._tick()
        node.linear_slot = linear_slot
        parent.children[key] = node
        self.num_nodes += 1
        self._unpinned += 1
        self._offer(node)
        return node, True

    # ------------------------------------------------------------------ pinning
    def increase_lock_ref(self, nodes: list[BlockNode]) -> None:
        for n in nodes:
            if n.lock_ref == 0:
                self._unpinned -= 1
            n.lock_ref += 1

    def decrease_lock_ref(self, nodes: list[BlockNode]) -> None:
        for n in nodes:
            if n.lock_ref > 0:
                n.lock_ref -= 1
                if n.lock_ref == 0:
                    self._unpinned += 1
                    self._offer(n)

    def register_request(self, request_id: str, nodes: list[BlockNode]) -> None:
        self.increase_lock_ref(nodes)
        self.request_to_nodes.setdefault(request_id, []).extend(nodes)

    def release_request(self, request_id: str) -> None:
        nodes = self.request_to_nodes.pop(request_id, None)
        if nodes:
            now = self._tick()
            for n in nodes:
                n.last_access = now
            self.decrease_lock_ref(nodes)

    # ------------------------------------------------------------------ eviction
    def evict_lru_blocks(self, num_blocks: int) -> int:
        """Evict up to ``num_blocks`` unpinned leaf blocks, least recently used first."""
        evicted = 0
        heap = self._lru
        while heap and evicted < num_blocks:
            stamp, _, n = heapq.heappop(heap)
            if not n.alive or n.children or n.lock_ref > 0:
                continue                          # deleted, extended or pinned since it was offered
            if stamp != n.last_access:
                self._offer(n)                    # touched since: back in line with its current time
                continue
            parent = n.parent
            self._delete_leaf(n)
            evicted += 1
            if parent is not self.root and parent.block_id >= 0:
                self._offer(parent)               # it may have become a leaf
        return evicted

    def _delete_leaf(self, node: BlockNode) -> None:
        node.alive = False
        del node.parent.children[node.key]
        self.num_nodes -= 1
        self._unpinned -= 1
        if self.on_evict_block is not None:
            self.on_evict_block(node.block_id)
        if node.linear_slot is not None and self.on_evict_linear_slot is not None:
            self.on_evict_linear_slot(node.linear_slot)

    def evictable_size(self) -> int:
        """Blocks that eviction could free. Requests pin whole root-to-node paths, so an
        unpinned node never has a pinned descendant and the count of unpinned nodes is exact."""
        return self._unpinned

    def get_stats(self) -> dict:
        return {
            "nodes": self.num_nodes,
            "queries": self.queries,
            "hits": self.hits,
            "hit_rate": self.hits / self.queries if self.queries else 0.0,
            "locked_requests": len(self.request_to_nodes),
        }

    def reset(self) -> None:
        stack = list(self.root.children.values())
        self.root.children.clear()
        while stack:
            n = stack.pop()
            stack.extend(n.children.values())
            n.alive = False
            if n.block_id < 0:
                continue                          # namespace pseudo-node
            if self.on_evict_block is not None:
                self.on_evict_block(n.block_id)
            if n.linear_slot is not None and self.on_evict_linear_slot is not None:
                self.on_evict_linear_slot(n.linear_slot)
        self.num_nodes = 0
        self._unpinned = 0
        self._lru = []
        self.request_to_nodes.clear()
