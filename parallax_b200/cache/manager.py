"""Paged-KV bookkeeping: block tables, context lengths, prefix reuse, LRU eviction.

``CacheManager`` is purely logical (block ids, no tensors) so that one instance on the
scheduling rank can plan for every pipeline stage of the box: all stages allocate the same
number of blocks and use identical block ids. The device tensors live in
:class:`parallax_b200.cache.kv_pool.KVPool`.

Semantics follow the reference's per-shard manager
(``src/parallax/server/cache_manager.py:449-629,704-791``): a new request matches the
prefix cache on ``tokens[:-1]`` (at least one token is always computed), matched blocks are
shared and pinned, the rest of the prompt's blocks are allocated up front, decode appends a
block every ``block_size`` tokens, allocation pressure evicts unpinned LRU prefix blocks,
and full blocks are published to the prefix cache after prefill.
"""

from __future__ import annotations

import logging
from typing import Optional

import numpy as np

from parallax_b200.cache.allocator import BlockAllocator, SlotAllocator
from parallax_b200.cache.radix import BlockNode, BlockRadixCache

logger = logging.getLogger(__name__)


class _ReqState:
    __slots__ = ("row", "num_blocks", "ctx_len", "matched", "tokens", "nodes", "linear_slot", "namespace")

    def __init__(self, row: int):
        self.row = row
        self.num_blocks = 0
        self.ctx_len = 0
        self.matched = 0
        self.tokens: Optional[list[int]] = None
        self.nodes: list[BlockNode] = []   # tree nodes backing the first len(nodes) blocks
        self.linear_slot = -1
        self.namespace = None              # prefix-cache namespace (e.g. the LoRA adapter the request runs under)


class CacheManager:
    def __init__(
        self,
        num_blocks: int,
        block_size: int,
        max_requests: int = 1024,
        max_blocks_per_seq: int = 2048,
        enable_prefix_cache: bool = True,
        num_linear_slots: int = 0,
        num_prefix_linear_slots: int = 0,
    ):
        self.block_size = block_size
        self.num_blocks = num_blocks
        self.max_blocks_per_seq = max_blocks_per_seq
        self.allocator = BlockAllocator(num_blocks)
        self.rows = SlotAllocator(max_requests)
        self.tables = np.zeros((max_requests, max_blocks_per_seq), dtype=np.int32)
        self.reqs: dict[str, _ReqState] = {}
        self.needs_slots = num_linear_slots > 0
        self.slot_allocator = SlotAllocator(num_linear_slots) if self.needs_slots else None
        self.prefix_slot_allocator = (
            SlotAllocator(num_prefix_linear_slots) if num_prefix_linear_slots > 0 else None
        )
        self.prefix_slot_base = num_linear_slots
        # hooks for the physical pools of hybrid models: zero / copy a state slot
        self.weights_epoch = 0          # bumped by invalidate_prefix_cache()
        self.on_zero_slot = None
        self.on_copy_slot = None
        self.prefix_cache: Optional[BlockRadixCache] = None
        if enable_prefix_cache:
            self.prefix_cache = BlockRadixCache(
                block_size,
                on_evict_block=self._on_evict_block,
                on_evict_linear_slot=self._on_evict_linear_slot,
                require_linear_slot=self.needs_slots,
            )

    # ------------------------------------------------------------------ weights changed
    def invalidate_prefix_cache(self) -> int:
        """The model's weights changed (online refit): K/V pages and state snapshots computed before are stale.
        Every cached block that no running request holds is freed now, and requests admitted from here on live in
        a new namespace, so they cannot match what running requests still publish or hold under the old weights
        (those blocks become evictable when their requests end). Returns the number of blocks freed."""
        if self.prefix_cache is None:
            return 0
        self.weights_epoch += 1
        freed = self.prefix_cache.evict_lru_blocks(self.num_blocks)
        root = self.prefix_cache.root
        for key in [k for k, n in root.children.items() if n.block_id < 0 and not n.children]:
            del root.children[key]              # empty per-namespace roots of earlier epochs
        return freed

    # ------------------------------------------------------------------ callbacks
    def _on_evict_block(self, block_id: int) -> None:
        self.allocator.free([block_id])

    def _on_evict_linear_slot(self, slot: int) -> None:
        if self.prefix_slot_allocator is not None:
            self.prefix_slot_allocator.free(slot - self.prefix_slot_base)

    def _evict(self, n: int) -> int:
        if self.prefix_cache is None or n <= 0:
            return 0
        return self.prefix_cache.evict_lru_blocks(n)

    # ------------------------------------------------------------------ queries
    def has_request(self, rid: str) -> bool:
        return rid in self.reqs

    def get_block_table(self, rid: str) -> list[int]:
        st = self.reqs[rid]
        return self.tables[st.row, :st.num_blocks].tolist()

    def get_context_length(self, rid: str) -> int:
        return self.reqs[rid].ctx_len

    def get_matched_tokens(self, rid: str) -> int:
        return self.reqs[rid].matched

    def get_row(self, rid: str) -> int:
        return self.reqs[rid].row

    def get_slot(self, rid: str) -> int:
        return self.reqs[rid].linear_slot

    def num_free_blocks(self) -> int:
        return self.allocator.get_num_free_blocks()

    def num_available_blocks(self) -> int:
        """Free blocks plus blocks that eviction could reclaim."""
        extra = self.prefix_cache.evictable_size() if self.prefix_cache else 0
        return self.allocator.get_num_free_blocks() + extra

    def blocks_needed(self, num_tokens: int) -> int:
        return (num_tokens + self.block_size - 1) // self.block_size

    def get_reusable_prefix_len(self, token_ids) -> int:
        if self.prefix_cache is None or not token_ids:
            return 0
        return len(self.prefix_cache.get_path(token_ids[:-1])) * self.block_size

    # ------------------------------------------------------------------ allocation
    def allocate_request(self, rid: str, prompt_len: int, token_ids=None, namespace=None) -> tuple[bool, int]:
        """Reserve blocks for the whole prompt. Returns (ok, tokens matched in prefix cache). ``namespace``:
        requests only share cached blocks with requests of the same namespace."""
        st = self.reqs.get(rid)
        if st is not None:
            return True, st.matched
        need = self.blocks_needed(prompt_len)
        if need > self.max_blocks_per_seq:
            return False, 0
        row = self.rows.allocate()
        if row < 0:
            return False, 0
        st = _ReqState(row)
        if self.weights_epoch:
            # blocks written under older weights must not be matched: the epoch is part of the namespace
            namespace = (namespace, self.weights_epoch)
        st.namespace = namespace
        matched_blocks: list[int] = []
        if self.prefix_cache is not None and token_ids is not None:
            st.tokens = list(token_ids)
            probe = st.tokens[:-1]
            matched_blocks, matched = self.prefix_cache.match_prefix(probe, namespace)
            if matched:
                nodes = self.prefix_cache.get_path(probe[:matched], namespace)
                if len(nodes) != len(matched_blocks):
                    matched_blocks, matched = [], 0
                else:
                    st.nodes = nodes
                    st.matched = matched
                    self.prefix_cache.register_request(rid, nodes)
        slot = -1
        if self.needs_slots:
            slot = self.slot_allocator.allocate()
            if slot < 0:
                self._abort_alloc(rid, st)
                return False, 0
            st.linear_slot = slot
        n_new = need - len(matched_blocks)
        new_blocks = np.empty(0, dtype=np.int32)
        if n_new > 0:
            free = self.allocator.get_num_free_blocks()
            if free < n_new:
                self._evict(n_new - free)
            got = self.allocator.allocate_np(n_new)
            if got is None:
                self._abort_alloc(rid, st)
                return False, 0
            new_blocks = got
        k = len(matched_blocks)
        if k:
            self.tables[row, :k] = matched_blocks
        if n_new > 0:
            self.tables[row, k:k + n_new] = new_blocks
        st.num_blocks = need
        st.ctx_len = prompt_len
        self.reqs[rid] = st
        if self.needs_slots:
            src = st.nodes[-1].linear_slot if st.nodes else None
            if src is not None and self.on_copy_slot is not None:
                self.on_copy_slot(slot, src)
            elif self.on_zero_slot is not None:
                self.on_zero_slot(slot)
        return True, st.matched

    def rematch_request(self, rid: str) -> int:
        """Probe the prefix cache again for a request whose prompt has not started to run: blocks that
        another request published since this one was admitted replace its private (still empty) blocks.
        Hybrid models keep their admission-time match (their state slot was initialised from it).
        Returns the matched token count."""
        st = self.reqs.get(rid)
        if st is None or self.prefix_cache is None or st.tokens is None or self.needs_slots:
            return st.matched if st is not None else 0
        have = len(st.nodes)
        if have * self.block_size != st.matched:
            return st.matched          # its own blocks are being published already
        probe = st.tokens[:st.ctx_len - 1] if st.ctx_len else st.tokens[:-1]
        path = self.prefix_cache.get_path(probe, st.namespace)
        if len(path) <= have:
            return st.matched
        fresh = path[have:]
        if any(a is not b for a, b in zip(path[:have], st.nodes)):
            return st.matched          # the tree changed under the old match (evicted and rebuilt): keep it
        self.allocator.free(self.tables[st.row, have:len(path)].tolist())
        self.tables[st.row, have:len(path)] = [n.block_id for n in fresh]
        self.prefix_cache.register_request(rid, fresh)
        self.prefix_cache.match_prefix(probe, st.namespace)      # statistics and time stamps
        st.nodes = list(path)
        st.matched = len(path) * self.block_size
        return st.matched

    def next_block_key(self, rid: str, computed: int):
        """Identity of the first block the request still has to compute: (parent tree node, tokens of the
        block); None when less than a full block is left. Two requests with the same key would compute
        the same KV block."""
        st = self.reqs.get(rid)
        if st is None or st.tokens is None or self.prefix_cache is None:
            return None
        bs = self.block_size
        i = computed // bs
        if computed % bs or (i + 1) * bs > len(st.tokens) - 1 or i != len(st.nodes):
            return None
        parent = st.nodes[-1] if st.nodes else None
        return (id(parent) if parent is not None else ("root", st.namespace), tuple(st.tokens[i * bs:(i + 1) * bs]))

    def _abort_alloc(self, rid: str, st: _ReqState) -> None:
        if self.prefix_cache is not None:
            self.prefix_cache.release_request(rid)
        if st.linear_slot >= 0:
            self.slot_allocator.free(st.linear_slot)
        self.rows.free(st.row)

    def append_slot(self, rid: str) -> bool:
        """Make room for one more token (decode). False = out of KV memory."""
        st = self.reqs.get(rid)
        if st is None:
            raise ValueError(f"request {rid} not found")
        if st.ctx_len % self.block_size == 0 and st.ctx_len // self.block_size >= st.num_blocks:
            if st.num_blocks >= self.max_blocks_per_seq:
                return False
            got = self.allocator.allocate_np(1)
            if got is None:
                self._evict(1)
                got = self.allocator.allocate_np(1)
            if got is None:
                return False
            self.tables[st.row, st.num_blocks] = got[0]
            st.num_blocks += 1
        st.ctx_len += 1
        return True

    def extend_request(self, rid: str, new_len: int) -> bool:
        """Grow a request's reservation to ``new_len`` tokens (later prefill chunks on peers that
        learn the prompt piecewise). False = out of KV memory; nothing is changed then."""
        st = self.reqs.get(rid)
        if st is None:
            raise ValueError(f"request {rid} not found")
        need = self.blocks_needed(new_len)
        if need > self.max_blocks_per_seq:
            return False
        extra = need - st.num_blocks
        if extra > 0:
            free = self.allocator.get_num_free_blocks()
            if free < extra:
                self._evict(extra - free)
            got = self.allocator.allocate_np(extra)
            if got is None:
                return False
            self.tables[st.row, st.num_blocks:need] = got
            st.num_blocks = need
        st.ctx_len = max(st.ctx_len, new_len)
        return True

    def slot_of(self, rid: str, pos: int) -> int:
        st = self.reqs[rid]
        return int(self.tables[st.row, pos // self.block_size]) * self.block_size + pos % self.block_size

    def free_request(self, rid: str) -> None:
        st = self.reqs.pop(rid, None)
        if st is None:
            return
        owned_by_tree = len(st.nodes)
        if self.prefix_cache is not None:
            self.prefix_cache.release_request(rid)
        if st.num_blocks > owned_by_tree:
            self.allocator.free(self.tables[st.row, owned_by_tree:st.num_blocks].tolist())
        if st.linear_slot >= 0:
            self.slot_allocator.free(st.linear_slot)
        self.rows.free(st.row)

    release_request = free_request

    # ------------------------------------------------------------------ prefix publishing
    def update_request_tokens(self, rid: str, new_token_ids) -> None:
        st = self.reqs.get(rid)
        if st is not None and st.tokens is not None:
            st.tokens.extend(int(t) for t in new_token_ids)

    def append_request_token(self, rid: str, token_id: int) -> None:
        """One generated token (the per-step case of :meth:`update_request_tokens`)."""
        st = self.reqs.get(rid)
        if st is not None and st.tokens is not None:
            st.tokens.append(token_id)

    def insert_full_blocks_to_cache(self, rid: str, num_computed_tokens: Optional[int] = None,
                                    snapshot_linear=None) -> int:
        """Publish every full block whose KV is computed. Returns number of new nodes.

        ``snapshot_linear(src_slot, dst_slot)`` is called for hybrid models to capture the
        recurrent state at the last published block boundary.
        """
        st = self.reqs.get(rid)
        if self.prefix_cache is None or st is None or st.tokens is None:
            return 0
        computed = st.ctx_len if num_computed_tokens is None else min(num_computed_tokens, st.ctx_len)
        computed = min(computed, len(st.tokens))
        full = computed // self.block_size
        inserted = 0
        bs = self.block_size
        new_nodes = []
        while len(st.nodes) < full:
            i = len(st.nodes)
            block_id = int(self.tables[st.row, i])
            node, is_new = self.prefix_cache.insert_block(st.nodes, st.tokens[i * bs:(i + 1) * bs], block_id,
                                                          namespace=st.namespace)
            if not is_new:
                if node.block_id != block_id:
                    # same content already cached by someone else: keep our private copy
                    break
            else:
                inserted += 1
            st.nodes.append(node)
            new_nodes.append(node)
        if new_nodes:
            self.prefix_cache.register_request(rid, new_nodes)
            if self.needs_slots and snapshot_linear is not None and self.prefix_slot_allocator is not None:
                last = new_nodes[-1]
                if last.linear_slot is None and len(st.nodes) * bs == computed:
                    ps = self.prefix_slot_allocator.allocate()
                    if ps >= 0:
                        snapshot_linear(st.linear_slot, self.prefix_slot_base + ps)
                        last.linear_slot = self.prefix_slot_base + ps
        return inserted

    def stats(self) -> dict:
        d = {
            "num_blocks": self.num_blocks,
            "free_blocks": self.allocator.get_num_free_blocks(),
            "requests": len(self.reqs),
        }
        if self.prefix_cache is not None:
            d["prefix"] = self.prefix_cache.get_stats()
        return d
