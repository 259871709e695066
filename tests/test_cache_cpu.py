"""Paged-KV bookkeeping on CPU: LRU eviction of the block radix cache under pressure, its O(1)
evictable count against a tree walk, and prefix sharing between requests admitted together."""

import random

from parallax_b200.cache.manager import CacheManager
from parallax_b200.cache.radix import BlockRadixCache
from parallax_b200.engine.request import Request, SamplingParams
from parallax_b200.engine.scheduler import BatchScheduler


def _walk_unpinned(cache: BlockRadixCache) -> int:
    n, stack = 0, list(cache.root.children.values())
    while stack:
        node = stack.pop()
        stack.extend(node.children.values())
        n += node.lock_ref == 0
    return n


def test_radix_lru_order_and_pinning():
    freed = []
    c = BlockRadixCache(2, on_evict_block=freed.append)
    a, _ = c.insert_block([], [1, 2], 10)
    b, _ = c.insert_block([a], [3, 4], 11)
    d, _ = c.insert_block([], [5, 6], 12)
    c.register_request("r", [a, b])
    assert c.evictable_size() == 1 == _walk_unpinned(c)
    assert c.evict_lru_blocks(5) == 1 and freed == [12]        # only the unpinned leaf goes
    c.release_request("r")
    assert c.evictable_size() == 2
    e, _ = c.insert_block([], [7, 8], 13)
    c.match_prefix([1, 2, 3, 4])                               # touch the chain: [7, 8] is now the oldest
    assert c.evict_lru_blocks(1) == 1 and freed[-1] == 13
    assert c.evict_lru_blocks(10) == 2 and freed[-2:] == [11, 10]      # leaf first, then its parent
    assert c.num_nodes == 0 and c.evictable_size() == 0


def test_radix_eviction_under_pressure_matches_a_tree_walk():
    rng = random.Random(3)
    freed = []
    c = BlockRadixCache(4, on_evict_block=freed.append)
    live, next_block = {}, 0
    for step in range(3000):
        op = rng.random()
        if op < 0.5:
            toks = [rng.randrange(6) for _ in range(4 * rng.randrange(1, 6))]
            path = c.get_path(toks)
            nodes = list(path)
            for i in range(len(path), len(toks) // 4):
                node, new = c.insert_block(nodes, toks[4 * i:4 * i + 4], next_block)
                next_block += new
                nodes.append(node)
            rid = f"r{step}"
            c.register_request(rid, nodes)
            live[rid] = nodes
        elif op < 0.85 and live:
            c.release_request(live.popitem()[0] if rng.random() < 0.5 else next(iter(live)))
            live = {k: v for k, v in live.items() if k in c.request_to_nodes}
        else:
            before = c.num_nodes
            got = c.evict_lru_blocks(rng.randrange(1, 8))
            assert c.num_nodes == before - got
        assert c.evictable_size() == _walk_unpinned(c)
        assert len(c._lru) <= 4 * c.num_nodes + 4097            # stale heap entries are compacted away
    for nodes in live.values():                                 # pinned nodes were never evicted
        assert all(n.alive for n in nodes)
    assert len(set(freed)) == len(freed)


def test_manager_reuses_blocks_under_kv_pressure():
    """A pool that holds four prompts: serving twelve different ones evicts cached prefixes of finished
    requests, never blocks of running ones, and leaves the pool consistent."""
    cm = CacheManager(num_blocks=16, block_size=4, max_requests=8, max_blocks_per_seq=8)
    rng = random.Random(0)
    for i in range(12):
        toks = [rng.randrange(1000) for _ in range(15)]
        ok, matched = cm.allocate_request(f"q{i}", len(toks), token_ids=toks)
        assert ok and matched == 0
        cm.insert_full_blocks_to_cache(f"q{i}", len(toks))
        if i >= 2:
            cm.free_request(f"q{i - 2}")                         # two requests live at any time
        assert cm.num_free_blocks() + cm.prefix_cache.num_nodes + sum(
            st.num_blocks - len(st.nodes) for st in cm.reqs.values()) == 16
    assert cm.prefix_cache.evictable_size() == _walk_unpinned(cm.prefix_cache)


def test_prompts_admitted_together_share_their_prefix():
    """Four requests with the same 32-token prefix arrive at once: one computes the prefix, the others
    wait a step and then reuse its blocks instead of computing it four times."""
    cm = CacheManager(num_blocks=64, block_size=8, max_requests=8, max_blocks_per_seq=16)
    sched = BatchScheduler(max_batch_size=8, max_num_tokens_per_batch=4096, cache_manager=cm, chunked_prefill_size=None)
    prefix = list(range(100, 132))
    reqs = [Request(input_ids=prefix + [200 + i, 300 + i, 400 + i], sampling_params=SamplingParams(max_new_tokens=2))
            for i in range(4)]
    for r in reqs:
        sched.enque_request(r)
    first = sched.form_batch()
    assert [s.req for s in first] == [reqs[0]] and first[0].num_tokens == 35
    # what the engine does when it launches the batch: progress + publishing
    reqs[0].num_computed_tokens = 35
    cm.insert_full_blocks_to_cache(reqs[0].request_id, 35)
    second = sched.form_batch()
    assert [s.req for s in second] == reqs[1:]
    assert all(s.start == 32 and s.num_tokens == 3 for s in second)          # only the tails are computed
    tables = [cm.get_block_table(r.request_id)[:4] for r in reqs]
    assert all(t == tables[0] for t in tables)                               # the same physical blocks
    for r in reqs:
        cm.free_request(r.request_id)
    assert cm.num_free_blocks() + cm.prefix_cache.num_nodes == 64
