"""Property test of the logical KV cache: random interleavings of the calls the engine makes (admit with a prompt,
publish computed blocks, grow by a token, finish) keep the block accounting exact."""

import numpy as np
from hypothesis import HealthCheck, given, settings
from hypothesis import strategies as st

from parallax_b200.cache.manager import CacheManager

PAGE, BLOCKS = 4, 48


def _tree_blocks(cm) -> list[int]:
    out, stack = [], list(cm.prefix_cache.root.children.values())
    while stack:
        n = stack.pop()
        out.append(n.block_id)
        stack.extend(n.children.values())
    return out


def _check(cm: CacheManager) -> None:
    free = set(np.nonzero(cm.allocator._is_free)[0].tolist())
    tree = _tree_blocks(cm)
    assert len(tree) == len(set(tree)), "a block is in the prefix tree twice"
    owned: dict[int, int] = {}
    for rid, stt in cm.reqs.items():
        table = cm.get_block_table(rid)
        assert len(table) == stt.num_blocks and len(set(table)) == len(table)
        assert stt.ctx_len <= stt.num_blocks * PAGE
        shared = {n.block_id for n in stt.nodes}
        for i, b in enumerate(table):
            if b in shared:
                continue
            assert b not in owned, f"private block {b} is held by two requests"
            owned[b] = 1
    private = set(owned)
    assert not (private & set(tree) - {b for stt in cm.reqs.values() for b in (n.block_id for n in stt.nodes)}), \
        "a request's private block is also a tree block it does not reference"
    used = private | set(tree)
    assert cm.num_free_blocks() == BLOCKS - len(used), (cm.num_free_blocks(), len(used))
    assert free == set(range(BLOCKS)) - used, "the allocator's free set and the blocks in use must partition the pool"


ops = st.lists(st.tuples(st.sampled_from(["admit", "publish", "grow", "finish"]), st.integers(0, 7), st.integers(1, 30),
                         st.integers(0, 3)), min_size=1, max_size=60)


@settings(max_examples=120, deadline=None, suppress_health_check=[HealthCheck.too_slow])
@given(ops)
def test_block_accounting_stays_exact(seq):
    cm = CacheManager(BLOCKS, PAGE, max_requests=16, max_blocks_per_seq=16, enable_prefix_cache=True)
    rng = np.random.default_rng(0)
    families = [rng.integers(0, 50, 40).tolist() for _ in range(4)]     # prompts of one family share prefixes
    prompts: dict[str, list[int]] = {}
    for op, slot, n, fam in seq:
        rid = f"r{slot}"
        if op == "admit" and rid not in cm.reqs:
            ids = families[fam][:n]
            ok, matched = cm.allocate_request(rid, len(ids), token_ids=ids)
            if ok:
                prompts[rid] = list(ids)
                assert matched % PAGE == 0 and matched < max(len(ids), 1) + PAGE
                assert cm.get_context_length(rid) == len(ids)
            else:
                assert rid not in cm.reqs
        elif op == "publish" and rid in cm.reqs:
            cm.insert_full_blocks_to_cache(rid, cm.get_context_length(rid))
        elif op == "grow" and rid in cm.reqs:
            before = cm.get_context_length(rid)
            if cm.reqs[rid].num_blocks < 16 or before < 16 * PAGE:
                if before < 15 * PAGE and cm.append_slot(rid):
                    cm.append_request_token(rid, int(n))
                    assert cm.get_context_length(rid) == before + 1
        elif op == "finish" and rid in cm.reqs:
            cm.free_request(rid)
            prompts.pop(rid, None)
        _check(cm)
    for rid in list(cm.reqs):
        cm.free_request(rid)
    _check(cm)
    # with nobody holding a reference every cached block can be reclaimed
    cm.prefix_cache.evict_lru_blocks(BLOCKS)
    assert cm.num_free_blocks() == BLOCKS and not _tree_blocks(cm)
