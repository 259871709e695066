"""Property test of the cross-node pipeline: for random splits of the layers over peers, slice sizes, batch limits
and prompt mixes (some sharing a prefix), chained peers with the wire emulated finish every request, release
everything on every peer, and produce tokens of the right count. (Equality with the single engine is covered by
fixed cases; here prompts arrive while others run.)"""

import torch
from hypothesis import HealthCheck, given, settings
from hypothesis import strategies as st

from parallax_b200.engine.peer import PeerExecutor
from parallax_b200.engine.request import Request, SamplingParams
from parallax_b200.models.config import named_config
from tests.test_peer_pipeline import _wire

CFG = named_config("tiny")          # 4 layers

splits = st.sampled_from([[(0, 4)], [(0, 2), (2, 4)], [(0, 1), (1, 4)], [(0, 1), (1, 3), (3, 4)], [(0, 1), (1, 2), (2, 3), (3, 4)]])
workload = st.fixed_dictionaries({
    "spans": splits, "batch": st.integers(1, 4), "budget": st.integers(32, 128), "chunk": st.sampled_from([None, 16, 48]),
    "blocks": st.integers(24, 64),
    "reqs": st.lists(st.tuples(st.integers(1, 90), st.integers(1, 5), st.booleans(), st.integers(0, 3)), min_size=1, max_size=6),
})


@settings(max_examples=40, deadline=None, suppress_health_check=[HealthCheck.too_slow])
@given(workload)
def test_every_request_ends_and_every_peer_lets_go(w):
    peers = [PeerExecutor(CFG, s, e, device="cpu", node_id=f"n{i}", num_blocks=w["blocks"], max_batch_size=w["batch"],
                          max_num_tokens_per_batch=w["budget"], chunked_prefill_size=w["chunk"], max_total_length=128)
             for i, (s, e) in enumerate(w["spans"])]
    table = [p.node_id for p in peers]
    g = torch.Generator().manual_seed(2)
    shared = torch.randint(0, CFG.vocab_size, (64,), generator=g).tolist()
    arrivals = []
    for n, max_new, share, delay in w["reqs"]:
        ids = (shared[:min(n, 64)] + torch.randint(0, CFG.vocab_size, (max(n - 64, 0),), generator=g).tolist()) if share \
            else torch.randint(0, CFG.vocab_size, (n,), generator=g).tolist()
        arrivals.append((delay, Request(input_ids=ids, routing_table=table,
                                        sampling_params=SamplingParams(max_new_tokens=max_new, temperature=0.0, ignore_eos=True))))
    reqs = [r for _d, r in arrivals]
    finished = set()
    step = 0
    while (arrivals or peers[0].has_work()) and step < 1500:
        for d, r in [a for a in arrivals if a[0] <= step]:
            peers[0].add_request(r)
        arrivals = [a for a in arrivals if a[0] > step]
        step += 1
        packets, events, releases = peers[0].step_first()
        finished |= {r.request_id for r, _t in events if r.is_finished}
        for peer in peers[1:]:
            peer.release(releases)
        back = []
        for peer in peers[1:]:
            packets = peer.process_packets(_wire(packets))
            back = packets
        if len(peers) > 1:
            events, releases = peers[0].receive_tokens(_wire([p for p in back if p.hidden_states is None]))
            finished |= {r.request_id for r, _t in events if r.is_finished}
            for peer in peers[1:]:
                peer.release(releases)
    assert step < 1500, "the pipeline does not drain"
    for r in reqs:
        assert r.is_finished, (r.status, len(r.input_ids))
        # a request ends with all its tokens, or aborted when some peer ran out of KV memory
        assert len(r.output_ids) == r.sampling_params.max_new_tokens or r.status.name == "FINISHED_ABORT", (r.status, r.output_ids)
    for p in peers:
        assert not p.cache.reqs and not p.mirror, (p.node_id, list(p.cache.reqs), list(p.mirror))
