"""Property tests of the cluster scheduler's allocation: whatever mix of nodes joins, the layer ranges the allocators
hand out are contiguous, within every node's capacity, and tile the model exactly for each pipeline they form."""

from hypothesis import HealthCheck, given, settings
from hypothesis import strategies as st

from parallax_b200.scheduling.layer_allocation import DynamicProgrammingLayerAllocator, GreedyLayerAllocator
from parallax_b200.scheduling.node_management import NodeManager
from parallax_b200.scheduling.request_routing import RandomizedOverDynamicPipelinesRouting
from tests.test_scheduling import HW, model, node

KINDS = sorted(HW)


@settings(max_examples=80, deadline=None, suppress_health_check=[HealthCheck.too_slow])
@given(st.integers(4, 40), st.lists(st.sampled_from(KINDS), min_size=1, max_size=9), st.sampled_from(["greedy", "dp"]))
def test_allocations_tile_the_model(num_layers, kinds, strategy):
    m = model(num_layers)
    nodes = [node(k, m, f"{k}-{i}") for i, k in enumerate(kinds)]
    nm = NodeManager(initial_nodes=nodes)
    cls = GreedyLayerAllocator if strategy == "greedy" else DynamicProgrammingLayerAllocator
    alloc = cls(model_info=m, node_management=nm)
    ok = alloc.allocate_from_standby()
    total_cap = sum(n.get_decoder_layer_capacity() for n in nodes)
    if total_cap < num_layers:
        assert not ok or nm.num_full_pipelines(num_layers) == 0
    for n in nm.active_nodes:
        assert n.start_layer is not None and 0 <= n.start_layer < n.end_layer <= num_layers
        # the first / last stage also hold the embedding / head, which the capacity accounts for
        cap = n.get_decoder_layer_capacity(include_input_embed=n.start_layer == 0, include_lm_head=n.end_layer == num_layers)
        assert n.end_layer - n.start_layer <= max(cap, 1), (n.node_id, n.start_layer, n.end_layer, cap)
    if ok:
        pipes = RandomizedOverDynamicPipelinesRouting.pipeline_discovery(nm.active_nodes, num_layers)
        assert pipes and nm.num_full_pipelines(num_layers) >= 1
        by_id = {n.node_id: n for n in nodes}
        for p in pipes:
            at = 0
            for nid in p:
                assert by_id[nid].start_layer == at
                at = by_id[nid].end_layer
            assert at == num_layers
    # standby nodes hold nothing
    for n in nm.standby_nodes:
        assert n.start_layer is None or n.start_layer == n.end_layer or n.num_current_layers == 0
