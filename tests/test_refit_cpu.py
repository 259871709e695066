"""Online weight refit for every model family: a stage that took checkpoint A and is then refitted with
checkpoint B must hold exactly what a fresh stage loaded from B holds, in the storage it already had, and an
incomplete layer must be refused before anything changes."""

import pytest
import torch

from helpers.hf_weights import hf_state_dict
from parallax_b200.models.config import named_config
from parallax_b200.models.registry import build_stage, family_of

CASES = [("tiny", (0, 4)), ("tiny-moe", (1, 4)), ("tiny-mla", (0, 3)), ("tiny-dsa", (0, 2)), ("tiny-hybrid", (0, 4)),
         ("tiny-msa", (0, 3))]


def _flat(stage):
    """name -> tensor for everything the stage holds."""
    out = {}

    def walk(prefix, v):
        if isinstance(v, torch.Tensor):
            out[prefix] = v
        elif isinstance(v, (tuple, list)):
            for i, x in enumerate(v):
                walk(f"{prefix}[{i}]", x)
        elif isinstance(v, dict):
            for k, x in v.items():
                walk(f"{prefix}.{k}", x)
        elif hasattr(v, "tensors") and hasattr(v, "__dict__"):
            for k, x in vars(v).items():
                walk(f"{prefix}.{k}", x)

    for name in ("embed", "norm_w", "lm_head"):
        walk(name, getattr(stage, name))
    for li, lw in enumerate(stage.layers):
        for cls in type(lw).__mro__:
            for s in getattr(cls, "__slots__", ()):
                walk(f"L{li}.{s}", getattr(lw, s, None))
    for li, d in getattr(stage, "idx", {}).items():
        walk(f"L{li}.idx", d)
    return out


@pytest.mark.parametrize("name,span", CASES)
def test_refit_equals_fresh_load_and_keeps_storage(name, span):
    cfg = named_config(name)
    fam = family_of(cfg.architecture)
    a, b = hf_state_dict(cfg, fam, seed=1), hf_state_dict(cfg, fam, seed=2)
    live = build_stage(cfg, span[0], span[1], "cpu", torch.float32)
    live.load_weights(a)
    before = _flat(live)
    ptrs = {k: t.data_ptr() for k, t in before.items()}
    n = live.update_weights(b)
    fresh = build_stage(cfg, span[0], span[1], "cpu", torch.float32)
    fresh.load_weights(b)
    want, got = _flat(fresh), _flat(live)
    assert set(want) == set(got)
    for k in want:
        assert torch.equal(want[k], got[k]), k
        assert got[k].data_ptr() == ptrs[k], f"{k} moved"
    used = [k for k in b if (live._layer_of_key(k) is None) or span[0] <= live._layer_of_key(k) < span[1]]
    if not live.is_first and not cfg.tie_word_embeddings:
        used = [k for k in used if "embed_tokens" not in k]
    assert n == len(used), (n, len(used))


def test_refit_refuses_an_incomplete_layer_and_changes_nothing():
    cfg = named_config("tiny-mla")
    a, b = hf_state_dict(cfg, "deepseek", seed=1), hf_state_dict(cfg, "deepseek", seed=2)
    st = build_stage(cfg, 0, 3, "cpu", torch.float32)
    st.load_weights(a)
    snap = {k: t.clone() for k, t in _flat(st).items()}
    part = {k: v for k, v in b.items() if k.startswith("model.layers.")}
    del part["model.layers.2.self_attn.kv_b_proj.weight"]
    with pytest.raises(ValueError, match="layer 2"):
        st.update_weights(part)
    for k, t in _flat(st).items():
        assert torch.equal(t, snap[k]), k
    # one complete layer alone is fine, the others stay as they were
    one = {k: v for k, v in b.items() if k.startswith("model.layers.1.")}
    assert st.update_weights(one) == len(one)
    fresh = build_stage(cfg, 0, 3, "cpu", torch.float32)
    fresh.load_weights(b)
    got, want = _flat(st), _flat(fresh)
    assert all(torch.equal(got[k], want[k]) for k in got if k.startswith("L1."))
    assert all(torch.equal(got[k], snap[k]) for k in got if k.startswith("L0."))


def test_refit_of_an_expert_parallel_stage_keeps_its_shard():
    cfg = named_config("tiny-moe")
    a, b = hf_state_dict(cfg, "decoder", seed=1), hf_state_dict(cfg, "decoder", seed=2)
    st = build_stage(cfg, 0, 2, "cpu", torch.float32, ep_rank=1, ep_size=2, ep_comm=None)
    st.load_weights(a)
    shapes = {k: t.shape for k, t in _flat(st).items()}
    st.update_weights(b)
    fresh = build_stage(cfg, 0, 2, "cpu", torch.float32, ep_rank=1, ep_size=2, ep_comm=None)
    fresh.load_weights(b)
    got, want = _flat(st), _flat(fresh)
    assert {k: t.shape for k, t in got.items()} == shapes
    assert all(torch.equal(got[k], want[k]) for k in want)


def test_refit_of_a_tensor_parallel_stage_goes_through_the_sharding_again():
    cfg = named_config("tiny")
    cfg.tie_word_embeddings = False
    a, b = hf_state_dict(cfg, "decoder", seed=1), hf_state_dict(cfg, "decoder", seed=2)
    kw = dict(tp_rank=1, tp_size=2, tp_group=None, comm=None)
    st = build_stage(cfg, 0, 4, "cpu", torch.float32, **kw)
    st.load_weights(a)
    ptrs = {k: t.data_ptr() for k, t in _flat(st).items()}
    assert st.update_weights(b) == len(b)
    fresh = build_stage(cfg, 0, 4, "cpu", torch.float32, **kw)
    fresh.load_weights(b)
    got, want = _flat(st), _flat(fresh)
    for k in want:
        assert torch.equal(got[k], want[k]), k
        assert got[k].data_ptr() == ptrs[k], k


@pytest.mark.parametrize("name", ["tiny-mla", "tiny-hybrid", "tiny-msa"])
def test_refit_of_tensor_parallel_family_stages(name):
    cfg = named_config(name)
    fam = family_of(cfg.architecture)
    a, b = hf_state_dict(cfg, fam, seed=1), hf_state_dict(cfg, fam, seed=2)
    n_layers = cfg.num_hidden_layers
    kw = dict(tp_rank=1, tp_size=2, tp_group=None, comm=None)
    if cfg.is_moe:
        kw.update(ep_rank=1, ep_size=2, ep_comm=None)
    st = build_stage(cfg, 0, n_layers, "cpu", torch.float32, **kw)
    st.load_weights(a)
    ptrs = {k: t.data_ptr() for k, t in _flat(st).items()}
    assert st.update_weights(b) == len(b)
    fresh = build_stage(cfg, 0, n_layers, "cpu", torch.float32, **kw)
    fresh.load_weights(b)
    got, want = _flat(st), _flat(fresh)
    assert set(got) == set(want)
    for k in want:
        assert torch.equal(got[k], want[k]), k
        assert got[k].data_ptr() == ptrs[k], k
    assert st.cfg.num_attention_heads == cfg.num_attention_heads // 2
