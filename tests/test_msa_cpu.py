"""Block-sparse (MSA) attention stage on CPU against a plain dense-mask restatement: the engine
selects blocks through virtual block tables over the paged cache; the oracle recomputes the whole
sequence and masks scores of unselected blocks."""

import torch

from parallax_b200.engine.engine import Engine
from parallax_b200.engine.request import Request, SamplingParams
from parallax_b200.models.config import named_config
from parallax_b200.models.msa import _norm_rope_neox
from parallax_b200.ops import reference as ref


def _rms(x, w, eps, off):
    x = x.float()
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * (w.float() + off)


def oracle_last_logits(stage, tokens):
    cfg = stage.cfg
    T = len(tokens)
    pos = torch.arange(T, dtype=torch.int32)
    Hq, Hkv, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    eps, off, rot = cfg.rms_norm_eps, stage.norm_offset, cfg.rot_dim
    h = stage.embed[torch.tensor(tokens)].float()
    causal = torch.tril(torch.ones(T, T, dtype=torch.bool))
    sb, topk = stage.sparse_block, stage.topk_blocks
    for li, lw in enumerate(stage.layers):
        xn = _rms(h, lw.ln1, eps, off)
        qkv = (xn @ lw.w_qkv.float().t()).view(T, Hq + 2 * Hkv, D)
        q = _norm_rope_neox(qkv[:, :Hq], lw.q_norm, stage.cos_sin, pos, rot, eps, off)
        k = _norm_rope_neox(qkv[:, Hq:Hq + Hkv], lw.k_norm, stage.cos_sin, pos, rot, eps, off)
        v = qkv[:, Hq + Hkv:]
        allowed = causal
        ix = stage.idx.get(li)
        if ix is not None:
            proj = xn @ ix["w"].float().t()
            iq = _norm_rope_neox(proj[:, : stage.Hi * stage.Di].view(T, stage.Hi, stage.Di), ix["q_norm"], stage.cos_sin,
                                 pos, rot, eps, off)
            ik = _norm_rope_neox(proj[:, stage.Hi * stage.Di:], ix["k_norm"], stage.cos_sin, pos, rot, eps, off)
            sc = (torch.einsum("thd,sd->ths", iq, ik) * stage.scale).masked_fill(~causal[:, None], float("-inf")).amax(1)
            allowed = causal.clone()
            for t in range(T):
                cur = t // sb
                if cur + 1 <= topk:
                    continue
                bs = torch.stack([sc[t, j * sb:(j + 1) * sb].max() for j in range(cur + 1)])
                bs[: stage.init_blocks] = 1e30
                bs[max(cur - stage.local_blocks + 1, 0):] = 1e29
                keep = torch.topk(bs, topk).indices
                blk_ok = torch.zeros(cur + 1, dtype=torch.bool)
                blk_ok[keep] = True
                allowed[t, : t + 1] = blk_ok[torch.arange(t + 1) // sb]
        rep = Hq // Hkv
        kk, vv = k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1)
        s = torch.einsum("thd,shd->hts", q, kk) * stage.scale
        s = s.masked_fill(~allowed[None], float("-inf"))
        o = torch.einsum("hts,shd->thd", torch.softmax(s, -1), vv).reshape(T, Hq * D)
        h = h + o @ lw.w_o.float().t()
        xn = _rms(h, lw.ln2, eps, off)
        act = ref.linear(xn, lw.w_gu.float(), epi=ref.EPI_SILU_MUL)
        h = h + act @ lw.w_down.float().t()
    hn = _rms(h[-1:], stage.norm_w, eps, off)
    return (hn @ stage.lm_head.float().t())[0]


def test_virtual_table_sparse_attention_matches_dense_mask():
    torch.manual_seed(0)
    cfg = named_config("tiny-msa")          # 32-token blocks, top-2 (1 initial + 1 local forced)
    eng = Engine(cfg, device="cpu", num_blocks=64, page_size=16, max_batch_size=4, max_num_tokens_per_batch=256,
                 chunked_prefill_size=48, max_total_length=256)
    stage = eng.stages[0].model
    assert stage.norm_offset == 1.0 and sorted(stage.idx) == [1, 2]
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (150, 20, 70)]
    reqs = [Request(input_ids=p, sampling_params=SamplingParams(max_new_tokens=4, temperature=0.0, ignore_eos=True),
                    max_total_length=256) for p in prompts]
    for r in reqs:
        eng.add_request(r)
    while eng.has_work():
        eng.step()
    for p, r in zip(prompts, reqs):
        seq = list(p)
        for tok in r.output_ids:
            assert int(oracle_last_logits(stage, seq).argmax()) == tok, len(seq)
            seq.append(tok)


def test_msa_select_forced_blocks_and_order():
    sc = torch.tensor([[0.1, 0.9, 0.5, 0.3, 0.2, 0.0]])
    bt = torch.arange(100, 124, dtype=torch.int32)[None]
    pos = torch.tensor([5 * 32 + 7], dtype=torch.int32)         # query in block 5
    vt, vctx = ref.msa_select(sc, pos, bt, None, 16, 32, 4, 1, 1)
    # kept: block 0 (initial), block 5 (local), then the best two of the rest: 1 and 2
    assert vt[0].tolist() == [100, 101, 102, 103, 104, 105, 110, 111]
    assert int(vctx[0]) == 3 * 32 + 8


def test_dense_layers_with_the_clipped_activation():
    """A dense FFN with ``swiglu_limit``: gate clipped from above, up clipped on both sides, ``g * sigmoid(1.702 g) * (u + 1)``."""
    import copy

    from helpers.hf_weights import hf_state_dict
    from parallax_b200.models.registry import build_stage

    cfg = copy.copy(named_config("tiny-msa"))
    cfg.swiglu_limit = 0.05            # small enough that the clipping really bites with these weights
    sd = hf_state_dict(cfg, "msa", seed=3)
    st = build_stage(cfg, 0, cfg.num_hidden_layers, "cpu", torch.float32)
    st.load_weights(sd)
    assert st.dense_act_mode == 1
    x = torch.randn(5, cfg.hidden_size)
    h = torch.randn(5, cfg.hidden_size)
    got = st._mlp(st.layers[1], x, h)
    g = x @ sd["model.layers.1.mlp.gate_proj.weight"].t()
    u = x @ sd["model.layers.1.mlp.up_proj.weight"].t()
    assert (g > 0.05).any() and (u.abs() > 0.05).any()
    g, u = g.clamp(max=0.05), u.clamp(-0.05, 0.05)
    want = h + (g * torch.sigmoid(1.702 * g) * (u + 1)) @ sd["model.layers.1.mlp.down_proj.weight"].t()
    assert torch.allclose(got, want, atol=1e-5)
    # the tensor-parallel cut of [gate rows | up rows] keeps the pairs together
    tp = build_stage(cfg, 0, cfg.num_hidden_layers, "cpu", torch.float32, tp_rank=1, tp_size=2)
    tp.load_weights(sd)
    I = cfg.intermediate_size
    assert torch.equal(tp.layers[1].w_gu[:I // 2], sd["model.layers.1.mlp.gate_proj.weight"][I // 2:])
    assert torch.equal(tp.layers[1].w_gu[I // 2:], sd["model.layers.1.mlp.up_proj.weight"][I // 2:])
    assert torch.equal(tp.layers[1].w_down, sd["model.layers.1.mlp.down_proj.weight"][:, I // 2:])
