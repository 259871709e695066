"""DeepSeek-style stages (MLA, and MLA + lightning-indexer sparse attention) on CPU against a
plain restatement of the architecture: expanded per-head K/V, full-sequence recomputation, dense
masks. The engine runs the absorbed form over the paged latent cache with chunked prefill."""

import pytest
import torch

from parallax_b200.engine.engine import Engine
from parallax_b200.engine.request import Request, SamplingParams
from parallax_b200.models.config import named_config
from parallax_b200.models.deepseek import derive_indexer_types
from parallax_b200.ops import reference as ref


def _rms(x, w, eps):
    x = x.float()
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w.float()


def oracle_last_logits(stage, tokens):
    cfg = stage.cfg
    T = len(tokens)
    pos = torch.arange(T, dtype=torch.int32)
    H, L, R, nope, V = stage.H, stage.L, stage.R, stage.nope, stage.V
    eps = cfg.rms_norm_eps
    h = stage.embed[torch.tensor(tokens)].float()
    causal = torch.tril(torch.ones(T, T, dtype=torch.bool))
    allowed = causal
    for lw in stage.layers:
        xn = _rms(h, lw.ln1, eps)
        qr = _rms(xn @ lw.w_q_a.float().t(), lw.q_a_norm, eps)
        q = (qr @ lw.w_q_b.float().t()).view(T, H, nope + R)
        kv = xn @ lw.w_kv_a.float().t()
        lat = _rms(kv[:, :L], lw.kv_a_norm, eps)
        k_pe = ref._rope_interleaved(kv[:, L:L + R], stage.cos_sin, pos)
        q_nope, q_pe = q[..., :nope], ref._rope_interleaved(q[..., nope:], stage.cos_sin, pos)
        w_uk = lw.w_uk_s.float().view(H, L, nope)
        w_uv = lw.w_uv_s.float().view(H, V, L)
        k_nope = torch.einsum("sc,hcd->shd", lat, w_uk)
        v = torch.einsum("sc,hvc->shv", lat, w_uv)
        if stage.dsa and lw.idx_mode == "full":
            Hi, Di = stage.Hi, stage.Di
            iq = (qr @ lw.idx_wq_b.float().t()).view(T, Hi, Di)
            iq = torch.cat([ref._rope_interleaved(iq[..., :R], stage.cos_sin, pos), iq[..., R:]], -1)
            n0 = lw.n_kv_a
            ik = torch.nn.functional.layer_norm(kv[:, n0:n0 + Di], (Di,), lw.idx_k_norm_w.float(),
                                                lw.idx_k_norm_b.float(), stage.idx_eps)
            ik = torch.cat([ref._rope_interleaved(ik[:, :R], stage.cos_sin, pos), ik[:, R:]], -1)
            iw = kv[:, n0 + Di:n0 + Di + Hi] * (Hi ** -0.5 * Di ** -0.5)
            sc = (torch.relu(torch.einsum("thd,sd->ths", iq, ik)) * iw[:, :, None]).sum(1)
            sc = sc.masked_fill(~causal, float("-inf"))
            allowed = causal.clone()
            k = cfg.index_topk
            for t in range(T):
                if t + 1 > k:
                    keep = torch.topk(sc[t, :t + 1], k).indices
                    allowed[t] = False
                    allowed[t, keep] = True
        s = torch.einsum("thd,shd->hts", q_nope, k_nope) + torch.einsum("thr,sr->hts", q_pe, k_pe)
        s = (s * stage.scale).masked_fill(~allowed[None], float("-inf"))
        o = torch.einsum("hts,shv->thv", torch.softmax(s, -1), v).reshape(T, H * V)
        h = h + o @ lw.w_o.float().t()
        xn = _rms(h, lw.ln2, eps)
        h = stage._mlp(lw, xn.to(stage.dtype), h.to(stage.dtype)).float()
    hn = _rms(h[-1:], stage.norm_w, eps)
    return (hn @ stage.lm_head.float().t())[0]


@pytest.mark.parametrize("name", ["tiny-mla", "tiny-dsa"])
def test_absorbed_paged_mla_matches_plain_restatement(name):
    torch.manual_seed(0)
    cfg = named_config(name)
    eng = Engine(cfg, device="cpu", num_blocks=64, page_size=16, max_batch_size=4, max_num_tokens_per_batch=256,
                 chunked_prefill_size=24, max_total_length=256)
    stage = eng.stages[0].model
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (41, 9, 30)]
    reqs = [Request(input_ids=p, sampling_params=SamplingParams(max_new_tokens=5, temperature=0.0, ignore_eos=True),
                    max_total_length=256) for p in prompts]
    for r in reqs:
        eng.add_request(r)
    while eng.has_work():
        eng.step()
    for p, r in zip(prompts, reqs):
        seq = list(p)
        for tok in r.output_ids:
            logits = oracle_last_logits(stage, seq)
            assert int(logits.argmax()) == tok, (name, len(seq))
            seq.append(tok)


def test_sparse_rows_differ_from_dense():
    """With more context than index_topk the DSA model must not equal plain MLA attention."""
    cfg = named_config("tiny-dsa")
    assert cfg.index_topk == 16 and derive_indexer_types(cfg) == ["full"] * cfg.num_hidden_layers
    cfg.raw["index_topk_freq"] = 2
    assert derive_indexer_types(cfg) == ["full", "shared", "full"]


def test_topk_select_and_index_scores_reference():
    torch.manual_seed(1)
    T, Hi, Di, page = 3, 4, 32, 16
    cache = torch.randn(8, 1, page, Di)
    bt = torch.tensor([[3, 1, 5], [0, 2, 4], [6, 7, 1]], dtype=torch.int32)
    pos = torch.tensor([40, 5, 33], dtype=torch.int32)
    q, w = torch.randn(T, Hi, Di), torch.rand(T, Hi)
    sc = ref.dsa_index_scores(q, w, cache, bt, None, pos, 41)
    assert sc.shape == (3, 64) and torch.isinf(sc[1, 6:]).all() and torch.isfinite(sc[0, :41]).all()
    top = ref.topk_select(sc, pos, 8)
    assert (top[1] == -1).all()
    assert set(top[0].tolist()) == set(torch.topk(sc[0, :41], 8).indices.tolist())
