"""Pipeline-stage model for the MLA families: DeepSeek-V3, Kimi-K2 (dense latent attention) and
DeepSeek-V3.2 / GLM-MoE-DSA (latent attention over the top-k keys of a lightning indexer).

Attention runs in absorbed form for decode and prefill: the per-head up-projections of
``kv_b_proj`` are folded into the query (``W_UK``) and the output (``W_UV``), so the paged cache
holds only ``[latent 512 | rope 64]`` per token and one kernel serves every case
(:func:`parallax_b200.ops.mla_attn`). The reference keeps the same compressed cache but expands
K/V for prefill (``src/parallax/models/deepseek_v3.py:74-83,158-171``); its indexer and sparse
attention are ``src/parallax/models/deepseek_v32.py:84-238,376-446``. Per-layer indexer modes
("full" layers score keys, "shared" layers reuse the previous full layer's selection) follow
``deepseek_v32.py:24-57``; a stage must begin with a full layer (``:499-519``).
"""

from __future__ import annotations

import math
from typing import Optional

import torch

from parallax_b200 import ops
from parallax_b200.engine.batch import ForwardBatch
from parallax_b200.models.config import ModelConfig
from parallax_b200.models.decoder import DecoderStage


def derive_indexer_types(cfg: ModelConfig) -> list[str]:
    raw = cfg.raw or {}
    n = cfg.num_hidden_layers
    if raw.get("indexer_types") is not None:
        return list(raw["indexer_types"])
    freq = int(raw.get("index_topk_freq") or 1)
    if freq <= 1:
        return ["full"] * n
    off = raw.get("index_skip_topk_offset")
    off = freq - 1 if off is None else int(off)
    k0 = cfg.first_k_dense_replace
    return ["full" if (i < k0 or (i - k0) % freq == off) else "shared" for i in range(n)]


class MLALayer:
    __slots__ = ("ln1", "ln2", "w_q_a", "q_a_norm", "w_q_b", "w_kv_a", "kv_a_norm", "w_uk_s", "w_uv_s", "w_o",
                 "idx_wq_b", "idx_k_norm_w", "idx_k_norm_b", "idx_mode", "w_gu", "w_down", "moe", "layer_idx",
                 "n_kv_a")

    def __init__(self):
        for s in self.__slots__:
            setattr(self, s, None)


class DeepseekStage(DecoderStage):
    def __init__(self, cfg: ModelConfig, start_layer: int, end_layer: int, device, dtype=None,
                 max_positions: Optional[int] = None):
        super().__init__(cfg, start_layer, end_layer, device, dtype, max_positions)
        self.layers = [MLALayer() for _ in range(start_layer, end_layer)]
        self.H = cfg.num_attention_heads
        self.nope, self.R, self.V, self.L = cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim, cfg.kv_lora_rank
        self.qd = self.nope + self.R
        scale = 1.0 / math.sqrt(self.qd)
        sc = cfg.rope_scaling or {}
        if (sc.get("rope_type") or sc.get("type")) == "yarn" and sc.get("mscale_all_dim"):
            m = 0.1 * float(sc["mscale_all_dim"]) * math.log(float(sc.get("factor", 1.0))) + 1.0
            scale *= m * m
        self.scale = scale
        self.dsa = cfg.index_topk > 0
        self.Hi, self.Di = cfg.index_n_heads, cfg.index_head_dim
        self.idx_types = derive_indexer_types(cfg) if self.dsa else []
        if self.dsa and self.layers and self.idx_types[start_layer] != "full":
            raise ValueError("a DSA stage must start on a layer that runs the indexer")
        self.idx_eps = float((cfg.raw or {}).get("indexer_norm_eps", 1e-5))

    # ------------------------------------------------------------------ weights
    def _install_attention(self, lw: MLALayer, q_a, q_a_norm, q_b, kv_a, kv_a_norm, kv_b, w_o, idx=None):
        H, nope, V, L = self.H, self.nope, self.V, self.L
        lw.w_q_a, lw.q_a_norm, lw.w_q_b = q_a, q_a_norm, q_b.contiguous()
        rows = [kv_a]
        if idx is not None:
            lw.idx_wq_b = idx["wq_b"].contiguous()
            lw.idx_k_norm_w, lw.idx_k_norm_b = idx["k_norm_w"], idx["k_norm_b"]
            rows += [idx["wk"], idx["weights_proj"]]
        lw.n_kv_a = kv_a.shape[0]
        lw.w_kv_a = torch.cat(rows, dim=0).contiguous()      # one GEMM: latent | rope (| index key | head weights)
        lw.kv_a_norm = kv_a_norm
        kvb = kv_b.view(H, nope + V, L)
        lw.w_uk_s = kvb[:, :nope].transpose(1, 2).reshape(H * L, nope).contiguous()   # q_lat = W_UK^T q_nope
        lw.w_uv_s = kvb[:, nope:].reshape(H * V, L).contiguous()                        # o = W_UV o_lat
        lw.w_o = w_o.contiguous()

    def init_random(self, seed: int = 0, std: float = 0.02) -> None:
        cfg, dev, dt = self.cfg, self.device, self.dtype
        g = torch.Generator(device=dev)

        def rnd(*shape, layer_seed):
            g.manual_seed(seed * 1000003 + layer_seed)
            return (torch.randn(*shape, generator=g, device=dev, dtype=torch.float32) * std).to(dt)

        Hd, H, I = cfg.hidden_size, self.H, cfg.intermediate_size
        ones = lambda n: torch.ones(n, device=dev, dtype=dt)  # noqa: E731
        if self.is_first or (self.is_last and cfg.tie_word_embeddings):
            self.embed = rnd(cfg.vocab_size, Hd, layer_seed=900001)
        if self.is_last:
            self.norm_w = ones(Hd)
            self.lm_head = self.embed if cfg.tie_word_embeddings else rnd(cfg.vocab_size, Hd, layer_seed=900002)
        ql = cfg.q_lora_rank
        for li, lw in enumerate(self.layers):
            gi = self.start_layer + li
            s = gi * 32
            lw.layer_idx = gi
            lw.ln1, lw.ln2 = ones(Hd), ones(Hd)
            if ql:
                q_a, q_a_norm, q_b = rnd(ql, Hd, layer_seed=s + 1), ones(ql), rnd(H * self.qd, ql, layer_seed=s + 2)
            else:
                q_a, q_a_norm, q_b = None, None, rnd(H * self.qd, Hd, layer_seed=s + 2)
            idx = None
            if self.dsa:
                lw.idx_mode = self.idx_types[gi]
                if lw.idx_mode == "full":
                    idx = dict(wq_b=rnd(self.Hi * self.Di, ql or Hd, layer_seed=s + 20), wk=rnd(self.Di, Hd, layer_seed=s + 21),
                               k_norm_w=ones(self.Di), k_norm_b=torch.zeros(self.Di, device=dev, dtype=dt),
                               weights_proj=rnd(self.Hi, Hd, layer_seed=s + 22))
            self._install_attention(lw, q_a, q_a_norm, q_b, rnd(self.L + self.R, Hd, layer_seed=s + 3), ones(self.L),
                                    rnd(H * (self.nope + self.V), self.L, layer_seed=s + 4),
                                    rnd(Hd, H * self.V, layer_seed=s + 5), idx)
            if cfg.layer_is_moe(gi):
                from parallax_b200.models.moe import MoEWeights

                lw.moe = MoEWeights.random(cfg, dev, dt, lambda *sh, k: rnd(*sh, layer_seed=s + 10 + k),
                                           expert_shard=self._ep_shard_arg())
                self._ep_finish(lw.moe)
            else:
                lw.w_gu = ops.interleave_gate_up(rnd(I, Hd, layer_seed=s + 6), rnd(I, Hd, layer_seed=s + 7))
                lw.w_down = rnd(Hd, I, layer_seed=s + 8)
            if cfg.quant_method == "fp8":
                self._quantize_layer(lw)      # layer by layer: the bf16 copy of a 671B model never exists at once
        if cfg.quant_method == "fp8":
            self.fp8 = True

    def load_weights(self, tensors: dict[str, torch.Tensor]) -> None:
        cfg, dev, dt = self.cfg, self.device, self.dtype
        from parallax_b200.loader.quant import dequant_if_needed

        def get(name, required=True):
            t = tensors.get(name)
            if t is None:
                if required:
                    raise KeyError(f"missing weight {name}")
                return None
            return dequant_if_needed(tensors, name, cfg).to(device=dev, dtype=dt)

        if self.is_first or (self.is_last and cfg.tie_word_embeddings):
            self.embed = get("model.embed_tokens.weight").contiguous()
        if self.is_last:
            self.norm_w = get("model.norm.weight")
            lm = get("lm_head.weight", required=False)
            self.lm_head = lm.contiguous() if lm is not None else self.embed
        for li, lw in enumerate(self.layers):
            gi = self.start_layer + li
            p = f"model.layers.{gi}."
            a = p + "self_attn."
            lw.layer_idx = gi
            lw.ln1 = get(p + "input_layernorm.weight")
            lw.ln2 = get(p + "post_attention_layernorm.weight")
            if cfg.q_lora_rank:
                q_a, q_a_norm, q_b = get(a + "q_a_proj.weight"), get(a + "q_a_layernorm.weight"), get(a + "q_b_proj.weight")
            else:
                q_a, q_a_norm, q_b = None, None, get(a + "q_proj.weight")
            idx = None
            if self.dsa:
                lw.idx_mode = self.idx_types[gi]
                if lw.idx_mode == "full":
                    i = a + "indexer."
                    kb = get(i + "k_norm.bias", required=False)
                    idx = dict(wq_b=get(i + "wq_b.weight"), wk=get(i + "wk.weight"), k_norm_w=get(i + "k_norm.weight"),
                               k_norm_b=kb if kb is not None else torch.zeros(self.Di, device=dev, dtype=dt),
                               weights_proj=get(i + "weights_proj.weight"))
            self._install_attention(lw, q_a, q_a_norm, q_b, get(a + "kv_a_proj_with_mqa.weight"),
                                    get(a + "kv_a_layernorm.weight"), get(a + "kv_b_proj.weight"),
                                    get(a + "o_proj.weight"), idx)
            if cfg.layer_is_moe(gi):
                from parallax_b200.models.moe import MoEWeights

                lw.moe = MoEWeights.from_hf(cfg, tensors, p + "mlp.", dev, dt)
                self._ep_finish(lw.moe)
            else:
                lw.w_gu = ops.interleave_gate_up(get(p + "mlp.gate_proj.weight"), get(p + "mlp.up_proj.weight"))
                lw.w_down = get(p + "mlp.down_proj.weight").contiguous()
        if cfg.quant_method == "fp8":
            self.quantize_fp8()

    def quantize_fp8(self) -> None:
        """Keep the large projections (q_b, o, dense FFN, experts) as block-scaled e4m3; the narrow
        down-projections into the latents, norms, router and embeddings stay bf16."""
        for lw in self.layers:
            self._quantize_layer(lw)
        self.fp8 = True

    @staticmethod
    def _quantize_layer(lw) -> None:
        from parallax_b200.loader.quant import quantize_fp8_block

        for name in ("w_q_b", "w_o", "w_gu", "w_down"):
            w = getattr(lw, name)
            if isinstance(w, torch.Tensor) and w.shape[0] % 128 == 0 and w.shape[1] % 128 == 0:
                setattr(lw, name, quantize_fp8_block(w, (64, 128)))
        if lw.moe is not None and lw.moe.fp8 is None:
            lw.moe.quantize_fp8()

    @staticmethod
    def _lin(x, w, residual=None, epi=ops.EPI_NONE):
        if isinstance(w, tuple):
            return ops.linear_fp8(x, w[0], w[1], residual=residual, epi=epi)
        return ops.linear(x, w, residual=residual, epi=epi)

    def _mlp(self, lw, xn, h):
        if lw.moe is not None:
            return lw.moe.forward(xn, h)
        return self._lin(self._lin(xn, lw.w_gu, epi=ops.EPI_SILU_MUL), lw.w_down, residual=h)

    def update_weights(self, tensors) -> int:
        """Online refit: every local layer named in ``tensors`` is rebuilt by the loader above (fused and
        absorbed layouts, expert shards, fp8 blocks) and moved into the live weights in place."""
        return self.reload_layers(tensors)

    def weight_bytes(self) -> int:
        seen, total = set(), 0
        def add(t):
            nonlocal total
            if isinstance(t, torch.Tensor) and t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()
        for t in (self.embed, self.norm_w, self.lm_head):
            add(t)
        for lw in self.layers:
            for s in MLALayer.__slots__:
                v = getattr(lw, s)
                if isinstance(v, torch.Tensor):
                    add(v)
                elif isinstance(v, tuple):
                    for t in v:
                        add(t)
                elif v is not None and hasattr(v, "tensors"):
                    for t in v.tensors():
                        add(t)
        return total

    # ------------------------------------------------------------------ forward
    def _index_topk(self, lw: MLALayer, li: int, qr: torch.Tensor, kv: torch.Tensor, fb: ForwardBatch):
        """Run the lightning indexer of a "full" layer: store this step's index keys, score the
        context and select the top-k key positions per query token (-1 rows = attend densely)."""
        cfg, T, Hi, Di, R = self.cfg, qr.shape[0], self.Hi, self.Di, self.R
        k_top = cfg.index_topk
        cache = self.kv_caches[li].index_k
        iq = ops.linear(qr, lw.idx_wq_b).view(T, Hi, Di)
        n0 = lw.n_kv_a
        # one launch: rotate the index queries, norm + rotate + store the index key, scale the head weights
        iw = ops.dsa_index_prep(iq, kv, n0, n0 + Di, lw.idx_k_norm_w, lw.idx_k_norm_b, self.idx_eps, self.cos_sin,
                                fb.positions, fb.slot_mapping, cache, Hi ** -0.5 * Di ** -0.5, R)
        Tp = fb.num_prefill_tokens
        need_p = Tp > 0 and fb.p_max_ctx > k_top
        need_d = fb.num_decode > 0 and fb.d_max_ctx > k_top
        if not (need_p or need_d):
            return None
        topk = torch.full((T, k_top), -1, dtype=torch.int32, device=qr.device)
        if need_p:
            sc = ops.dsa_index_scores(iq[:Tp], iw[:Tp], cache, fb.p_block_tables, fb.p_cu_q, fb.positions[:Tp],
                                      fb.p_max_ctx)
            topk[:Tp] = ops.topk_select(sc, fb.positions[:Tp], k_top)
        if need_d:
            sc = ops.dsa_index_scores(iq[Tp:], iw[Tp:], cache, fb.d_block_tables, None, fb.positions[Tp:],
                                      fb.d_max_ctx)
            topk[Tp:] = ops.topk_select(sc, fb.positions[Tp:], k_top)
        return topk

    def _attention(self, lw: MLALayer, li: int, xn: torch.Tensor, fb: ForwardBatch, topk_prev):
        cfg, T, H = self.cfg, xn.shape[0], self.H
        eps = cfg.rms_norm_eps
        if lw.w_q_a is not None:
            qr = ops.rmsnorm(ops.linear(xn, lw.w_q_a), lw.q_a_norm, eps)
        else:
            qr = xn
        q = self._lin(qr, lw.w_q_b)
        kv = ops.linear(xn, lw.w_kv_a)
        cache = self.kv_caches[li].k
        ops.mla_kv_prep(kv[:, :lw.n_kv_a], lw.kv_a_norm, self.cos_sin, fb.positions, fb.slot_mapping, cache, eps, self.L)
        topk = topk_prev
        if self.dsa and lw.idx_mode == "full":
            topk = self._index_topk(lw, li, qr, kv, fb)
        q_lat, q_pe = ops.mla_q_absorb(q, lw.w_uk_s, self.cos_sin, fb.positions, H, self.nope, self.L)
        Tp = fb.num_prefill_tokens
        o_lat = None
        if Tp:
            o_lat = ops.mla_attn(q_lat, q_pe, cache, fb.p_block_tables, fb.p_cu_q, fb.positions, self.scale, 0, Tp,
                                 topk=topk)
        if fb.num_decode:
            o_lat = ops.mla_attn(q_lat, q_pe, cache, fb.d_block_tables, None, fb.positions, self.scale, Tp,
                                 fb.num_decode, topk=topk, out=o_lat)
        return ops.mla_unabsorb(o_lat, lw.w_uv_s, T), topk

    def forward_layers(self, h: torch.Tensor, fb: ForwardBatch) -> torch.Tensor:
        eps = self.cfg.rms_norm_eps
        topk = None
        for li, lw in enumerate(self.layers):
            xn = ops.rmsnorm(h, lw.ln1, eps)
            a, topk = self._attention(lw, li, xn, fb, topk)
            h = self._lin(a.contiguous(), lw.w_o, residual=h)
            xn = ops.rmsnorm(h, lw.ln2, eps)
            h = self._mlp(lw, xn, h)
        return h
