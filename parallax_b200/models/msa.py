"""Pipeline-stage model for block-sparse ("MSA") attention models (MiniMax-M3 family).

Layers flagged in ``sparse_attention_config.sparse_attention_freq`` carry a small index head
(``index_q_proj`` with a few heads, ``index_k_proj`` with one) whose keys are cached next to K/V.
For every query token the indexer scores the 128-token blocks of the context, keeps the top-k
(initial and local blocks are always kept) and attention runs over those blocks only. Here the
selection becomes a *virtual block table* and the ordinary paged GQA kernel does the attention,
for decode and prefill alike; while the context still fits into top-k blocks the dense path is
used because the selection would keep everything.

Reference: ``src/parallax/models/minimax_m3.py:428-446`` (index projections), ``:456-565`` (block
top-k mask for prefill), ``:612-654`` (sparse decode), Gemma-style norms ``:194-203``. The clipped
``swigluoai`` activation of that family (``:176-180``) runs as a separate kernel between the two
grouped expert GEMMs (:mod:`parallax_b200.models.moe`) and between the gate/up and down projections of a dense
layer (:mod:`parallax_b200.models.decoder`).
"""

from __future__ import annotations

from typing import Optional

import torch

from parallax_b200 import ops
from parallax_b200.engine.batch import ForwardBatch
from parallax_b200.models.config import MSA_ATTENTION, ModelConfig
from parallax_b200.models.decoder import DecoderStage, _adopt


def _norm_rope_neox(x, w, cos_sin, positions, rot_dim: int, eps: float, offset: float):
    """RMSNorm over the last dim then rotate-half RoPE on its first ``rot_dim`` entries (fp32)."""
    xf = x.float()
    xf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * (w.float() + offset)
    if rot_dim:
        cs = cos_sin[positions.long()].float()
        cos, sin = cs[:, : rot_dim // 2], cs[:, rot_dim // 2:]
        while cos.dim() < xf.dim():
            cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)
        x1, x2 = xf[..., : rot_dim // 2], xf[..., rot_dim // 2:rot_dim]
        xf = torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin, xf[..., rot_dim:]], dim=-1)
    return xf.to(x.dtype)


class MSAStage(DecoderStage):
    def __init__(self, cfg: ModelConfig, start_layer: int, end_layer: int, device, dtype=None,
                 max_positions: Optional[int] = None):
        super().__init__(cfg, start_layer, end_layer, device, dtype, max_positions)
        raw = cfg.raw or {}
        sp = raw.get("sparse_attention_config") or {}
        self.norm_offset = 1.0 if raw.get("use_gemma_norm") else 0.0
        self.sparse_block = int(sp.get("sparse_block_size", raw.get("index_block_size") or 128))
        self.topk_blocks = int(sp.get("sparse_topk_blocks", raw.get("index_topk_blocks") or 16))
        self.init_blocks = int(sp.get("sparse_init_block", 0))
        self.local_blocks = max(1, int(sp.get("sparse_local_block", raw.get("index_local_blocks") or 1)))
        self.Di = int(sp.get("sparse_index_dim", raw.get("index_head_dim") or cfg.head_dim))
        self.Hi = int(sp.get("sparse_num_index_heads", 4))
        self.idx: dict[int, dict] = {}          # local layer index -> index-head weights

    def _is_sparse(self, gi: int) -> bool:
        return self.cfg.layer_kind(gi) == MSA_ATTENTION

    # ------------------------------------------------------------------ weights
    def init_random(self, seed: int = 0, std: float = 0.02) -> None:
        super().init_random(seed, std)
        dev, dt, H = self.device, self.dtype, self.cfg.hidden_size
        g = torch.Generator(device=dev)
        fill = 0.0 if self.norm_offset else 1.0
        if self.norm_offset:
            if self.norm_w is not None:
                self.norm_w = torch.zeros_like(self.norm_w)
            for lw in self.layers:
                lw.ln1, lw.ln2 = torch.zeros_like(lw.ln1), torch.zeros_like(lw.ln2)
                if lw.q_norm is not None:
                    lw.q_norm, lw.k_norm = torch.zeros_like(lw.q_norm), torch.zeros_like(lw.k_norm)
        for li, lw in enumerate(self.layers):
            if not self._is_sparse(lw.layer_idx):
                continue
            g.manual_seed(seed * 1000003 + lw.layer_idx * 16 + 777)
            w = (torch.randn((self.Hi + 1) * self.Di, H, generator=g, device=dev, dtype=torch.float32) * 0.1).to(dt)
            self.idx[li] = dict(w=w.contiguous(), q_norm=torch.full((self.Di,), fill, device=dev, dtype=dt),
                                k_norm=torch.full((self.Di,), fill, device=dev, dtype=dt))

    def load_weights(self, tensors) -> None:
        super().load_weights(tensors)
        dev, dt = self.device, self.dtype
        for li, lw in enumerate(self.layers):
            if not self._is_sparse(lw.layer_idx):
                continue
            a = f"model.layers.{lw.layer_idx}.self_attn."
            w = torch.cat([tensors[a + "index_q_proj.weight"], tensors[a + "index_k_proj.weight"]], dim=0)
            self.idx[li] = dict(w=w.to(device=dev, dtype=dt).contiguous(),
                                q_norm=tensors[a + "index_q_norm.weight"].to(device=dev, dtype=dt),
                                k_norm=tensors[a + "index_k_norm.weight"].to(device=dev, dtype=dt))

    def update_weights(self, tensors) -> int:
        """Online refit by layer reload, so that the index heads follow their layers."""
        return self.reload_layers(tensors)

    def _prepare_shadow(self, shadow) -> None:
        shadow.idx = {}

    def _adopt_layer(self, li: int, shadow) -> bool:
        replaced = super()._adopt_layer(li, shadow)
        if 0 in shadow.idx:
            self.idx[li], r = _adopt(self.idx.get(li), shadow.idx[0])
            replaced |= r
        return replaced

    def weight_bytes(self) -> int:
        extra = sum(t.numel() * t.element_size() for d in self.idx.values() for t in d.values())
        return super().weight_bytes() + extra

    # ------------------------------------------------------------------ forward
    def _attention(self, lw, li: int, xn: torch.Tensor, fb: ForwardBatch) -> torch.Tensor:
        ix = self.idx.get(li)
        limit = self.topk_blocks * self.sparse_block
        Tp = fb.num_prefill_tokens
        sparse_p = ix is not None and Tp > 0 and fb.p_max_ctx > limit
        sparse_d = ix is not None and fb.num_decode > 0 and fb.d_max_ctx > limit
        cache = self.kv_caches[li]
        if ix is not None:
            # index keys are written on every step, whether or not this step selects blocks
            T, Hi, Di = xn.shape[0], self.Hi, self.Di
            proj = ops.linear(xn, ix["w"])
            eps, rot = self.cfg.rms_norm_eps, self.cfg.rot_dim
            ik = _norm_rope_neox(proj[:, Hi * Di:], ix["k_norm"], self.cos_sin, fb.positions, rot, eps, self.norm_offset)
            ops.store_rows(ik.contiguous(), fb.slot_mapping, cache.index_k)
        if not (sparse_p or sparse_d):
            return super()._attention(lw, li, xn, fb)
        cfg = self.cfg
        Hq, Hkv, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        iq = _norm_rope_neox(proj[:, :Hi * Di].view(T, Hi, Di), ix["q_norm"], self.cos_sin, fb.positions, rot, eps,
                             self.norm_offset).contiguous()
        qkv = ops.linear(xn, lw.w_qkv, bias=lw.b_qkv)
        kc, vc = cache.k, cache.v
        kvs = cache.kv_scale
        ops.qk_norm_rope_cache(qkv, lw.q_norm, lw.k_norm, self.cos_sin, fb.positions, fb.slot_mapping, kc, vc, Hq, Hkv,
                               D, cfg.rot_dim, eps, self.norm_offset, kv_scale=kvs)
        q = qkv.view(T, Hq + 2 * Hkv, D)[:, :Hq]
        attn = torch.empty((T, Hq, D), dtype=qkv.dtype, device=qkv.device)
        page = kc.shape[-2]

        def sparse(part, tables, cu_q, max_ctx):
            pos = fb.positions[part]
            sc = ops.msa_block_scores(iq[part], cache.index_k, tables, cu_q, pos, max_ctx, self.sparse_block, self.scale)
            vt, vctx = ops.msa_select(sc, pos, tables, cu_q, page, self.sparse_block, self.topk_blocks, self.init_blocks,
                                      self.local_blocks)
            ops.attn_decode(q[part], kc, vc, vt, vctx, self.scale, max_ctx=limit, out=attn[part], kv_scale=kvs)

        if Tp:
            if sparse_p:
                sparse(slice(0, Tp), fb.p_block_tables, fb.p_cu_q, fb.p_max_ctx)
            else:
                ops.attn_prefill(q[:Tp], kc, vc, fb.p_block_tables, fb.p_cu_q, fb.p_ctx_lens, fb.p_max_q, self.scale,
                                 out=attn[:Tp], kv_scale=kvs)
        if fb.num_decode:
            if sparse_d:
                sparse(slice(Tp, T), fb.d_block_tables, None, fb.d_max_ctx)
            else:
                ops.attn_decode(q[Tp:], kc, vc, fb.d_block_tables, fb.d_ctx_lens, self.scale, max_ctx=fb.d_max_ctx,
                                out=attn[Tp:], kv_scale=kvs)
        return attn.view(T, Hq * D)
