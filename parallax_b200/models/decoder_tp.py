"""Tensor-parallel pipeline stage for the GQA decoder families.

Column-parallel QKV / gate-up, row-parallel o_proj / down_proj, KV heads split over ranks,
vocabulary-parallel lm_head. Between the fused ops the residual stream is sequence-sharded
(rank r owns token rows ``[r*Rp, (r+1)*Rp)``), so every collective is either an all-gather that
feeds a GEMM or a reduce-scatter that follows one - exactly the two fused kernels of
:mod:`parallax_b200.parallel.fused`. The same class runs on CPU ranks over gloo with plain
collectives (tests of the sharding logic).

Sharding rules follow the reference's ``shard()`` methods (``src/parallax/models/qwen3.py:181-195``:
q/k/v/gate/up "all-to-sharded", o/down "sharded-to-all"; KV heads divided by the TP size,
``src/parallax/server/executor/mlx_executor.py:218``).
"""

from __future__ import annotations

from typing import Optional

import torch

from parallax_b200 import ops
from parallax_b200.engine.batch import ForwardBatch
from parallax_b200.models.config import ModelConfig
from parallax_b200.models.decoder import DecoderStage


class TPStageMixin:
    """What every tensor-parallel stage shares, whatever its family: the sequence-sharded residual stream
    (rank r owns token rows ``[r*Rp, (r+1)*Rp)``), the embedding of the own rows, the vocabulary-parallel head
    and refit by reload. A family adds ``shard_weights`` and ``forward_layers_tp``."""

    def _tp_setup(self, tp_rank: int, tp_size: int, tp_group, comm) -> None:
        self.tp_rank, self.tp_size, self.tp_group = tp_rank, tp_size, tp_group
        self.comm = comm
        self._sharded = False

    # ------------------------------------------------------------------ weights
    def init_random(self, seed: int = 0, std: float = 0.02) -> None:
        super().init_random(seed, std)     # identical full weights on every rank, then slice
        self.shard_weights()

    def load_weights(self, tensors) -> None:
        super().load_weights(tensors)
        self.shard_weights()

    def update_weights(self, tensors) -> int:
        """Online refit: full tensors arrive, so every named layer goes through load + shard again."""
        return self.reload_layers(tensors)

    def _prepare_shadow(self, shadow) -> None:
        shadow._sharded = False

    def _shard_head(self) -> None:
        if self.lm_head is None:
            return
        r, tp = self.tp_rank, self.tp_size
        V = self.lm_head.shape[0]
        self.v_pad = (V + tp * 8 - 1) // (tp * 8) * (tp * 8)
        vl = self.v_pad // tp
        lo, hi = r * vl, min((r + 1) * vl, V)
        part = self.lm_head[lo:hi]
        if part.shape[0] < vl:   # last rank: pad with zero rows (cut off after the gather)
            part = torch.cat([part, part.new_zeros(vl - part.shape[0], part.shape[1])])
        tied = self.embed is not None and self.lm_head.data_ptr() == self.embed.data_ptr()
        self.lm_head = part.contiguous()
        self.vocab = V
        if tied and not self.is_first:
            self.embed = None

    # ------------------------------------------------------------------ forward
    def _embed_shard(self, fb: ForwardBatch, Rp: int) -> torch.Tensor:
        T, r = fb.num_tokens, self.tp_rank
        lo, hi = min(r * Rp, T), min((r + 1) * Rp, T)
        h = torch.zeros((Rp, self.cfg.hidden_size), dtype=self.dtype, device=self.device)
        if hi > lo:
            ops.gather_rows(self.embed, fb.input_ids[lo:hi], out=h[:hi - lo])
        return h

    def logits_tp(self, h_shard: torch.Tensor, fb: ForwardBatch) -> torch.Tensor:
        """Vocabulary-parallel head: every rank ends up with the full logits of the wanted rows."""
        hn = ops.rmsnorm(h_shard, self.norm_w, self.cfg.rms_norm_eps, w_offset=self.norm_offset)
        full = self.comm.all_gather_rows(hn)
        rows = ops.gather_rows(full, fb.logit_rows)
        local = ops.linear(rows, self.lm_head)
        return self.comm.all_gather_cols(local)[:, :self.vocab]

    def forward(self, fb: ForwardBatch, hidden: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``hidden`` (non-first stages) is this rank's row shard ``[Rp, H]``. Returns the shard
        (non-last stage) or logits ``[num_logits, V]`` (last stage)."""
        Rp = self.comm.rows_per_rank(fb.num_tokens)
        h = self._embed_shard(fb, Rp) if self.is_first else hidden
        h = self.forward_layers_tp(h, fb)
        return self.logits_tp(h, fb) if self.is_last else h


class TPDecoderStage(TPStageMixin, DecoderStage):
    def __init__(self, cfg: ModelConfig, start_layer: int, end_layer: int, device, dtype=None,
                 max_positions: Optional[int] = None, tp_rank: int = 0, tp_size: int = 1, tp_group=None,
                 comm=None):
        DecoderStage.__init__(self, cfg, start_layer, end_layer, device, dtype, max_positions)
        self._tp_setup(tp_rank, tp_size, tp_group, comm)
        if cfg.num_attention_heads % tp_size or cfg.num_key_value_heads % tp_size:
            raise ValueError("attention heads must divide by the tensor-parallel size")
        if not cfg.is_moe and cfg.intermediate_size % (64 * tp_size):
            raise ValueError("intermediate size must divide by 64 * tp")
        self.hq_l = cfg.num_attention_heads // tp_size
        self.hkv_l = cfg.num_key_value_heads // tp_size

    def shard_weights(self) -> None:
        if self._sharded:
            return
        cfg, r, tp = self.cfg, self.tp_rank, self.tp_size
        Hq, Hkv, D, I = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.intermediate_size
        hq, hkv, il = self.hq_l, self.hkv_l, I // tp
        for lw in self.layers:
            if lw.moe is not None:
                lw.moe.shard_experts(r, tp)     # expert parallelism over the same group
            q, k, v = lw.w_qkv.split([Hq * D, Hkv * D, Hkv * D], dim=0)
            lw.w_qkv = torch.cat([q[r * hq * D:(r + 1) * hq * D], k[r * hkv * D:(r + 1) * hkv * D],
                                  v[r * hkv * D:(r + 1) * hkv * D]], dim=0).contiguous()
            if lw.b_qkv is not None:
                bq, bk, bv = lw.b_qkv.split([Hq * D, Hkv * D, Hkv * D])
                lw.b_qkv = torch.cat([bq[r * hq * D:(r + 1) * hq * D], bk[r * hkv * D:(r + 1) * hkv * D],
                                      bv[r * hkv * D:(r + 1) * hkv * D]]).contiguous()
            lw.w_o = lw.w_o[:, r * hq * D:(r + 1) * hq * D].contiguous()
            if lw.moe is None:
                if self.dense_act_mode:     # [gate rows | up rows]
                    lw.w_gu = torch.cat([lw.w_gu[r * il:(r + 1) * il], lw.w_gu[I + r * il:I + (r + 1) * il]]).contiguous()
                else:
                    # gate/up are interleaved in groups of 64 outputs: a contiguous slice of groups is a slice of I
                    g = lw.w_gu.view(I // 64, 128, -1)
                    lw.w_gu = g[r * il // 64:(r + 1) * il // 64].reshape(2 * il, -1).contiguous()
                lw.w_down = lw.w_down[:, r * il:(r + 1) * il].contiguous()
            if lw.sinks is not None:
                lw.sinks = lw.sinks[r * hq:(r + 1) * hq].contiguous()
        self._shard_head()
        self._sharded = True

    # ------------------------------------------------------------------ forward
    def forward_layers_tp(self, h_shard: torch.Tensor, fb: ForwardBatch) -> torch.Tensor:
        cfg, comm = self.cfg, self.comm
        eps, D, T = cfg.rms_norm_eps, cfg.head_dim, fb.num_tokens
        hq, hkv = self.hq_l, self.hkv_l
        Tp = fb.num_prefill_tokens
        # per-request adapters: only steps in which some row uses one pay for them
        lora = self.lora if (self.lora is not None and fb.extras.get("lora_ids") is not None) else None
        for li, lw in enumerate(self.layers):
            qkv = comm.norm_ag_linear(h_shard, lw.ln1, eps, lw.w_qkv, bias=lw.b_qkv, w_offset=self.norm_offset)
            if lora is not None:
                qkv = lora.apply_tp("qkv", li, ops.rmsnorm(h_shard, lw.ln1, eps, w_offset=self.norm_offset), qkv, fb, comm)
            T_pad = qkv.shape[0]
            kc, vc = self.kv_caches[li]
            kvs = getattr(self.kv_caches[li], "kv_scale", (1.0, 1.0))
            real = qkv[:T]
            ops.qk_norm_rope_cache(real, lw.q_norm, lw.k_norm, self.cos_sin, fb.positions, fb.slot_mapping, kc, vc,
                                   hq, hkv, D, cfg.rot_dim, eps, self.norm_offset, kv_scale=kvs)
            q = real.view(T, hq + 2 * hkv, D)[:, :hq]
            attn = torch.zeros((T_pad, hq, D), dtype=qkv.dtype, device=qkv.device)
            if Tp:
                ops.attn_prefill(q[:Tp], kc, vc, fb.p_block_tables, fb.p_cu_q, fb.p_ctx_lens, fb.p_max_q,
                                 self.scale, window=lw.window, sinks=lw.sinks, out=attn[:Tp], kv_scale=kvs)
            if fb.num_decode:
                ops.attn_decode(q[Tp:], kc, vc, fb.d_block_tables, fb.d_ctx_lens, self.scale, window=lw.window,
                                sinks=lw.sinks, max_ctx=fb.d_max_ctx, out=attn[Tp:T], kv_scale=kvs)
            h_shard = comm.linear_rs(attn.view(T_pad, hq * D), lw.w_o, residual=h_shard)
            if lora is not None:
                h_shard = lora.apply_tp("o", li, attn.view(T_pad, hq * D), h_shard, fb, comm)
            if lw.moe is not None:
                # attention is tensor parallel, the experts are expert parallel: every rank routes its
                # own token rows and the dispatch / combine kernels move them to the experts' owners
                Rp = h_shard.shape[0]
                n_valid = min(max(T - self.tp_rank * Rp, 0), Rp)
                xn = ops.rmsnorm(h_shard, lw.ln2, eps, w_offset=self.norm_offset)
                ids, w = lw.moe.route(xn)
                base = lw.moe.shared_base(xn, h_shard)
                h_shard = comm.moe_ffn(xn, n_valid, ids, w, lw.moe.w1, lw.moe.w2, lw.moe.experts_per_rank, base=base)
                continue
            if self.dense_act_mode:
                act = ops.act_mul(comm.norm_ag_linear(h_shard, lw.ln2, eps, lw.w_gu, w_offset=self.norm_offset),
                                  self.dense_act_mode, self.dense_limit)
            else:
                act = comm.norm_ag_linear(h_shard, lw.ln2, eps, lw.w_gu, epi=ops.EPI_SILU_MUL, w_offset=self.norm_offset)
            h_shard = comm.linear_rs(act, lw.w_down, residual=h_shard)
            if lora is not None:
                h_shard = lora.apply_tp("down", li, act, h_shard, fb, comm)
        return h_shard
