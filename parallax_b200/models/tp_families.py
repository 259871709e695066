"""Tensor-parallel pipeline stages for the latent-attention (DeepSeek-V3 / V3.2, Kimi-K2, GLM-MoE-DSA), hybrid
(Qwen3-Next / Qwen3.5) and block-sparse (MiniMax-M3) families.

Layout, shared by the three: the residual stream is sequence-sharded between layers (rank r owns token rows
``[r*Rp, (r+1)*Rp)``, like the GQA decoder's tensor-parallel stage). A layer gathers the normalised rows, runs
the family's own attention code on this rank's HEADS over all tokens, and the output projection is followed by
a reduce-scatter that leaves every rank with its rows again. Dense FFNs are column- then row-parallel; layers
with experts keep their router and shared expert on every rank, split the experts over the group and run each
rank's own rows through the expert-parallel exchange, so no token is computed twice.

What is split and what is kept whole:

* MLA: ``q_b`` / ``kv_b`` (absorbed as ``W_UK`` / ``W_UV``) and ``o_proj`` by head; the two down-projections
  into the latents, their norms and the lightning indexer are kept whole, and every rank writes the same
  latent (and index-key) cache - the cache has no head dimension to split.
* Gated DeltaNet: key and value heads (their ``in_proj`` rows, convolution channels, decay parameters and
  ``out_proj`` columns); the recurrent and convolution state of a rank covers its heads only.
* Gated / block-sparse softmax attention: query and KV heads, the output gate with the query heads; the small
  index heads of the block-sparse layers are kept whole.

The reference shards the same families in their ``shard()`` methods
(``src/parallax/models/deepseek_v3.py:203-222``, ``src/parallax/models/deepseek_v32.py:449-487``,
``src/parallax/models/qwen3_next.py:232-262``, ``src/parallax/models/minimax_m3.py:801-816,867-909``) with an
all-reduce after the row-parallel projections.
"""

from __future__ import annotations

import copy
from typing import Optional

import torch

from parallax_b200 import ops
from parallax_b200.engine.batch import ForwardBatch
from parallax_b200.models.config import LINEAR, ModelConfig
from parallax_b200.models.decoder_tp import TPStageMixin
from parallax_b200.models.deepseek import DeepseekStage
from parallax_b200.models.hybrid import HybridStage
from parallax_b200.models.msa import MSAStage


def _part(t: Optional[torch.Tensor], rank: int, tp: int, dim: int = 0) -> Optional[torch.Tensor]:
    """Rank's ``1/tp`` slice of ``t`` along ``dim``."""
    if t is None:
        return None
    n = t.shape[dim] // tp
    return t.narrow(dim, rank * n, n).contiguous()


def _segments(t: Optional[torch.Tensor], sizes: list[int], rank: int, tp: int) -> Optional[torch.Tensor]:
    """``t`` is a stack of row segments of the given sizes; keep the rank's slice of each segment."""
    if t is None:
        return None
    return torch.cat([_part(seg, rank, tp) for seg in t.split(sizes, dim=0)], dim=0).contiguous()


class FamilyTPMixin(TPStageMixin):
    """The layer loop over a sequence-sharded residual stream; a family supplies its attention on local heads
    (``_tp_attention``), the row-parallel output weight and how its weights are cut."""

    def _family_setup(self, cfg: ModelConfig, tp_rank: int, tp_size: int, tp_group, comm) -> None:
        self._tp_setup(tp_rank, tp_size, tp_group, comm)
        self.full_cfg = cfg
        if cfg.num_attention_heads % tp_size:
            raise ValueError("attention heads must divide by the tensor-parallel size")
        if cfg.intermediate_size % (64 * tp_size) and any(not cfg.layer_is_moe(i) for i in
                                                          range(self.start_layer, self.end_layer)):
            raise ValueError("intermediate size must divide by 64 * tp")

    def _local_cfg(self) -> ModelConfig:
        c, tp = copy.copy(self.full_cfg), self.tp_size
        c.num_attention_heads = self.full_cfg.num_attention_heads // tp
        c.num_key_value_heads = max(1, self.full_cfg.num_key_value_heads // tp)
        c.intermediate_size = self.full_cfg.intermediate_size // tp
        return c

    def _prepare_shadow(self, shadow) -> None:
        shadow._sharded = False
        shadow.cfg = self.full_cfg
        self._set_head_view(shadow, full=True)

    def _set_head_view(self, stage, full: bool) -> None:
        """Family hook: point the head counts that the family's code reads at the full or the local numbers."""

    def _shard_dense_mlp(self, lw) -> None:
        I = self.full_cfg.intermediate_size
        r, tp = self.tp_rank, self.tp_size
        if isinstance(lw.w_gu, torch.Tensor) and lw.w_gu.shape[0] == 2 * I:
            il = I // tp
            if self.dense_act_mode:     # [gate rows | up rows]
                lw.w_gu = torch.cat([lw.w_gu[r * il:(r + 1) * il], lw.w_gu[I + r * il:I + (r + 1) * il]]).contiguous()
            else:
                # gate/up are interleaved in groups of 64 outputs: a contiguous run of groups is a slice of I
                lw.w_gu = lw.w_gu.view(I // 64, 128, -1)[r * il // 64:(r + 1) * il // 64].reshape(2 * il, -1).contiguous()
            lw.w_down = _part(lw.w_down, r, tp, dim=1)

    def shard_weights(self) -> None:
        if self._sharded:
            return
        for lw in self.layers:
            self._shard_layer(lw)
            if lw.moe is not None:
                self._ep_finish(lw.moe)
            else:
                self._shard_dense_mlp(lw)
        self._shard_head()
        self.cfg = self._local_cfg()
        self._set_head_view(self, full=False)
        self._sharded = True

    # ------------------------------------------------------------------ forward
    def _tp_mlp(self, lw, h_shard: torch.Tensor, n_valid: int) -> torch.Tensor:
        eps = self.cfg.rms_norm_eps
        if lw.moe is None:
            if self.dense_act_mode:
                act = ops.act_mul(self.comm.norm_ag_linear(h_shard, lw.ln2, eps, lw.w_gu, w_offset=self.norm_offset),
                                  self.dense_act_mode, self.dense_limit)
            else:
                act = self.comm.norm_ag_linear(h_shard, lw.ln2, eps, lw.w_gu, epi=ops.EPI_SILU_MUL,
                                               w_offset=self.norm_offset)
            return self.comm.linear_rs(act, lw.w_down, residual=h_shard)
        if lw.moe.ep is not None:
            lw.moe.ep.step_max_rows = h_shard.shape[0]
        if n_valid == 0:
            if lw.moe.ep is not None:
                lw.moe.idle(self.device, self.dtype)     # no row of its own: still part of the exchange
            return h_shard
        rows = h_shard[:n_valid]
        xn = ops.rmsnorm(rows, lw.ln2, eps, w_offset=self.norm_offset)
        out = lw.moe.forward(xn, rows)
        if n_valid == h_shard.shape[0]:
            return out
        h_shard = h_shard.clone()
        h_shard[:n_valid] = out
        return h_shard

    def forward_layers_tp(self, h_shard: torch.Tensor, fb: ForwardBatch) -> torch.Tensor:
        comm, eps, T = self.comm, self.cfg.rms_norm_eps, fb.num_tokens
        Rp = h_shard.shape[0]
        n_valid = min(max(T - self.tp_rank * Rp, 0), Rp)
        state: dict = {}
        for li, lw in enumerate(self.layers):
            xn = comm.all_gather_rows(ops.rmsnorm(h_shard, lw.ln1, eps, w_offset=self.norm_offset))
            a = self._tp_attention(lw, li, xn[:T], fb, state)                  # [T, local heads x head width]
            if a.shape[0] != Rp * self.tp_size:
                pad = torch.zeros((Rp * self.tp_size, a.shape[1]), dtype=a.dtype, device=a.device)
                pad[:T] = a
                a = pad
            h_shard = comm.linear_rs(a.contiguous(), self._tp_out_weight(lw), residual=h_shard)
            h_shard = self._tp_mlp(lw, h_shard, n_valid)
        return h_shard


# ---------------------------------------------------------------------------------------- MLA / DSA
class TPDeepseekStage(FamilyTPMixin, DeepseekStage):
    def __init__(self, cfg: ModelConfig, start_layer: int, end_layer: int, device, dtype=None,
                 max_positions: Optional[int] = None, tp_rank: int = 0, tp_size: int = 1, tp_group=None,
                 comm=None):
        DeepseekStage.__init__(self, cfg, start_layer, end_layer, device, dtype, max_positions)
        self._family_setup(cfg, tp_rank, tp_size, tp_group, comm)
        self.H_full = self.H

    def _set_head_view(self, stage, full: bool) -> None:
        stage.H = self.H_full if full else self.H_full // self.tp_size

    def _install_attention(self, lw, q_a, q_a_norm, q_b, kv_a, kv_a_norm, kv_b, w_o, idx=None):
        """Full tensors come in (from the checkpoint or the generator); the per-head ones are cut here, before
        the absorbed forms are built and before any fp8 quantisation."""
        r, tp = self.tp_rank, self.tp_size
        keep = self.H
        self.H = self.H_full // tp
        try:
            DeepseekStage._install_attention(self, lw, q_a, q_a_norm, _part(q_b, r, tp), kv_a, kv_a_norm,
                                             _part(kv_b, r, tp), _part(w_o, r, tp, dim=1), idx)
        finally:
            self.H = keep

    def _quantize_layer(self, lw) -> None:          # instance method on purpose: cut first, quantise after
        if lw.moe is None:
            self._shard_dense_mlp(lw)
        else:
            self._ep_finish(lw.moe)
        DeepseekStage._quantize_layer(lw)

    def _shard_layer(self, lw) -> None:
        pass                                        # attention was cut when it was installed

    def _tp_attention(self, lw, li, xn, fb, state):
        a, state["topk"] = self._attention(lw, li, xn, fb, state.get("topk"))
        return a

    def _tp_out_weight(self, lw):
        return lw.w_o


# ---------------------------------------------------------------------------------------- hybrid
class TPHybridStage(FamilyTPMixin, HybridStage):
    def __init__(self, cfg: ModelConfig, start_layer: int, end_layer: int, device, dtype=None,
                 max_positions: Optional[int] = None, tp_rank: int = 0, tp_size: int = 1, tp_group=None,
                 comm=None):
        HybridStage.__init__(self, cfg, start_layer, end_layer, device, dtype, max_positions)
        self._family_setup(cfg, tp_rank, tp_size, tp_group, comm)
        if cfg.linear_num_key_heads % tp_size or cfg.linear_num_value_heads % tp_size \
                or cfg.num_key_value_heads % tp_size:
            raise ValueError("linear-attention and KV heads must divide by the tensor-parallel size")
        self._heads_full = (self.Hk, self.Hv)

    def _set_head_view(self, stage, full: bool) -> None:
        d = 1 if full else self.tp_size
        stage.Hk, stage.Hv = self._heads_full[0] // d, self._heads_full[1] // d
        stage.qkv_dim = 2 * stage.Hk * stage.Dk + stage.Hv * stage.Dv

    def _shard_layer(self, lw) -> None:
        r, tp, cfg = self.tp_rank, self.tp_size, self.full_cfg
        if lw.kind == LINEAR:
            Hk, Hv = self._heads_full
            qk, vv = Hk * self.Dk, Hv * self.Dv
            if lw.w_in.shape[0] != 2 * qk + 2 * vv + 2 * Hv or lw.w_out.shape[1] != vv:
                return                              # already cut
            w_in = _segments(lw.w_in, [qk, qk, vv, vv, Hv, Hv], r, tp)
            if w_in.shape[0] % 8:        # the GEMM wants a multiple of 8 output columns: zero rows at the end
                w_in = torch.cat([w_in, w_in.new_zeros(8 - w_in.shape[0] % 8, w_in.shape[1])]).contiguous()
            lw.w_in = w_in
            lw.conv_w = _segments(lw.conv_w, [qk, qk, vv], r, tp)
            lw.conv_b = _segments(lw.conv_b, [qk, qk, vv], r, tp)
            lw.A_log, lw.dt_bias = _part(lw.A_log, r, tp), _part(lw.dt_bias, r, tp)
            lw.w_out = _part(lw.w_out, r, tp, dim=1)
            return
        Hq, Hkv, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        if lw.w_qkv.shape[0] != (Hq + 2 * Hkv) * D:
            return
        lw.w_qkv = _segments(lw.w_qkv, [Hq * D, Hkv * D, Hkv * D], r, tp)
        lw.w_gate = _part(lw.w_gate, r, tp)
        lw.w_o = _part(lw.w_o, r, tp, dim=1)

    def _tp_attention(self, lw, li, xn, fb, state):
        if lw.kind == LINEAR:
            return self._linear_attention(lw, li, xn, fb)
        a = self._attention(lw, li, xn, fb)
        return ops.sigmoid_gate_mul(a, ops.linear(xn, lw.w_gate))

    def _tp_out_weight(self, lw):
        return lw.w_out if lw.kind == LINEAR else lw.w_o


# ---------------------------------------------------------------------------------------- block-sparse
class TPMSAStage(FamilyTPMixin, MSAStage):
    def __init__(self, cfg: ModelConfig, start_layer: int, end_layer: int, device, dtype=None,
                 max_positions: Optional[int] = None, tp_rank: int = 0, tp_size: int = 1, tp_group=None,
                 comm=None):
        MSAStage.__init__(self, cfg, start_layer, end_layer, device, dtype, max_positions)
        self._family_setup(cfg, tp_rank, tp_size, tp_group, comm)
        if cfg.num_key_value_heads % tp_size:
            raise ValueError("KV heads must divide by the tensor-parallel size")

    def _prepare_shadow(self, shadow) -> None:
        FamilyTPMixin._prepare_shadow(self, shadow)
        shadow.idx = {}

    def _shard_layer(self, lw) -> None:
        r, tp, cfg = self.tp_rank, self.tp_size, self.full_cfg
        Hq, Hkv, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        if lw.w_qkv.shape[0] != (Hq + 2 * Hkv) * D:
            return
        lw.w_qkv = _segments(lw.w_qkv, [Hq * D, Hkv * D, Hkv * D], r, tp)
        lw.b_qkv = _segments(lw.b_qkv, [Hq * D, Hkv * D, Hkv * D], r, tp)
        lw.w_o = _part(lw.w_o, r, tp, dim=1)
        lw.w_g = _part(lw.w_g, r, tp)
        lw.sinks = _part(lw.sinks, r, tp)
        if cfg.qk_norm_full and lw.q_norm is not None:
            raise NotImplementedError("a norm over the whole q / k projection cannot be computed on a head shard")

    def _tp_attention(self, lw, li, xn, fb, state):
        return self._attention(lw, li, xn, fb)

    def _tp_out_weight(self, lw):
        return lw.w_o
