"""Pipeline-stage model for the hybrid families (Qwen3-Next, Qwen3.5): most layers are Gated
DeltaNet linear-attention layers with a per-request recurrent state, every
``full_attention_interval``-th layer is a gated softmax-attention layer (output multiplied by
``sigmoid(gate)``, partial rotary, zero-centred RMSNorm weights).

Reference blocks: ``src/parallax/models/qwen3_next.py:63-66,146`` (gated attention),
``:149-230`` (Gated DeltaNet with conv and recurrent state slots), ``src/parallax/models/qwen3_5.py``
(same layers with split input projections); state slots are handed out per request like the
reference's ``LinearCache`` (``src/parallax/server/cache_manager.py:188-259``).

Projection layout used here (rows of one fused weight): ``in_proj = [q | k | v | z | b | a]`` with
heads in plain order, so checkpoints are re-ordered once at load time.
"""

from __future__ import annotations

from typing import Optional

import torch

from parallax_b200 import ops
from parallax_b200.engine.batch import ForwardBatch
from parallax_b200.models.config import LINEAR, ModelConfig
from parallax_b200.models.decoder import DecoderStage, LayerWeights


class LinearLayerWeights:
    __slots__ = ("ln1", "ln2", "w_in", "conv_w", "conv_b", "A_log", "dt_bias", "norm_w", "w_out", "w_gu", "w_down",
                 "moe", "layer_idx", "kind")

    def __init__(self):
        for s in self.__slots__:
            setattr(self, s, None)
        self.kind = LINEAR


class GatedAttnWeights(LayerWeights):
    __slots__ = ("w_gate", "kind")

    def __init__(self):
        for s in LayerWeights.__slots__:
            setattr(self, s, None)
        self.window = 0
        self.w_gate = None
        self.kind = "attention"


class HybridStage(DecoderStage):
    def __init__(self, cfg: ModelConfig, start_layer: int, end_layer: int, device, dtype=None,
                 max_positions: Optional[int] = None):
        super().__init__(cfg, start_layer, end_layer, device, dtype, max_positions)
        self.layers = [LinearLayerWeights() if cfg.layer_kind(i) == LINEAR else GatedAttnWeights()
                       for i in range(start_layer, end_layer)]
        self.norm_offset = 1.0      # these families store RMSNorm weights zero-centred
        self.Hk, self.Hv = cfg.linear_num_key_heads, cfg.linear_num_value_heads
        self.Dk, self.Dv = cfg.linear_key_head_dim, cfg.linear_value_head_dim
        self.Kc = cfg.linear_conv_kernel_dim
        self.qkv_dim = 2 * self.Hk * self.Dk + self.Hv * self.Dv

    # ------------------------------------------------------------------ weights
    def init_random(self, seed: int = 0, std: float = 0.02) -> None:
        cfg, dev, dt = self.cfg, self.device, self.dtype
        g = torch.Generator(device=dev)

        def rnd(*shape, layer_seed, scale=std):
            g.manual_seed(seed * 1000003 + layer_seed)
            return (torch.randn(*shape, generator=g, device=dev, dtype=torch.float32) * scale).to(dt)

        H, D = cfg.hidden_size, cfg.head_dim
        Hq, Hkv, I = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.intermediate_size
        zeros = lambda n: torch.zeros(n, device=dev, dtype=dt)  # noqa: E731  (zero-centred norm weight = scale 1)
        if self.is_first or (self.is_last and cfg.tie_word_embeddings):
            self.embed = rnd(cfg.vocab_size, H, layer_seed=900001)
        if self.is_last:
            self.norm_w = zeros(H)
            self.lm_head = self.embed if cfg.tie_word_embeddings else rnd(cfg.vocab_size, H, layer_seed=900002)
        for li, lw in enumerate(self.layers):
            gi = self.start_layer + li
            s = gi * 32
            lw.layer_idx = gi
            lw.ln1, lw.ln2 = zeros(H), zeros(H)
            if lw.kind == LINEAR:
                n_in = self.qkv_dim + self.Hv * self.Dv + 2 * self.Hv
                lw.w_in = rnd(n_in, H, layer_seed=s + 1)
                lw.conv_w = rnd(self.qkv_dim, self.Kc, layer_seed=s + 2, scale=0.3)
                lw.A_log = torch.log(torch.linspace(1.0, 8.0, self.Hv, device=dev)).float()
                lw.dt_bias = torch.linspace(-1.0, 1.0, self.Hv, device=dev).float()
                lw.norm_w = torch.ones(self.Dv, device=dev, dtype=dt)
                lw.w_out = rnd(H, self.Hv * self.Dv, layer_seed=s + 3)
            else:
                lw.window = 0
                lw.w_qkv = torch.cat([rnd(Hq * D, H, layer_seed=s + 1), rnd(Hkv * D, H, layer_seed=s + 2),
                                      rnd(Hkv * D, H, layer_seed=s + 3)], dim=0).contiguous()
                lw.w_gate = rnd(Hq * D, H, layer_seed=s + 4)
                lw.q_norm, lw.k_norm = zeros(D), zeros(D)
                lw.w_o = rnd(H, Hq * D, layer_seed=s + 5)
            if cfg.layer_is_moe(gi):
                from parallax_b200.models.moe import MoEWeights

                lw.moe = MoEWeights.random(cfg, dev, dt, lambda *sh, k: rnd(*sh, layer_seed=s + 10 + k))
            else:
                lw.w_gu = ops.interleave_gate_up(rnd(I, H, layer_seed=s + 6), rnd(I, H, layer_seed=s + 7))
                lw.w_down = rnd(H, I, layer_seed=s + 8)

    def load_weights(self, tensors: dict[str, torch.Tensor]) -> None:
        cfg, dev, dt = self.cfg, self.device, self.dtype
        Hk, Hv, Dk, Dv = self.Hk, self.Hv, self.Dk, self.Dv
        Hq, D = cfg.num_attention_heads, cfg.head_dim

        def get(name, required=True, dtype=dt):
            t = tensors.get(name)
            if t is None:
                for alt in (name.replace("model.", "model.language_model.", 1), name.replace("model.", "language_model.model.", 1)):
                    t = tensors.get(alt)
                    if t is not None:
                        break
            if t is None:
                if required:
                    raise KeyError(f"missing weight {name}")
                return None
            return t.to(device=dev, dtype=dtype)

        if self.is_first or (self.is_last and cfg.tie_word_embeddings):
            self.embed = get("model.embed_tokens.weight").contiguous()
        if self.is_last:
            self.norm_w = get("model.norm.weight")
            lm = get("lm_head.weight", required=False)
            self.lm_head = lm.contiguous() if lm is not None else self.embed
        for li, lw in enumerate(self.layers):
            gi = self.start_layer + li
            p = f"model.layers.{gi}."
            lw.layer_idx = gi
            lw.ln1 = get(p + "input_layernorm.weight")
            lw.ln2 = get(p + "post_attention_layernorm.weight")
            if lw.kind == LINEAR:
                a = p + "linear_attn."
                qkvz = get(a + "in_proj_qkvz.weight", required=False)
                if qkvz is not None:
                    # Qwen3-Next: rows grouped per key head as [q | k | v-heads | z-heads]; b/a likewise
                    r = Hv // Hk
                    g4 = qkvz.view(Hk, 2 * Dk + 2 * r * Dv, -1)
                    q, k = g4[:, :Dk].reshape(Hk * Dk, -1), g4[:, Dk:2 * Dk].reshape(Hk * Dk, -1)
                    v = g4[:, 2 * Dk:2 * Dk + r * Dv].reshape(Hv * Dv, -1)
                    z = g4[:, 2 * Dk + r * Dv:].reshape(Hv * Dv, -1)
                    ba = get(a + "in_proj_ba.weight").view(Hk, 2 * r, -1)
                    b, aa = ba[:, :r].reshape(Hv, -1), ba[:, r:].reshape(Hv, -1)
                else:
                    # Qwen3.5: separate projections in plain head order
                    qkv = get(a + "in_proj_qkv.weight")
                    q, k, v = qkv.split([Hk * Dk, Hk * Dk, Hv * Dv], dim=0)
                    z, b, aa = get(a + "in_proj_z.weight"), get(a + "in_proj_b.weight"), get(a + "in_proj_a.weight")
                lw.w_in = torch.cat([q, k, v, z, b, aa], dim=0).contiguous()
                lw.conv_w = get(a + "conv1d.weight").reshape(self.qkv_dim, self.Kc).contiguous()
                lw.conv_b = get(a + "conv1d.bias", required=False)
                lw.A_log = get(a + "A_log", dtype=torch.float32)
                lw.dt_bias = get(a + "dt_bias", dtype=torch.float32)
                lw.norm_w = get(a + "norm.weight")
                lw.w_out = get(a + "out_proj.weight").contiguous()
            else:
                a = p + "self_attn."
                lw.window = 0
                qg = get(a + "q_proj.weight").view(Hq, 2 * D, -1)          # per head: [q | gate]
                lw.w_qkv = torch.cat([qg[:, :D].reshape(Hq * D, -1), get(a + "k_proj.weight"), get(a + "v_proj.weight")],
                                     dim=0).contiguous()
                lw.w_gate = qg[:, D:].reshape(Hq * D, -1).contiguous()
                lw.q_norm, lw.k_norm = get(a + "q_norm.weight"), get(a + "k_norm.weight")
                lw.w_o = get(a + "o_proj.weight").contiguous()
            if cfg.layer_is_moe(gi):
                from parallax_b200.models.moe import MoEWeights

                lw.moe = MoEWeights.from_hf(cfg, tensors, p + "mlp.", dev, dt)
            else:
                lw.w_gu = ops.interleave_gate_up(get(p + "mlp.gate_proj.weight"), get(p + "mlp.up_proj.weight"))
                lw.w_down = get(p + "mlp.down_proj.weight").contiguous()

    def update_weights(self, tensors) -> int:
        """Online refit: every local layer named in ``tensors`` is rebuilt by the loader above (fused and
        absorbed layouts, expert shards, fp8 blocks) and moved into the live weights in place."""
        return self.reload_layers(tensors)

    def weight_bytes(self) -> int:
        seen, total = set(), 0
        for t in (self.embed, self.norm_w, self.lm_head):
            if t is not None and t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()
        for lw in self.layers:
            for cls in type(lw).__mro__:
                for s in getattr(cls, "__slots__", ()):
                    v = getattr(lw, s, None)
                    ts = [v] if isinstance(v, torch.Tensor) else (v.tensors() if hasattr(v, "tensors") else [])
                    for t in ts:
                        if t.data_ptr() not in seen:
                            seen.add(t.data_ptr())
                            total += t.numel() * t.element_size()
        return total

    # ------------------------------------------------------------------ forward
    def _linear_attention(self, lw: LinearLayerWeights, li: int, xn: torch.Tensor, fb: ForwardBatch) -> torch.Tensor:
        Hk, Hv, Dk, Dv = self.Hk, self.Hv, self.Dk, self.Dv
        cache = self.kv_caches[li]
        proj = ops.linear(xn, lw.w_in)                                   # [T, qkv | z | b | a]
        n_qkv, n_z = self.qkv_dim, Hv * Dv
        conv = ops.causal_conv1d_silu(proj[:, :n_qkv], lw.conv_w, lw.conv_b, cache.conv_state, fb.seq_cu, fb.seq_slots,
                                      fb.positions)
        z = proj[:, n_qkv:n_qkv + n_z]
        b = proj[:, n_qkv + n_z:n_qkv + n_z + Hv]
        a = proj[:, n_qkv + n_z + Hv:n_qkv + n_z + 2 * Hv]
        return ops.gated_delta_rule(conv, a, b, lw.A_log, lw.dt_bias, z, lw.norm_w, cache.rec_state, fb.seq_cu,
                                    fb.seq_slots, fb.positions, Hk, Hv, Dk, Dv, self.cfg.rms_norm_eps)

    def forward_layers(self, h: torch.Tensor, fb: ForwardBatch) -> torch.Tensor:
        eps = self.cfg.rms_norm_eps
        for li, lw in enumerate(self.layers):
            xn = ops.rmsnorm(h, lw.ln1, eps, w_offset=self.norm_offset)
            if lw.kind == LINEAR:
                a = self._linear_attention(lw, li, xn, fb)
                h = ops.linear(a, lw.w_out, residual=h)
            else:
                a = self._attention(lw, li, xn, fb)                      # q/k norm, partial RoPE, paged attention
                gate = ops.linear(xn, lw.w_gate)
                h = ops.linear(ops.sigmoid_gate_mul(a, gate), lw.w_o, residual=h)
            xn = ops.rmsnorm(h, lw.ln2, eps, w_offset=self.norm_offset)
            h = self._mlp(lw, xn, h)
        return h
