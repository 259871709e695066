"""Pipeline-stage model for GQA decoder-only transformers (Llama, Qwen2, Qwen3, Qwen3-MoE,
GLM4-MoE, MiniMax-M2, GPT-OSS, Step-3.5 families).

A stage owns decoder layers ``[start_layer, end_layer)``; the first stage also owns the
embedding table, the last stage the final norm, lm_head and sampling inputs — the same
split the reference uses for its shards (``src/parallax/server/model.py:52-73``) and
contract per block (``src/parallax/models/qwen3.py:56-203``).

Weights are stored in the fused layouts the kernels want:
  * ``w_qkv``  [(Hq+2Hkv)*D, H]       (q | k | v rows)
  * ``w_gu``   [2I, H]                gate/up rows interleaved in groups of 64 (see
                                      :func:`parallax_b200.ops.interleave_gate_up`)
The same code runs on CPU (fp32, reference ops) and on B200 (bf16, sm_100a kernels).
"""

from __future__ import annotations

import math
import re
from typing import Optional

import torch

from parallax_b200 import ops
from parallax_b200.engine.batch import ForwardBatch
from parallax_b200.models.config import ModelConfig
from parallax_b200.models.rope import build_rope_table


class LayerWeights:
    __slots__ = (
        "ln1", "ln2", "w_qkv", "b_qkv", "q_norm", "k_norm", "w_o", "b_o", "w_gu", "w_down", "sinks",
        "moe", "window", "layer_idx", "w_g",
    )

    def __init__(self):
        for s in self.__slots__:
            setattr(self, s, None)
        self.window = 0


def _adopt(old, new):
    """Move ``new`` (a tensor, a tuple / dict of tensors, or a weights object) into ``old``'s storage where the
    two are congruent. Returns ``(value to keep, replaced)``; ``replaced`` is True when some storage changed."""
    if isinstance(new, torch.Tensor):
        if isinstance(old, torch.Tensor) and old.shape == new.shape and old.dtype == new.dtype \
                and old.device == new.device:
            old.copy_(new)
            return old, False
        return new, True
    if isinstance(new, (tuple, list)):
        if isinstance(old, (tuple, list)) and len(old) == len(new):
            pairs = [_adopt(o, n) for o, n in zip(old, new)]
            return type(new)(v for v, _r in pairs), any(r for _v, r in pairs)
        return new, True
    if isinstance(new, dict):
        if not isinstance(old, dict):
            return new, True
        replaced = set(old) != set(new)
        out = {}
        for k, v in new.items():
            out[k], r = _adopt(old.get(k), v)
            replaced |= r
        return out, replaced
    slots = [s for c in type(new).__mro__ for s in getattr(c, "__slots__", ())]
    names = slots or (list(vars(new)) if hasattr(new, "__dict__") and hasattr(new, "tensors") else None)
    if names and old is not None and type(old) is type(new):
        replaced = False
        for name in names:
            if not hasattr(new, name):
                continue
            val, r = _adopt(getattr(old, name, None), getattr(new, name))
            setattr(old, name, val)
            replaced |= r
        return old, replaced
    return new, (old is not None and new is not old and isinstance(old, (torch.Tensor, tuple, list, dict)))


from parallax_b200.models.moe import ExpertParallelMixin  # noqa: E402


class DecoderStage(ExpertParallelMixin):
    def __init__(self, cfg: ModelConfig, start_layer: int, end_layer: int, device, dtype=None,
                 max_positions: Optional[int] = None):
        self.cfg = cfg
        self.start_layer = start_layer
        self.end_layer = end_layer
        self.device = torch.device(device)
        self.dtype = dtype or (torch.bfloat16 if self.device.type == "cuda" else torch.float32)
        self.is_first = start_layer == 0
        self.is_last = end_layer == cfg.num_hidden_layers
        self.layers: list[LayerWeights] = [LayerWeights() for _ in range(start_layer, end_layer)]
        self.embed: Optional[torch.Tensor] = None
        self.norm_w: Optional[torch.Tensor] = None
        self.lm_head: Optional[torch.Tensor] = None
        self.scale = 1.0 / math.sqrt(cfg.head_dim)
        self.max_positions = max_positions or cfg.max_position_embeddings
        self.cos_sin = build_rope_table(cfg, self.max_positions, self.device)
        self.kv_caches: list = []  # per local layer: (k_cache, v_cache)
        self.norm_offset = 0.0
        self._native = None     # native stage executor (built on first use) or False if not applicable
        # dense FFN activation: 0 = SwiGLU fused into the gate/up GEMM's epilogue (rows interleaved in groups
        # of 64); 1 = the clipped "swigluoai" of GPT-OSS / MiniMax-M3 (``src/parallax/models/minimax_m3.py:176-180``),
        # gate rows then up rows, activation as its own kernel between the two GEMMs
        self.dense_act_mode = 1 if (cfg.swiglu_limit or cfg.hidden_act == "swigluoai") else 0
        self.dense_limit = float(cfg.swiglu_limit or 7.0)
        self.lora = None        # parallax_b200.loader.lora.LoRAStack when per-request adapters are enabled
        self.routed_buf = None  # [kv slots, MoE layers, top-k] int16 when routed experts are recorded
        self._route_slots = None

    # ------------------------------------------------------------------ weights
    def num_local_layers(self) -> int:
        return self.end_layer - self.start_layer

    def init_random(self, seed: int = 0, std: float = 0.02) -> None:
        """Random N(0, std) weights of the configured architecture (benchmarks, tests)."""
        cfg, dev, dt = self.cfg, self.device, self.dtype
        g = torch.Generator(device=dev)

        def rnd(*shape, layer_seed):
            g.manual_seed(seed * 1000003 + layer_seed)
            return (torch.randn(*shape, generator=g, device=dev, dtype=torch.float32) * std).to(dt)

        H, D = cfg.hidden_size, cfg.head_dim
        Hq, Hkv, I = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.intermediate_size
        if self.is_first or (self.is_last and cfg.tie_word_embeddings):
            self.embed = rnd(cfg.vocab_size, H, layer_seed=900001)
        if self.is_last:
            self.norm_w = torch.ones(H, device=dev, dtype=dt)
            self.lm_head = self.embed if cfg.tie_word_embeddings else rnd(cfg.vocab_size, H, layer_seed=900002)
        for li, lw in enumerate(self.layers):
            gi = self.start_layer + li
            s = gi * 16
            lw.layer_idx = gi
            lw.window = cfg.layer_window(gi)
            lw.ln1 = torch.ones(H, device=dev, dtype=dt)
            lw.ln2 = torch.ones(H, device=dev, dtype=dt)
            wq = rnd(Hq * D, H, layer_seed=s + 1)
            wk = rnd(Hkv * D, H, layer_seed=s + 2)
            wv = rnd(Hkv * D, H, layer_seed=s + 3)
            lw.w_qkv = torch.cat([wq, wk, wv], dim=0).contiguous()
            if cfg.attention_bias:
                lw.b_qkv = rnd((Hq + 2 * Hkv) * D, layer_seed=s + 4)
            if cfg.qk_norm_full:      # one norm over the whole q / k projection (MiniMax-M2)
                lw.q_norm = 1.0 + rnd(Hq * D, layer_seed=s + 30)
                lw.k_norm = 1.0 + rnd(Hkv * D, layer_seed=s + 31)
            elif cfg.qk_norm:
                lw.q_norm = torch.ones(D, device=dev, dtype=dt)
                lw.k_norm = torch.ones(D, device=dev, dtype=dt)
            if (cfg.raw or {}).get("use_head_wise_attn_gate"):  # head-wise sigmoid gate on the attention output (Step-3.5)
                lw.w_g = rnd(Hq, H, layer_seed=s + 32)
            lw.w_o = rnd(H, Hq * D, layer_seed=s + 5)
            if cfg.attention_sinks:
                lw.sinks = rnd(Hq, layer_seed=s + 9).float()
            if cfg.layer_is_moe(gi):
                from parallax_b200.models.moe import MoEWeights

                lw.moe = MoEWeights.random(cfg, dev, dt, lambda *sh, k: rnd(*sh, layer_seed=s + 10 + k),
                                           expert_shard=self._ep_shard_arg())
                self._ep_finish(lw.moe)
            else:
                wg = rnd(I, H, layer_seed=s + 6)
                wu = rnd(I, H, layer_seed=s + 7)
                lw.w_gu = self._pack_gate_up(wg, wu)
                lw.w_down = rnd(H, I, layer_seed=s + 8)

    def load_weights(self, tensors: dict[str, torch.Tensor]) -> None:
        """Install HF-named tensors (already filtered to this stage's layer range)."""
        cfg, dev, dt = self.cfg, self.device, self.dtype

        def get(name, required=True):
            t = tensors.get(name)
            if t is None:
                if required:
                    raise KeyError(f"missing weight {name}")
                return None
            return t.to(device=dev, dtype=dt)

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
            lw.window = cfg.layer_window(gi)
            lw.ln1 = get(p + "input_layernorm.weight")
            lw.ln2 = get(p + "post_attention_layernorm.weight")
            lw.w_qkv = torch.cat([get(p + "self_attn.q_proj.weight"), get(p + "self_attn.k_proj.weight"),
                                  get(p + "self_attn.v_proj.weight")], dim=0).contiguous()
            bq = get(p + "self_attn.q_proj.bias", required=False)
            if bq is not None:
                lw.b_qkv = torch.cat([bq, get(p + "self_attn.k_proj.bias"),
                                      get(p + "self_attn.v_proj.bias")]).contiguous()
            lw.q_norm = get(p + "self_attn.q_norm.weight", required=False)
            lw.k_norm = get(p + "self_attn.k_norm.weight", required=False)
            lw.w_o = get(p + "self_attn.o_proj.weight").contiguous()
            lw.b_o = get(p + "self_attn.o_proj.bias", required=False)
            lw.w_g = get(p + "self_attn.g_proj.weight", required=False)
            sk = tensors.get(p + "self_attn.sinks")
            if sk is not None:
                lw.sinks = sk.to(device=dev, dtype=torch.float32)
            if cfg.layer_is_moe(gi):
                from parallax_b200.models.moe import MoEWeights

                lw.moe = MoEWeights.from_hf(cfg, tensors, p + "mlp.", dev, dt)
                self._ep_finish(lw.moe)
            else:
                lw.w_gu = self._pack_gate_up(get(p + "mlp.gate_proj.weight"), get(p + "mlp.up_proj.weight"))
                lw.w_down = get(p + "mlp.down_proj.weight").contiguous()

    def _pack_gate_up(self, wg: torch.Tensor, wu: torch.Tensor) -> torch.Tensor:
        if self.dense_act_mode:
            return torch.cat([wg, wu], dim=0).contiguous()
        return ops.interleave_gate_up(wg, wu)

    # ------------------------------------------------------------------ online refit
    _LAYER_KEY = re.compile(r"(?:^|\.)layers\.(\d+)\.")
    _GLOBAL_KEYS = ("embed_tokens.weight", ".norm.weight", "lm_head.weight")

    @classmethod
    def _layer_of_key(cls, key: str) -> Optional[int]:
        m = cls._LAYER_KEY.search(key)
        return int(m.group(1)) if m else None

    @torch.no_grad()
    def reload_layers(self, tensors: dict[str, torch.Tensor], only: Optional[set] = None) -> int:
        """Refit by re-running this family's own loader on every local layer that ``tensors`` names, then
        moving the result into the live weights (copied in place wherever shape and dtype are unchanged, so
        pointers that kernels or the native executor hold stay valid). Works for every family, sharding and
        quantisation because it is the loader itself that builds the new layer: fused layouts, expert shards,
        tensor-parallel slices and fp8 blocks come out the way ``load_weights`` makes them. A layer must be
        complete in ``tensors`` (the reference's refit ships whole checkpoints:
        ``src/parallax/server/shard_loader.py:557-651``); an incomplete one raises ``ValueError`` before anything
        is changed. ``only`` restricts the reload to a set of global layer numbers. Returns the number of
        tensors used."""
        import copy

        by_layer: dict[int, int] = {}
        n_global = 0
        for key in tensors:
            gi = self._layer_of_key(key)
            if gi is not None:
                if self.start_layer <= gi < self.end_layer and (only is None or gi in only):
                    by_layer[gi] = by_layer.get(gi, 0) + 1
            elif only is None and key.endswith(self._GLOBAL_KEYS):
                n_global += 1
        built = []
        for gi in sorted(by_layer):
            shadow = copy.copy(self)
            shadow.start_layer, shadow.end_layer = gi, gi + 1
            shadow.is_first = shadow.is_last = False
            shadow.embed = shadow.norm_w = shadow.lm_head = None
            shadow.layers = [type(self.layers[gi - self.start_layer])()]
            shadow.kv_caches, shadow._native, shadow.lora = [], False, None
            self._prepare_shadow(shadow)
            try:
                shadow.load_weights(tensors)
            except KeyError as e:
                raise ValueError(f"refit of layer {gi} needs every tensor of that layer: {e}") from e
            built.append((gi, shadow))
        glob = None
        wants_embed = self.is_first or (self.is_last and self.cfg.tie_word_embeddings)
        if n_global and (wants_embed or self.is_last):
            glob = copy.copy(self)
            glob.start_layer = glob.end_layer = self.start_layer
            glob.layers, glob.kv_caches, glob._native, glob.lora = [], [], False, None
            glob.embed = glob.norm_w = glob.lm_head = None
            self._prepare_shadow(glob)
            try:
                glob.load_weights(tensors)
            except KeyError as e:
                raise ValueError(f"refit of the embedding / head needs all of their tensors: {e}") from e
        replaced = False
        for gi, shadow in built:
            replaced |= self._adopt_layer(gi - self.start_layer, shadow)
        if glob is not None:
            tied = self.embed is not None and self.lm_head is not None and self.embed.data_ptr() == self.lm_head.data_ptr()
            for name in ("embed", "norm_w", "lm_head"):
                new = getattr(glob, name)
                if new is None or (tied and name == "lm_head"):
                    continue
                val, rep = _adopt(getattr(self, name), new)
                setattr(self, name, val)
                replaced |= rep
            if tied:
                self.lm_head = self.embed
        if replaced and self._native:
            self._native = None            # rebuilt on the next step with the new pointers
        if self.routed_buf is not None:
            self._install_route_capture()
        return sum(by_layer.values()) + (n_global if glob is not None else 0)

    # ------------------------------------------------------------------ routed-experts record
    def enable_routed_capture(self, num_kv_slots: int) -> bool:
        """Record which experts every token was routed to, per KV slot (the slot a token's K/V is written to
        names the token for as long as its request lives, prefix-cache hits included): ``routed_buf[slot, j]``
        holds the top-k expert ids of this stage's j-th MoE layer. The reference exposes the same record for
        rollout replay in RL training behind ``--enable-return-routed-experts``
        (``src/parallax/server/executor/vllm_executor.py:480-584``). Returns False for a stage without MoE layers."""
        n_moe = sum(1 for lw in self.layers if getattr(lw, "moe", None) is not None)
        if n_moe == 0:
            return False
        self.routed_buf = torch.full((num_kv_slots + 1, n_moe, self.cfg.num_experts_per_tok), -1, dtype=torch.int16,
                                     device=self.device)
        self._install_route_capture()
        return True

    def _install_route_capture(self) -> None:
        j = 0
        for lw in self.layers:
            if getattr(lw, "moe", None) is not None:
                lw.moe.capture = (lambda ids, j=j: self._record_route(j, ids))
                j += 1

    def _record_route(self, j: int, ids: torch.Tensor) -> None:
        slots = self._route_slots
        if slots is not None and slots.shape[0] == ids.shape[0]:
            # rows without a KV slot (negative) are parked in the last row of the buffer, which no request reads
            self.routed_buf[torch.where(slots < 0, self.routed_buf.shape[0] - 1, slots), j] = ids.to(torch.int16)

    def routed_experts_of(self, slots: torch.Tensor) -> torch.Tensor:
        """``[len(slots), MoE layers, top-k]`` for the given KV slots (int64, on this device)."""
        return self.routed_buf[slots]

    def _prepare_shadow(self, shadow) -> None:
        """Hook for subclasses: reset per-stage loader state on the temporary stage that reloads one layer."""

    def _adopt_layer(self, li: int, shadow) -> bool:
        """Move layer 0 of ``shadow`` into local layer ``li``. True when some tensor had to be replaced."""
        _val, replaced = _adopt(self.layers[li], shadow.layers[0])
        return replaced

    @torch.no_grad()
    def update_weights(self, tensors: dict[str, torch.Tensor]) -> int:
        """Patch weights in place from HF-named tensors (online refit). Tensors of layers that
        this stage does not own are ignored. Returns the number of tensors applied. Dense layers take single
        tensors; a layer with experts is reloaded whole when any of its ``mlp.`` tensors is present."""
        cfg = self.cfg
        if self.dense_act_mode:
            return self.reload_layers(tensors)
        moe_layers = {lw.layer_idx for lw in self.layers if lw.moe is not None}
        reload = {gi for gi in moe_layers if any(k.startswith(f"model.layers.{gi}.mlp.") for k in tensors)}
        n_reloaded = self.reload_layers(tensors, only=reload) if reload else 0
        if reload:
            tensors = {k: t for k, t in tensors.items() if self._layer_of_key(k) not in reload}
        Hq, Hkv, D, I = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.intermediate_size
        by_layer = {lw.layer_idx: lw for lw in self.layers}
        n = 0

        def cp(dst, src):
            dst.copy_(src.to(device=dst.device, dtype=dst.dtype))

        for key, t in tensors.items():
            if key == "model.embed_tokens.weight" and self.embed is not None:
                cp(self.embed, t); n += 1
            elif key == "model.norm.weight" and self.norm_w is not None:
                cp(self.norm_w, t); n += 1
            elif key == "lm_head.weight" and self.lm_head is not None:
                cp(self.lm_head, t); n += 1
            elif key.startswith("model.layers."):
                parts = key.split(".")
                lw = by_layer.get(int(parts[2]))
                if lw is None:
                    continue
                name = ".".join(parts[3:])
                qkv_off = {"self_attn.q_proj": (0, Hq * D), "self_attn.k_proj": (Hq * D, Hkv * D),
                           "self_attn.v_proj": ((Hq + Hkv) * D, Hkv * D)}
                base, _, kind = name.rpartition(".")
                if base in qkv_off:
                    o, ln = qkv_off[base]
                    tgt = lw.w_qkv if kind == "weight" else lw.b_qkv
                    if tgt is not None:
                        cp(tgt[o:o + ln], t); n += 1
                elif name == "self_attn.o_proj.weight":
                    cp(lw.w_o, t); n += 1
                elif name in ("mlp.gate_proj.weight", "mlp.up_proj.weight") and lw.w_gu is not None:
                    view = lw.w_gu.view(I // 64, 2, 64, -1)
                    cp(view[:, 0 if "gate" in name else 1], t.reshape(I // 64, 64, -1)); n += 1
                elif name == "mlp.down_proj.weight" and lw.w_down is not None:
                    cp(lw.w_down, t); n += 1
                else:
                    simple = {"input_layernorm.weight": "ln1", "post_attention_layernorm.weight": "ln2",
                              "self_attn.q_norm.weight": "q_norm", "self_attn.k_norm.weight": "k_norm"}.get(name)
                    if simple and getattr(lw, simple) is not None:
                        cp(getattr(lw, simple), t); n += 1
        return n + n_reloaded

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
            for s in LayerWeights.__slots__:
                v = getattr(lw, s)
                if isinstance(v, torch.Tensor):
                    add(v)
                elif v is not None and hasattr(v, "tensors"):
                    for t in v.tensors():
                        add(t)
        return total

    # ------------------------------------------------------------------ forward
    def attach_kv(self, kv_caches: list) -> None:
        assert len(kv_caches) == len(self.layers)
        self.kv_caches = kv_caches

    def embed_tokens(self, fb: ForwardBatch) -> torch.Tensor:
        return ops.gather_rows(self.embed, fb.input_ids)

    def _attention(self, lw: LayerWeights, li: int, xn: torch.Tensor, fb: ForwardBatch) -> torch.Tensor:
        cfg = self.cfg
        Hq, Hkv, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        T = xn.shape[0]
        qkv = ops.linear(xn, lw.w_qkv, bias=lw.b_qkv)
        rows_lora = fb.extras.get("lora_ids") if self.lora is not None else None
        if rows_lora is not None:
            qkv = self.lora.apply("qkv", li, xn, qkv, rows_lora, fb.extras.get("lora_plan"))
        kc, vc = self.kv_caches[li]
        kvs = getattr(self.kv_caches[li], "kv_scale", (1.0, 1.0))
        qn, kn = lw.q_norm, lw.k_norm
        if cfg.qk_norm_full and qn is not None:
            # norm over the whole projection, in place on the column slices of the packed activation
            ops.rmsnorm(qkv[:, :Hq * D], qn, cfg.rms_norm_eps, w_offset=self.norm_offset, out=qkv[:, :Hq * D])
            ops.rmsnorm(qkv[:, Hq * D:(Hq + Hkv) * D], kn, cfg.rms_norm_eps, w_offset=self.norm_offset,
                        out=qkv[:, Hq * D:(Hq + Hkv) * D])
            qn = kn = None
        ops.qk_norm_rope_cache(qkv, qn, kn, self.cos_sin, fb.positions, fb.slot_mapping,
                               kc, vc, Hq, Hkv, D, cfg.rot_dim, cfg.rms_norm_eps, self.norm_offset, kv_scale=kvs)
        q = qkv.view(T, Hq + 2 * Hkv, D)[:, :Hq]
        attn = torch.empty((T, Hq, D), dtype=qkv.dtype, device=qkv.device)
        Tp = fb.num_prefill_tokens
        if Tp:
            ops.attn_prefill(q[:Tp], kc, vc, fb.p_block_tables, fb.p_cu_q, fb.p_ctx_lens, fb.p_max_q,
                             self.scale, window=lw.window, sinks=lw.sinks, out=attn[:Tp], kv_scale=kvs)
        if fb.num_decode:
            ops.attn_decode(q[Tp:], kc, vc, fb.d_block_tables, fb.d_ctx_lens, self.scale,
                            window=lw.window, sinks=lw.sinks, max_ctx=fb.d_max_ctx, out=attn[Tp:], kv_scale=kvs)
        if lw.w_g is not None:      # head-wise gate: every head's output times sigmoid of that head's gate logit
            return ops.gate_mul_grouped(attn.view(T, Hq * D), ops.linear(xn, lw.w_g), D)
        return attn.view(T, Hq * D)

    def _mlp(self, lw: LayerWeights, xn: torch.Tensor, h: torch.Tensor, li: int = 0, fb=None) -> torch.Tensor:
        if lw.moe is not None:
            return lw.moe.forward(xn, h)
        if self.dense_act_mode:
            act = ops.act_mul(ops.linear(xn, lw.w_gu), self.dense_act_mode, self.dense_limit)
        else:
            act = ops.linear(xn, lw.w_gu, epi=ops.EPI_SILU_MUL)
        out = ops.linear(act, lw.w_down, residual=h)
        rows_lora = fb.extras.get("lora_ids") if (self.lora is not None and fb is not None) else None
        if rows_lora is not None:
            out = self.lora.apply("down", li, act, out, rows_lora, fb.extras.get("lora_plan"))
        return out

    def forward_layers(self, h: torch.Tensor, fb: ForwardBatch) -> torch.Tensor:
        if self._native is None and type(self).forward_layers is DecoderStage.forward_layers \
                and type(self)._attention is DecoderStage._attention:
            from parallax_b200.engine.native_stage import NativeDenseStage

            # dense GQA stage on a GPU: all layers of a step run behind one call into the library
            import os

            self._native = NativeDenseStage(self) if NativeDenseStage.supported(self) \
                and not os.environ.get("PXL_NO_NATIVE_STAGE") else False
        rows_lora = fb.extras.get("lora_ids") if self.lora is not None else None
        if rows_lora is not None and h.is_cuda and "lora_plan" not in fb.extras:
            from parallax_b200.ops import cuda as _cu

            # which rows go to which adapter: the same grouping serves every projection of every layer
            fb.extras["lora_plan"] = _cu.moe_align(rows_lora.view(-1, 1), self.lora.slots)
        if self._native and rows_lora is None:
            out = self._native.forward(h.contiguous(), fb)
            # the result lives in the executor's workspace: hand out a copy when it leaves the stage
            return out if self.is_last else out.clone()
        eps = self.cfg.rms_norm_eps
        for li, lw in enumerate(self.layers):
            xn = ops.rmsnorm(h, lw.ln1, eps, w_offset=self.norm_offset)
            a = self._attention(lw, li, xn, fb)
            h = ops.linear(a, lw.w_o, bias=lw.b_o, residual=h)
            if rows_lora is not None:
                h = self.lora.apply("o", li, a, h, rows_lora, fb.extras.get("lora_plan"))
            xn = ops.rmsnorm(h, lw.ln2, eps, w_offset=self.norm_offset)
            h = self._mlp(lw, xn, h, li, fb)
        return h

    def logits(self, h: torch.Tensor, fb: ForwardBatch) -> torch.Tensor:
        rows = ops.gather_rows(h, fb.logit_rows) if fb.num_logits != h.shape[0] else h
        hn = ops.rmsnorm(rows, self.norm_w, self.cfg.rms_norm_eps, w_offset=self.norm_offset)
        return ops.linear(hn, self.lm_head)

    def forward(self, fb: ForwardBatch, hidden: Optional[torch.Tensor] = None) -> torch.Tensor:
        """First stage: ``hidden`` is ignored and tokens are embedded. Returns hidden states
        ``[T, H]`` (non-last stage) or logits ``[num_logits, V]`` (last stage)."""
        if fb.num_tokens == 0:
            # expert parallelism with data-parallel attention: no token on this rank in this step
            self.ep_idle_step()
            n_out = self.cfg.vocab_size if self.is_last else self.cfg.hidden_size
            return torch.empty((0, n_out), dtype=self.dtype, device=self.device)
        h = self.embed_tokens(fb) if self.is_first else hidden
        if self.routed_buf is not None:
            self._route_slots = fb.slot_mapping
        h = self.forward_layers(h, fb)
        if self.is_last:
            return self.logits(h, fb)
        return h
