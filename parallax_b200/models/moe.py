"""Mixture-of-experts FFN block (router + stacked SwiGLU experts + optional shared experts).

Covers the routing variants of the supported families: softmax top-k with renormalisation
(Qwen3-MoE, GLM4-MoE, MiniMax-M2, GPT-OSS style) and sigmoid + correction bias with
group-limited selection and a routed scaling factor (DeepSeek-V3 / Kimi-K2, MiniMax-M3).
The reference reaches these through mlx-lm switch layers (``src/parallax/models/qwen3_moe.py``)
or its own ``minimax_m3.py:155-277``; here routing, permutation, the grouped tcgen05 GEMMs and
the weighted combine are the kernels of ``csrc/moe.cu`` / ``csrc/gemm_tcgen05.cu``.

Expert weights are stacked: ``w1 [E*2I, H]`` (gate/up rows interleaved in groups of 64 per
expert) and ``w2 [E*H, I]``. With expert parallelism a rank holds experts ``[e_lo, e_hi)``.
"""

from __future__ import annotations

from typing import Callable, Optional

import torch

from parallax_b200 import ops
from parallax_b200.models.config import ModelConfig


class MoEWeights:
    def __init__(self, cfg: ModelConfig):
        self.cfg = cfg
        self.router: Optional[torch.Tensor] = None      # [E, H]
        self.e_bias: Optional[torch.Tensor] = None      # [E] fp32 (noaux_tc correction bias)
        self.w1: Optional[torch.Tensor] = None          # [E*2I, H]
        self.w2: Optional[torch.Tensor] = None          # [E*H, I]
        self.shared_gu: Optional[torch.Tensor] = None   # [2*Is, H] interleaved
        self.shared_down: Optional[torch.Tensor] = None  # [H, Is]
        self.shared_gate: Optional[torch.Tensor] = None  # [1, H] sigmoid gate on the shared expert (Qwen2-MoE style)
        self.fp8: Optional[dict] = None                 # block-scaled e4m3 copies: name -> (q, scales per 64 rows)
        self.router_bias: Optional[torch.Tensor] = None  # [E] (GPT-OSS)
        self.b1: Optional[torch.Tensor] = None          # [E*2I] expert biases of the first projection
        self.b2: Optional[torch.Tensor] = None          # [E*H]
        # 0: SwiGLU fused into the GEMM epilogue (w1 interleaved); 1: clipped swigluoai (w1 = [gate | up] per expert)
        self.act_mode = 1 if (cfg.swiglu_limit or cfg.hidden_act == "swigluoai") else 0
        self.limit = float(cfg.swiglu_limit or 7.0)
        self.num_experts = cfg.num_experts
        self.top_k = cfg.num_experts_per_tok
        self.mode = 1 if cfg.scoring_func == "sigmoid" else 0

    def tensors(self):
        ts = [t for t in (self.router, self.e_bias, self.w1, self.w2, self.shared_gu, self.shared_down,
                          self.shared_gate, self.router_bias, self.b1, self.b2) if t is not None]
        for q, s in (self.fp8 or {}).values():
            ts += [q, s]
        return ts

    def shard_experts(self, rank: int, ep: int) -> int:
        """Keep only this rank's ``E / ep`` consecutive experts (router and shared expert stay
        replicated). Returns the number of local experts."""
        E = self.num_experts
        if E % ep:
            raise ValueError("the number of experts must divide by the expert-parallel size")
        epr = E // ep
        n1, n2 = self.w1.shape[0] // E, self.w2.shape[0] // E
        self.w1 = self.w1[rank * epr * n1:(rank + 1) * epr * n1].contiguous()
        self.w2 = self.w2[rank * epr * n2:(rank + 1) * epr * n2].contiguous()
        self.experts_per_rank = epr
        return epr

    def shared_base(self, xn: torch.Tensor, h: torch.Tensor) -> torch.Tensor:
        """``h`` plus the shared expert's output (``h`` itself when the model has none)."""
        if self.shared_gu is None:
            return h
        act = ops.linear(xn, self.shared_gu, epi=ops.EPI_SILU_MUL)
        if self.shared_gate is None:
            return ops.linear(act, self.shared_down, residual=h)
        gate = torch.sigmoid(xn.float() @ self.shared_gate.float().t()).to(h.dtype)
        return h + gate * ops.linear(act, self.shared_down)

    def quantize_fp8(self) -> None:
        """Replace the expert (and shared-expert) matrices by e4m3 + scales per 64 x 128 block."""
        from parallax_b200.loader.quant import quantize_fp8_block

        self.fp8 = {}
        for name in ("w1", "w2", "shared_gu", "shared_down"):
            w = getattr(self, name)
            if w is not None:
                self.fp8[name] = quantize_fp8_block(w, (64, 128))
                setattr(self, name, None)

    # ------------------------------------------------------------------ construction
    @classmethod
    def random(cls, cfg: ModelConfig, device, dtype, rnd: Callable) -> "MoEWeights":
        m = cls(cfg)
        E, H, I = cfg.num_experts, cfg.hidden_size, cfg.moe_intermediate_size
        m.router = rnd(E, H, k=0)
        if cfg.moe_router_bias:
            m.e_bias = torch.zeros(E, device=device, dtype=torch.float32)
        g = rnd(E * I, H, k=1).view(E, I, H)
        u = rnd(E * I, H, k=2).view(E, I, H)
        if m.act_mode == 0:
            m.w1 = torch.stack([ops.interleave_gate_up(g[e], u[e]) for e in range(E)]).view(E * 2 * I, H).contiguous()
        else:
            m.w1 = torch.cat([g, u], dim=1).reshape(E * 2 * I, H).contiguous()
            m.b1, m.b2 = rnd(E * 2 * I, k=7), rnd(E * H, k=8)
            m.router_bias = rnd(E, k=9)
        m.w2 = rnd(E * H, I, k=3)
        Is = cfg.shared_expert_intermediate_size or (cfg.n_shared_experts * I)
        if Is:
            m.shared_gu = ops.interleave_gate_up(rnd(Is, H, k=4), rnd(Is, H, k=5))
            m.shared_down = rnd(H, Is, k=6)
        return m

    @classmethod
    def from_hf(cls, cfg: ModelConfig, tensors: dict, prefix: str, device, dtype) -> "MoEWeights":
        m = cls(cfg)
        E = cfg.num_experts

        def get(name, required=True, dt=dtype):
            t = tensors.get(prefix + name)
            if t is None:
                if required:
                    raise KeyError(f"missing weight {prefix + name}")
                return None
            return t.to(device=device, dtype=dt)

        if prefix + "experts.gate_up_proj_blocks" in tensors:
            # GPT-OSS as published: MXFP4 expert matrices, expanded to bf16 here. The rows of gate_up
            # alternate gate / up; [E, rows, K] is already the [N, K] layout of the grouped GEMM.
            from parallax_b200.loader.quant import dequant_mxfp4

            def expand(name):
                return dequant_mxfp4(tensors[prefix + name + "_blocks"], tensors[prefix + name + "_scales"],
                                     dtype).to(device)

            m.router = get("router.weight").contiguous()
            m.router_bias = get("router.bias", required=False)
            gu = expand("experts.gate_up_proj")                                   # [E, 2I, H]
            m.w1 = torch.cat([gu[:, 0::2], gu[:, 1::2]], dim=1).reshape(E * gu.shape[1], -1).contiguous()
            del gu
            b = get("experts.gate_up_proj_bias", required=False)
            if b is not None:
                m.b1 = torch.cat([b[:, 0::2], b[:, 1::2]], dim=1).reshape(-1).contiguous()
            dn = expand("experts.down_proj")                                      # [E, H, I]
            m.w2 = dn.reshape(E * dn.shape[1], -1).contiguous()
            b2 = get("experts.down_proj_bias", required=False)
            m.b2 = None if b2 is None else b2.reshape(-1).contiguous()
            m.act_mode = 1
            return m
        fused = get("experts.gate_up_proj", required=False)
        if fused is not None and get("router.weight", required=False) is not None:
            # GPT-OSS layout: gate_up_proj [E, H, 2I] with gate / up in even / odd columns, expert biases
            m.router = get("router.weight").contiguous()
            m.router_bias = get("router.bias", required=False)
            I2 = fused.shape[2]
            gate, up = fused[:, :, 0::2], fused[:, :, 1::2]                       # [E, H, I]
            m.w1 = torch.cat([gate.transpose(1, 2), up.transpose(1, 2)], dim=1).reshape(E * I2, -1).contiguous()
            b = get("experts.gate_up_proj_bias", required=False)
            if b is not None:
                m.b1 = torch.cat([b[:, 0::2], b[:, 1::2]], dim=1).reshape(-1).contiguous()
            m.w2 = get("experts.down_proj").transpose(1, 2).reshape(E * fused.shape[1], -1).contiguous()   # [E*H, I]
            b2 = get("experts.down_proj_bias", required=False)
            m.b2 = None if b2 is None else b2.reshape(-1).contiguous()
            m.act_mode = 1
            return m
        m.router = get("gate.weight").contiguous()
        m.e_bias = get("gate.e_score_correction_bias", required=False, dt=torch.float32)
        if m.e_bias is None:      # MiniMax-M2 keeps the selection bias one level up
            m.e_bias = get("e_score_correction_bias", required=False, dt=torch.float32)
        w1, w2 = [], []
        for e in range(E):
            g_w, u_w = get(f"experts.{e}.gate_proj.weight"), get(f"experts.{e}.up_proj.weight")
            w1.append(ops.interleave_gate_up(g_w, u_w) if m.act_mode == 0 else torch.cat([g_w, u_w], dim=0))
            w2.append(get(f"experts.{e}.down_proj.weight"))
        m.w1 = torch.cat(w1, dim=0).contiguous()
        m.w2 = torch.cat(w2, dim=0).contiguous()
        for shared in ("shared_experts", "shared_expert"):
            g = get(f"{shared}.gate_proj.weight", required=False)
            if g is not None:
                m.shared_gu = ops.interleave_gate_up(g, get(f"{shared}.up_proj.weight"))
                m.shared_down = get(f"{shared}.down_proj.weight").contiguous()
        m.shared_gate = get("shared_expert_gate.weight", required=False)
        return m

    # ------------------------------------------------------------------ forward
    def route(self, xn: torch.Tensor):
        cfg = self.cfg
        logits = ops.linear(xn, self.router, bias=self.router_bias, epi=ops.EPI_F32)
        return ops.moe_route(logits, self.e_bias, self.top_k, self.mode, cfg.norm_topk_prob, cfg.n_group,
                             cfg.topk_group, cfg.routed_scaling_factor)

    def forward(self, xn: torch.Tensor, h: torch.Tensor) -> torch.Tensor:
        """Returns ``h + MoE(xn)`` (the residual add is fused into the combine / shared-expert GEMM)."""
        ids, w = self.route(xn)
        base = h
        if self.fp8 is not None:
            f = self.fp8
            if "shared_gu" in f:
                act = ops.linear_fp8(xn, *f["shared_gu"], epi=ops.EPI_SILU_MUL)
                base = ops.linear_fp8(act, *f["shared_down"], residual=h)
            return ops.moe_ffn_fp8(xn, ids, w, *f["w1"], *f["w2"], self.num_experts, base=base)
        if self.shared_gu is not None:
            act = ops.linear(xn, self.shared_gu, epi=ops.EPI_SILU_MUL)
            if self.shared_gate is None:
                base = ops.linear(act, self.shared_down, residual=h)
            else:
                gate = torch.sigmoid(xn.float() @ self.shared_gate.float().t()).to(h.dtype)  # [T, 1]: too thin for a tile
                base = h + gate * ops.linear(act, self.shared_down)
        if self.act_mode:
            return ops.moe_ffn(xn, ids, w, self.w1, self.w2, self.num_experts, base=base, act_mode=self.act_mode,
                               limit=self.limit, b1=self.b1, b2=self.b2)
        return ops.moe_ffn(xn, ids, w, self.w1, self.w2, self.num_experts, base=base)
