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


class ExpertParallelMixin:
    """Stage-side switch for expert parallelism with data-parallel attention: every rank of the group
    keeps the whole attention stack and ``E / ep`` experts of each MoE layer, and runs its own token rows."""

    ep_rank, ep_size, ep_comm, ep_local_init = 0, 1, None, False

    def set_expert_parallel(self, rank: int, size: int, comm, local_init: bool = False) -> None:
        """Call before the weights are created. ``local_init``: random initialisation generates only this
        rank's experts (for models whose full expert set does not fit one device)."""
        self.ep_rank, self.ep_size, self.ep_comm, self.ep_local_init = rank, size, comm, local_init

    def _ep_shard_arg(self):
        return (self.ep_rank, self.ep_size) if self.ep_size > 1 and self.ep_local_init else None

    def _ep_finish(self, moe: "MoEWeights") -> None:
        if self.ep_size > 1:
            moe.shard_experts(self.ep_rank, self.ep_size)
            moe.ep = self.ep_comm

    def ep_idle_step(self) -> None:
        """A step in which this rank has no token: it still takes part in every MoE layer's exchange."""
        for lw in self.layers:
            if getattr(lw, "moe", None) is not None and lw.moe.ep is not None:
                lw.moe.idle(self.device, self.dtype)


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
        self.experts_per_rank = cfg.num_experts
        # expert parallelism with data-parallel attention: set to the group's exchange object
        # (parallax_b200.parallel.ep.EPComm); the local expert weights then hold `experts_per_rank` experts
        self.ep = None
        self.capture = None        # callable(ids [T, k]) when the engine records the routed experts

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
        if self.experts_per_rank == epr:      # already built with this rank's experts only
            return epr

        def rows(t):
            n = t.shape[0] // E
            return t[rank * epr * n:(rank + 1) * epr * n].contiguous()

        for name in ("w1", "w2", "b1", "b2"):
            t = getattr(self, name)
            if t is not None:
                setattr(self, name, rows(t))
        if self.fp8 is not None:
            for name in ("w1", "w2"):
                q, sc = self.fp8[name]
                self.fp8[name] = (rows(q), rows(sc))
        self.experts_per_rank = epr
        return epr

    def shared_base(self, xn: torch.Tensor, h: torch.Tensor) -> torch.Tensor:
        """``h`` plus the shared expert's output (``h`` itself when the model has none)."""
        if self.shared_gu is None:
            return h
        act = ops.linear(xn, self.shared_gu, epi=ops.EPI_SILU_MUL)
        if self.shared_gate is None:
            return ops.linear(act, self.shared_down, residual=h)
        y = ops.linear(act, self.shared_down)
        return ops.gate_mul_grouped(y, ops.row_dot(xn, self.shared_gate), y.shape[1], residual=h)

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
    def random(cls, cfg: ModelConfig, device, dtype, rnd: Callable, expert_shard=None) -> "MoEWeights":
        """``expert_shard=(rank, ep)``: generate only that rank's experts (models whose full expert set
        does not fit one device). The values then differ from a slice of the unsharded generation."""
        m = cls(cfg)
        E_all, H, I = cfg.num_experts, cfg.hidden_size, cfg.moe_intermediate_size
        m.router = rnd(E_all, H, k=0)
        if cfg.moe_router_bias:
            m.e_bias = torch.zeros(E_all, device=device, dtype=torch.float32)
        E = E_all
        shared_rnd = rnd          # router, router bias and shared expert are replicated: same on every rank
        if expert_shard is not None:
            r, ep = expert_shard
            E = E_all // ep
            m.experts_per_rank = E
            rnd = lambda *sh, k: shared_rnd(*sh, k=k + 100 * (r + 1))  # noqa: E731
        g = rnd(E * I, H, k=1).view(E, I, H)
        u = rnd(E * I, H, k=2).view(E, I, H)
        if m.act_mode == 0:
            m.w1 = torch.stack([ops.interleave_gate_up(g[e], u[e]) for e in range(E)]).view(E * 2 * I, H).contiguous()
        else:
            m.w1 = torch.cat([g, u], dim=1).reshape(E * 2 * I, H).contiguous()
            m.b1, m.b2 = rnd(E * 2 * I, k=7), rnd(E * H, k=8)
            m.router_bias = shared_rnd(E_all, k=9)
        m.w2 = rnd(E * H, I, k=3)
        Is = cfg.shared_expert_intermediate_size or (cfg.n_shared_experts * I)
        if Is:
            m.shared_gu = ops.interleave_gate_up(shared_rnd(Is, H, k=4), shared_rnd(Is, H, k=5))
            m.shared_down = shared_rnd(H, Is, k=6)
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
    def idle(self, device, dtype) -> None:
        H, k = self.cfg.hidden_size, self.top_k
        xn = torch.empty((0, H), dtype=dtype, device=device)
        ids = torch.empty((0, k), dtype=torch.int32, device=device)
        w = torch.empty((0, k), dtype=torch.float32, device=device)
        self.ep.moe_ffn(self, xn, ids, w, base=None)

    def route(self, xn: torch.Tensor):
        cfg = self.cfg
        logits = ops.linear(xn, self.router, bias=self.router_bias, epi=ops.EPI_F32)
        ids, w = ops.moe_route(logits, self.e_bias, self.top_k, self.mode, cfg.norm_topk_prob, cfg.n_group,
                               cfg.topk_group, cfg.routed_scaling_factor)
        if self.capture is not None:
            self.capture(ids)          # routed-experts record for rollout replay (see DecoderStage.enable_routed_capture)
        return ids, w

    def forward(self, xn: torch.Tensor, h: torch.Tensor) -> torch.Tensor:
        """Returns ``h + MoE(xn)`` (the residual add is fused into the combine / shared-expert GEMM)."""
        ids, w = self.route(xn)
        base = h
        if self.fp8 is not None:
            f = self.fp8
            if "shared_gu" in f:
                act = ops.linear_fp8(xn, *f["shared_gu"], epi=ops.EPI_SILU_MUL)
                base = ops.linear_fp8(act, *f["shared_down"], residual=h)
            if self.ep is not None:
                return self.ep.moe_ffn(self, xn, ids, w, base=base)
            return ops.moe_ffn_fp8(xn, ids, w, *f["w1"], *f["w2"], self.num_experts, base=base)
        if self.shared_gu is not None:
            act = ops.linear(xn, self.shared_gu, epi=ops.EPI_SILU_MUL)
            if self.shared_gate is None:
                base = ops.linear(act, self.shared_down, residual=h)
            else:
                # scalar gate per token: a [T, H] x [H] row dot (too thin for a GEMM tile), applied with the residual
                y = ops.linear(act, self.shared_down)
                base = ops.gate_mul_grouped(y, ops.row_dot(xn, self.shared_gate), y.shape[1], residual=h)
        if self.ep is not None:
            return self.ep.moe_ffn(self, xn, ids, w, base=base)
        if self.act_mode:
            return ops.moe_ffn(xn, ids, w, self.w1, self.w2, self.num_experts, base=base, act_mode=self.act_mode,
                               limit=self.limit, b1=self.b1, b2=self.b2)
        return ops.moe_ffn(xn, ids, w, self.w1, self.w2, self.num_experts, base=base)
