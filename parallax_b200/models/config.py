"""Model configuration: a normalised view of a HuggingFace ``config.json``.

The normalisation mirrors what the reference does before building a shard: nested
``text_config`` of VLM-style checkpoints is flattened, sparse-attention fields are mapped to
common names and the per-layer attention type is derived
(``src/parallax/utils/utils.py:310-397,430-483``).
"""

from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Optional

# layer kinds (same vocabulary as the reference's ``utils/layer_types.py:5-20``)
ATTENTION = "attention"
MLA_ATTENTION = "mla_attention"
DSA_ATTENTION = "dsa_attention"
MSA_ATTENTION = "msa_attention"
LINEAR = "linear"


@dataclass
class ModelConfig:
    architecture: str = "Qwen3ForCausalLM"
    model_type: str = "qwen3"
    hidden_size: int = 1024
    num_hidden_layers: int = 28
    num_attention_heads: int = 16
    num_key_value_heads: int = 8
    head_dim: int = 128
    intermediate_size: int = 3072
    vocab_size: int = 151936
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e6
    rope_scaling: Optional[dict] = None
    partial_rotary_factor: float = 1.0
    max_position_embeddings: int = 40960
    tie_word_embeddings: bool = False
    attention_bias: bool = False
    qk_norm: bool = False
    qk_norm_full: bool = False       # norm over the whole projection (MiniMax-M2 style)
    hidden_act: str = "silu"
    sliding_window: int = 0
    layer_types: list = field(default_factory=list)  # per layer: "full_attention"/"sliding_attention"/"linear_attention"
    attention_sinks: bool = False
    attn_output_gate: bool = False
    # MoE
    num_experts: int = 0
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0
    norm_topk_prob: bool = True
    n_shared_experts: int = 0
    shared_expert_intermediate_size: int = 0
    first_k_dense_replace: int = 0
    moe_layer_freq: int = 1
    mlp_only_layers: list = field(default_factory=list)
    scoring_func: str = "softmax"
    routed_scaling_factor: float = 1.0
    n_group: int = 1
    topk_group: int = 1
    moe_router_bias: bool = False       # e_score_correction_bias (noaux_tc)
    swiglu_limit: float = 0.0
    # MLA
    q_lora_rank: int = 0
    kv_lora_rank: int = 0
    qk_nope_head_dim: int = 0
    qk_rope_head_dim: int = 0
    v_head_dim: int = 0
    # DSA (DeepSeek-V3.2 lightning indexer)
    index_n_heads: int = 0
    index_head_dim: int = 0
    index_topk: int = 0
    # linear attention (gated delta net)
    linear_num_key_heads: int = 0
    linear_num_value_heads: int = 0
    linear_key_head_dim: int = 0
    linear_value_head_dim: int = 0
    linear_conv_kernel_dim: int = 0
    full_attention_interval: int = 0
    # quantisation
    quant_method: str = ""
    weight_block_size: Optional[list] = None
    dtype: str = "bfloat16"
    raw: dict = field(default_factory=dict, repr=False)

    # ------------------------------------------------------------------ derived
    @property
    def is_moe(self) -> bool:
        return self.num_experts > 0

    @property
    def is_mla(self) -> bool:
        return self.kv_lora_rank > 0

    @property
    def rot_dim(self) -> int:
        base = self.qk_rope_head_dim if self.is_mla else self.head_dim
        r = int(base * self.partial_rotary_factor)
        return r - (r % 2)

    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    def layer_is_moe(self, layer_idx: int) -> bool:
        if not self.is_moe:
            return False
        if layer_idx in self.mlp_only_layers:
            return False
        if layer_idx < self.first_k_dense_replace:
            return False
        return (layer_idx + 1) % max(1, self.moe_layer_freq) == 0 if self.moe_layer_freq > 1 else True

    def layer_kind(self, layer_idx: int) -> str:
        if self.layer_types and layer_idx < len(self.layer_types):
            if self.layer_types[layer_idx] == "linear_attention":
                return LINEAR
        elif self.full_attention_interval and (layer_idx + 1) % self.full_attention_interval != 0:
            return LINEAR
        if self.is_mla:
            return DSA_ATTENTION if self.index_topk > 0 else MLA_ATTENTION
        if self.raw.get("index_topk_blocks"):
            freq = (self.raw.get("sparse_attention_config") or {}).get("sparse_attention_freq")
            if isinstance(freq, list) and not (layer_idx < len(freq) and freq[layer_idx]):
                return ATTENTION
            return MSA_ATTENTION
        return ATTENTION

    @property
    def has_linear_layers(self) -> bool:
        return any(self.layer_kind(i) == LINEAR for i in range(self.num_hidden_layers))

    def layer_window(self, layer_idx: int) -> int:
        if not self.sliding_window:
            return 0
        if self.layer_types and layer_idx < len(self.layer_types):
            return self.sliding_window if self.layer_types[layer_idx] == "sliding_attention" else 0
        return self.sliding_window

    def kv_bytes_per_token_per_layer(self, elem_bytes: int = 2) -> int:
        if self.is_mla:
            return (self.kv_lora_rank + self.qk_rope_head_dim) * elem_bytes
        return 2 * self.num_key_value_heads * self.head_dim * elem_bytes


def normalize_hf_config(cfg: dict) -> dict:
    """Flatten VLM-style configs so that text-model fields sit at the top level."""
    text = cfg.get("text_config")
    if isinstance(text, dict) and cfg.get("model_type") in {"qwen3_5", "qwen3_5_moe", "minimax_m3_vl"}:
        out = {**cfg, **text}
        out["architectures"] = cfg.get("architectures") or text.get("architectures")
        out["model_type"] = "minimax_m3" if cfg["model_type"] == "minimax_m3_vl" else cfg["model_type"]
        out["tie_word_embeddings"] = text.get("tie_word_embeddings", cfg.get("tie_word_embeddings", False))
        sparse = out.get("sparse_attention_config")
        if isinstance(sparse, dict):
            out.setdefault("index_head_dim", sparse.get("sparse_index_dim"))
            out.setdefault("index_block_size", sparse.get("sparse_block_size"))
            out.setdefault("index_topk_blocks", sparse.get("sparse_topk_blocks"))
            out.setdefault("index_local_blocks", sparse.get("sparse_local_block"))
        if out.get("moe_intermediate_size") is None and out.get("intermediate_size") is not None:
            out["moe_intermediate_size"] = out["intermediate_size"]
        return out
    return cfg


def config_from_hf(cfg: dict) -> ModelConfig:
    cfg = normalize_hf_config(cfg)
    arch = (cfg.get("architectures") or ["Qwen3ForCausalLM"])[0]
    mt = cfg.get("model_type", "")
    nh = cfg.get("num_attention_heads", 16)
    hidden = cfg.get("hidden_size", 1024)
    head_dim = cfg.get("head_dim") or hidden // nh
    q = cfg.get("quantization_config") or cfg.get("quantization") or {}
    rope_scaling = cfg.get("rope_scaling") or cfg.get("rope_parameters")
    rope_theta = cfg.get("rope_theta")
    if rope_theta is None and isinstance(rope_scaling, dict):
        rope_theta = rope_scaling.get("rope_theta")
    mc = ModelConfig(
        architecture=arch,
        model_type=mt,
        hidden_size=hidden,
        num_hidden_layers=cfg.get("num_hidden_layers", 1),
        num_attention_heads=nh,
        num_key_value_heads=cfg.get("num_key_value_heads") or nh,
        head_dim=head_dim,
        intermediate_size=cfg.get("intermediate_size", 4 * hidden),
        vocab_size=cfg.get("vocab_size", 32000),
        rms_norm_eps=cfg.get("rms_norm_eps", 1e-6),
        rope_theta=float(rope_theta or 10000.0),
        rope_scaling=rope_scaling if isinstance(rope_scaling, dict) else None,
        partial_rotary_factor=float(cfg.get("partial_rotary_factor")
                                    or (rope_scaling or {}).get("partial_rotary_factor")
                                    or (cfg["rotary_dim"] / head_dim if cfg.get("rotary_dim") else 1.0)),
        max_position_embeddings=cfg.get("max_position_embeddings", 32768),
        tie_word_embeddings=bool(cfg.get("tie_word_embeddings", False)),
        attention_bias=bool(cfg.get("attention_bias", cfg.get("qkv_bias", mt == "qwen2"))),
        qk_norm=bool(cfg.get("use_qk_norm", mt in {"qwen3", "qwen3_moe", "qwen3_next", "qwen3_5", "qwen3_5_moe"})),
        qk_norm_full=mt in {"minimax", "minimax_m2"},
        hidden_act=cfg.get("hidden_act", "silu"),
        sliding_window=int(cfg.get("sliding_window") or 0) if cfg.get("use_sliding_window", True) else 0,
        layer_types=list(cfg.get("layer_types") or []),
        attention_sinks=mt == "gpt_oss",
        attn_output_gate=bool(cfg.get("attn_output_gate", mt in {"qwen3_next", "qwen3_5", "qwen3_5_moe"})),
        num_experts=cfg.get("num_experts") or cfg.get("n_routed_experts") or cfg.get("num_local_experts") or 0,
        num_experts_per_tok=cfg.get("num_experts_per_tok") or cfg.get("experts_per_token") or 0,
        moe_intermediate_size=cfg.get("moe_intermediate_size") or 0,
        norm_topk_prob=bool(cfg.get("norm_topk_prob", True)),
        n_shared_experts=cfg.get("n_shared_experts") or 0,
        shared_expert_intermediate_size=cfg.get("shared_expert_intermediate_size") or 0,
        first_k_dense_replace=cfg.get("first_k_dense_replace") or 0,
        moe_layer_freq=cfg.get("moe_layer_freq") or cfg.get("decoder_sparse_step") or 1,
        mlp_only_layers=list(cfg.get("mlp_only_layers") or []),
        scoring_func=cfg.get("scoring_func") or ("sigmoid" if mt in {"minimax_m2", "minimax_m3", "glm4_moe", "deepseek_v3",
                                                                       "deepseek_v32", "kimi_k2"} else "softmax"),
        routed_scaling_factor=float(cfg.get("routed_scaling_factor", 1.0)),
        n_group=cfg.get("n_group") or 1,
        topk_group=cfg.get("topk_group") or 1,
        moe_router_bias=cfg.get("topk_method") == "noaux_tc" or bool(cfg.get("use_routing_bias", False))
        or mt in {"minimax_m2", "minimax_m3", "glm4_moe"},
        swiglu_limit=float(cfg.get("swiglu_limit") or (7.0 if mt == "gpt_oss" else 0.0)),
        q_lora_rank=cfg.get("q_lora_rank") or 0,
        kv_lora_rank=cfg.get("kv_lora_rank") or 0,
        qk_nope_head_dim=cfg.get("qk_nope_head_dim") or 0,
        qk_rope_head_dim=cfg.get("qk_rope_head_dim") or 0,
        v_head_dim=cfg.get("v_head_dim") or 0,
        index_n_heads=cfg.get("index_n_heads") or 0,
        index_head_dim=cfg.get("index_head_dim") or 0,
        index_topk=cfg.get("index_topk") or 0,
        linear_num_key_heads=cfg.get("linear_num_key_heads") or 0,
        linear_num_value_heads=cfg.get("linear_num_value_heads") or 0,
        linear_key_head_dim=cfg.get("linear_key_head_dim") or 0,
        linear_value_head_dim=cfg.get("linear_value_head_dim") or 0,
        linear_conv_kernel_dim=cfg.get("linear_conv_kernel_dim") or 0,
        full_attention_interval=cfg.get("full_attention_interval") or 0,
        quant_method=q.get("quant_method", "") if isinstance(q, dict) else "",
        weight_block_size=q.get("weight_block_size") if isinstance(q, dict) else None,
        dtype=str(cfg.get("torch_dtype") or cfg.get("dtype") or "bfloat16"),
        raw=cfg,
    )
    if mc.is_mla:
        mc.head_dim = mc.qk_nope_head_dim + mc.qk_rope_head_dim
    if mt == "gpt_oss" and not mc.layer_types:
        mc.layer_types = ["sliding_attention" if i % 2 == 0 else "full_attention"
                          for i in range(mc.num_hidden_layers)]
    return mc


def load_config(model_path: str) -> ModelConfig:
    with open(os.path.join(model_path, "config.json")) as f:
        return config_from_hf(json.load(f))


# ------------------------------------------------------------------ named shapes
def named_config(name: str) -> ModelConfig:
    """Architectures used by the benchmarks and tests (random-init, no checkpoint)."""
    n = name.lower()
    if n in {"qwen3-0.6b", "qwen3_0.6b"}:
        return config_from_hf(dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=1024,
                                   num_hidden_layers=28, num_attention_heads=16, num_key_value_heads=8,
                                   head_dim=128, intermediate_size=3072, vocab_size=151936,
                                   tie_word_embeddings=True, rope_theta=1e6))
    if n in {"qwen3-8b", "qwen3_8b"}:
        return config_from_hf(dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=4096,
                                   num_hidden_layers=36, num_attention_heads=32, num_key_value_heads=8,
                                   head_dim=128, intermediate_size=12288, vocab_size=151936, rope_theta=1e6))
    if n in {"qwen3-32b", "qwen3_32b"}:
        return config_from_hf(dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=5120,
                                   num_hidden_layers=64, num_attention_heads=64, num_key_value_heads=8,
                                   head_dim=128, intermediate_size=25600, vocab_size=151936, rope_theta=1e6))
    if n in {"qwen3-30b-a3b", "qwen3_30b_a3b"}:
        return config_from_hf(dict(architectures=["Qwen3MoeForCausalLM"], model_type="qwen3_moe",
                                   hidden_size=2048, num_hidden_layers=48, num_attention_heads=32,
                                   num_key_value_heads=4, head_dim=128, intermediate_size=6144,
                                   moe_intermediate_size=768, num_experts=128, num_experts_per_tok=8,
                                   norm_topk_prob=True, vocab_size=151936, rope_theta=1e6))
    if n in {"deepseek-v3", "deepseek_v3", "deepseek-v3.2", "deepseek_v32"}:
        v32 = "2" in n.split("v3")[-1]
        d = dict(architectures=["DeepseekV32ForCausalLM" if v32 else "DeepseekV3ForCausalLM"],
                 model_type="deepseek_v32" if v32 else "deepseek_v3", hidden_size=7168,
                 num_hidden_layers=61, num_attention_heads=128, num_key_value_heads=128,
                 q_lora_rank=1536, kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64,
                 v_head_dim=128, intermediate_size=18432, moe_intermediate_size=2048,
                 n_routed_experts=256, num_experts_per_tok=8, n_shared_experts=1,
                 first_k_dense_replace=3, scoring_func="sigmoid", topk_method="noaux_tc", n_group=8,
                 topk_group=4, routed_scaling_factor=2.5, norm_topk_prob=True, vocab_size=129280,
                 rope_theta=10000.0,
                 quantization_config=dict(quant_method="fp8", weight_block_size=[128, 128]))
        if v32:
            d.update(index_n_heads=64, index_head_dim=128, index_topk=2048)
        return config_from_hf(d)
    if n in {"tiny-mla", "tiny-dsa", "small-mla", "small-dsa"}:
        small = n.startswith("small")   # "small": the widths the sm_100a MLA kernels are built for
        d = dict(architectures=["DeepseekV32ForCausalLM" if n.endswith("dsa") else "DeepseekV3ForCausalLM"],
                 model_type="deepseek_v32" if n.endswith("dsa") else "deepseek_v3",
                 hidden_size=512 if small else 128, num_hidden_layers=3, num_attention_heads=8 if small else 4,
                 num_key_value_heads=8 if small else 4, q_lora_rank=256 if small else 48,
                 kv_lora_rank=512 if small else 32, qk_nope_head_dim=128 if small else 32,
                 qk_rope_head_dim=64 if small else 16, v_head_dim=128 if small else 32,
                 intermediate_size=1024 if small else 256, moe_intermediate_size=256 if small else 64,
                 n_routed_experts=8, num_experts_per_tok=2, n_shared_experts=1, first_k_dense_replace=1,
                 scoring_func="sigmoid", topk_method="noaux_tc", n_group=2, topk_group=1, routed_scaling_factor=2.5,
                 norm_topk_prob=True, vocab_size=1024, rope_theta=10000.0, max_position_embeddings=4096)
        if n.endswith("dsa"):
            d.update(index_n_heads=8 if small else 4, index_head_dim=128 if small else 32,
                     index_topk=64 if small else 16)
        return config_from_hf(d)
    if n in {"tiny-hybrid", "small-hybrid"}:
        small = n.startswith("small")   # "small": the head sizes the sm_100a kernels are built for
        hd = 128 if small else 32
        return config_from_hf(dict(architectures=["Qwen3NextForCausalLM"], model_type="qwen3_next",
                                   hidden_size=512 if small else 128, num_hidden_layers=4, num_attention_heads=4,
                                   num_key_value_heads=2, head_dim=hd, intermediate_size=1024 if small else 256,
                                   vocab_size=1024, rope_theta=1e4, partial_rotary_factor=0.25,
                                   full_attention_interval=2, linear_num_key_heads=2, linear_num_value_heads=4,
                                   linear_key_head_dim=hd, linear_value_head_dim=hd, linear_conv_kernel_dim=4,
                                   num_experts=0, max_position_embeddings=4096))
    if n in {"tiny-msa", "small-msa"}:
        small = n.startswith("small")
        hd = 128 if small else 32
        sparse = dict(use_sparse_attention=True, sparse_attention_freq=[0, 1, 1], sparse_block_size=32 if not small else 128,
                      sparse_topk_blocks=2 if not small else 3, sparse_init_block=1, sparse_local_block=1,
                      sparse_index_dim=hd, sparse_num_index_heads=2)
        return config_from_hf(dict(architectures=["MiniMaxM3SparseForCausalLM"], model_type="minimax_m3",
                                   hidden_size=512 if small else 128, num_hidden_layers=3, num_attention_heads=4,
                                   num_key_value_heads=2, head_dim=hd, intermediate_size=1024 if small else 256,
                                   vocab_size=1024, rope_theta=1e4, rotary_dim=hd // 2, use_qk_norm=True,
                                   use_gemma_norm=True, sparse_attention_config=sparse,
                                   index_head_dim=hd, index_block_size=sparse["sparse_block_size"],
                                   index_topk_blocks=sparse["sparse_topk_blocks"], index_local_blocks=1,
                                   max_position_embeddings=4096))
    if n == "tiny":
        return config_from_hf(dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=256,
                                   num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2,
                                   head_dim=64, intermediate_size=512, vocab_size=1024,
                                   tie_word_embeddings=True, rope_theta=1e4))
    if n == "tiny-moe":
        return config_from_hf(dict(architectures=["Qwen3MoeForCausalLM"], model_type="qwen3_moe",
                                   hidden_size=256, num_hidden_layers=4, num_attention_heads=4,
                                   num_key_value_heads=2, head_dim=64, intermediate_size=512,
                                   moe_intermediate_size=128, num_experts=8, num_experts_per_tok=2,
                                   norm_topk_prob=True, vocab_size=1024, rope_theta=1e4))
    raise KeyError(f"unknown named config {name!r}")
